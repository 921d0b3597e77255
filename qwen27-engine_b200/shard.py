"""Partitioning of the attention path over the GPUs of one box, one process per GPU.

The reference shards attention by KV head only (2 KV heads + their 12 query heads per card,
src/model.cu:161-164) and never exchanges anything inside attention. The same split is used here
up to 4 GPUs; beyond that one sequence is also split by KV length, and the only exchange of the
path appears: each rank's (m, l, O) partial of 6*T rows (24.8 KB at T = 4) is all-gathered among
the ranks that share a head group and merged by the log-sum-exp kernel. Batched decode shards whole
sequences, with no exchange. The collective is torch.distributed (NCCL on GPUs, gloo in CPU tests).
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist

TILE = 64


@dataclass
class SeqShard:
    rank: int
    world: int
    kv_head0: int     # first KV head of this rank
    n_kv_heads: int   # KV heads of this rank
    z: int            # index of this rank's KV-length slice
    nz: int           # KV-length slices per head group
    peers: tuple      # ranks holding the other slices of the same heads (including this rank), by z


def plan_single_sequence(rank, world, nkvh=4):
    """KV-head groups first, then KV-length slices once there are more ranks than KV heads."""
    if world < 1 or rank < 0 or rank >= world:
        raise ValueError("bad rank/world")
    if world <= nkvh:
        if nkvh % world:
            raise ValueError("world must divide the KV heads")
        per = nkvh // world
        return SeqShard(rank, world, rank * per, per, 0, 1, (rank,))
    if world % nkvh:
        raise ValueError("world must be a multiple of the KV heads")
    nz = world // nkvh
    hg, z = rank // nz, rank % nz
    return SeqShard(rank, world, hg, 1, z, nz, tuple(hg * nz + i for i in range(nz)))


def kv_slice(n, z, nz):
    """Positions [lo, hi) of KV-length slice z of nz; boundaries are multiples of the 64-position tile."""
    per = -(-n // nz)
    per = -(-per // TILE) * TILE
    lo = min(n, z * per)
    return lo, min(n, lo + per)


def shard_sequences(lengths, world):
    """Greedy longest-first assignment of sequences to ranks, balanced by KV length.
    Returns a list of index lists, one per rank."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world
    out = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(x) for x in out]


@dataclass
class PrefillShard:
    rank: int
    world: int
    kv_head0: int     # first KV head of this rank
    n_kv_heads: int   # KV heads of this rank
    ranges: tuple     # query-token ranges [a, b) of the chunk this rank computes, ascending


Q_TILE = 128


def plan_prefill(rank, world, M, pos0=0, nkvh=4):
    """One prefill chunk of M tokens over the ranks: KV-head groups first (the reference's split,
    src/model.cu:161-164), then query-token ranges within a head group. Every rank of a head group
    holds the group's K and V rows, so nothing is exchanged: outputs are disjoint [token][head]
    slices. A token's cost grows with its position (causal), so the chunk is cut into 2 * nq blocks
    of equal cost area and slice s takes blocks s and 2 nq - 1 - s (an early one and a late one);
    block boundaries are multiples of the kernel's 128-token query tile. Each range is one
    attn_prefill call at pos0 + a."""
    if world < 1 or rank < 0 or rank >= world or M < 1:
        raise ValueError("bad rank/world/M")
    if world <= nkvh:
        if nkvh % world:
            raise ValueError("world must divide the KV heads")
        per = nkvh // world
        return PrefillShard(rank, world, rank * per, per, ((0, M),))
    if world % nkvh:
        raise ValueError("world must be a multiple of the KV heads")
    nq = world // nkvh
    hg, s = rank // nq, rank % nq
    tiles = -(-M // Q_TILE)
    nb = 2 * nq
    # cost of tile i ~ positions it attends: pos0 + (i + 1) * Q_TILE; cuts at equal cumulative cost
    cost = [pos0 + min(M, (i + 1) * Q_TILE) for i in range(tiles)]
    total = float(sum(cost))
    cuts, acc, k = [0], 0.0, 1
    for i, c in enumerate(cost):
        acc += c
        while k < nb and acc >= total * k / nb - 1e-9:
            cuts.append(i + 1)
            k += 1
    while len(cuts) < nb + 1:
        cuts.append(tiles)
    cuts[nb] = tiles
    blocks = [(min(M, cuts[b] * Q_TILE), min(M, cuts[b + 1] * Q_TILE)) for b in range(nb)]
    mine = sorted([blocks[s], blocks[nb - 1 - s]])
    out = []
    for a, b in mine:
        if b <= a:
            continue
        if out and out[-1][1] == a:
            out[-1] = (out[-1][0], b)
        else:
            out.append((a, b))
    return PrefillShard(rank, world, hg, 1, tuple(out))


_groups = {}


def peer_group(shard):
    """Process group of the ranks that share this rank's KV heads. Every rank must call this
    (new_group is collective over the default group)."""
    if shard.nz == 1:
        return None
    key = (shard.world, shard.nz)
    if key not in _groups:
        nkvh_groups = shard.world // shard.nz
        gs = [dist.new_group([g * shard.nz + i for i in range(shard.nz)]) for g in range(nkvh_groups)]
        _groups[key] = gs
    return _groups[key][shard.rank // shard.nz]


def gather_partials(part, shard, group=None):
    """part [rows][258] of this rank -> [nz][rows][258] holding every KV-length slice of the head
    group, in slice order. The result lives in this rank's own memory before anything reads it."""
    if shard.nz == 1:
        return part.unsqueeze(0)
    out = torch.empty((shard.nz,) + tuple(part.shape), dtype=part.dtype, device=part.device)
    if part.is_cuda:
        dist.all_gather_into_tensor(out, part.contiguous(), group=group)
    else:
        lst = [out[i] for i in range(shard.nz)]
        dist.all_gather(lst, part.contiguous(), group=group)
    return out



def make_exchange(q, shard, group, rows):
    """Exchange buffers for the peer-memory merge of a KV-length split (q27b_attn_decode_partial_push /
    q27b_lse_merge_wait), one process per GPU: every rank of the head group allocates one, sends its
    CUDA IPC handle to the group and maps the peers' handles with ITS OWN device current. Returns
    (address of the own buffer, [address of rank k's buffer as seen from this GPU, k in group order]).
    If any rank of the group fails, every rank raises (the ranks agree before they return)."""
    return _exchange_buffers(q, lambda: q.xbuf_alloc(shard.nz, rows), shard.z, shard.nz, group)


def make_sum_exchange(q, rank, world, rows, n, group=None):
    """The same for the sum over all ranks that follows the attention output projection
    (q27b_sum_push / q27b_sum_norm_q8_wait): one buffer per rank for `rows` rows of n floats from each of
    `world` ranks. Returns (own address, [addresses in rank order as seen from this GPU])."""
    return _exchange_buffers(q, lambda: q.xbuf_alloc_bytes(q.sum_xbuf_bytes(world, rows, n)), rank, world, group)


_PEER_FAILED = "a peer could not export its buffer"


def _exchange_buffers(q, alloc, me, count, group):
    err, own, peers = None, 0, []
    try:
        own = alloc()
        mine = q.ipc_export(own)
    except Exception as e:  # still take part in the collectives below
        err, mine = str(e), None
    handles = [None] * count
    dist.all_gather_object(handles, mine, group=group)
    if err is None and all(h is not None for h in handles):
        try:
            peers = [own if k == me else q.ipc_open(h) for k, h in enumerate(handles)]
        except Exception as e:
            err = str(e)
    elif err is None:
        err = _PEER_FAILED
    errs = [None] * count
    dist.all_gather_object(errs, err, group=group)
    bad = [e for e in errs if e]
    if bad:  # every rank reports the same cause: the failing rank's own message where there is one
        own_msgs = [e for e in bad if e != _PEER_FAILED]
        raise RuntimeError("peer-memory exchange not available: " + (own_msgs or bad)[0])
    return own, peers
