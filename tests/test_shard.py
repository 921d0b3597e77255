"""Host-side partitioning of the path over GPUs, and the one exchange it has (the gather of
KV-length partials), run as two gloo ranks on CPU with the oracle standing in for the kernels."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT, assert_close


def test_plan_single_sequence(q27):
    from qwen27_engine_b200 import shard
    for world in (1, 2, 4):
        heads = []
        for r in range(world):
            s = shard.plan_single_sequence(r, world, 4)
            assert s.nz == 1 and s.z == 0 and s.peers == (r,)
            heads += list(range(s.kv_head0, s.kv_head0 + s.n_kv_heads))
        assert heads == [0, 1, 2, 3]
    seen = set()
    for r in range(8):
        s = shard.plan_single_sequence(r, 8, 4)
        assert s.n_kv_heads == 1 and s.nz == 2 and r in s.peers and len(s.peers) == 2
        seen.add((s.kv_head0, s.z))
    assert seen == {(h, z) for h in range(4) for z in range(2)}
    with pytest.raises(ValueError):
        shard.plan_single_sequence(0, 3, 4)


def test_kv_slices_cover_and_align(q27):
    from qwen27_engine_b200 import shard
    for n in (1, 63, 64, 65, 1000, 150000):
        for nz in (1, 2, 4):
            cuts = [shard.kv_slice(n, z, nz) for z in range(nz)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            for (a, b), (c, d) in zip(cuts, cuts[1:]):
                assert b == c and (b % 64 == 0 or b == n)


def test_shard_sequences_balance(q27):
    from qwen27_engine_b200 import shard, synth
    lens = synth.integers(synth.SEED_LEN, 1024, 131072, 64)
    for world in (1, 2, 4, 8):
        parts = shard.shard_sequences(lens, world)
        assert sorted(sum(parts, [])) == list(range(64))
        loads = [int(sum(lens[i] for i in p)) for p in parts]
        assert max(loads) - min(loads) <= int(lens.max())


def test_plan_prefill_covers_every_token_once_and_balances(q27):
    from qwen27_engine_b200 import shard
    for M, pos0 in [(2048, 0), (2048, 32768), (2048, 148000), (300, 0), (100, 5), (129, 0), (1, 0)]:
        for world in (1, 2, 4, 8, 16):
            seen = {}
            cost = {}
            for r in range(world):
                s = shard.plan_prefill(r, world, M, pos0, 4)
                for a, b in s.ranges:
                    assert 0 <= a < b <= M and (a % 128 == 0) and (b % 128 == 0 or b == M)
                    for h in range(s.kv_head0, s.kv_head0 + s.n_kv_heads):
                        for t in range(a, b, 64):
                            assert (h, t) not in seen
                            seen[(h, t)] = r
                cost[r] = sum((b - a) * (2 * pos0 + a + b + 1) / 2 for a, b in s.ranges) * s.n_kv_heads
            assert len(seen) == 4 * len(range(0, M, 64))
            if M == 2048:  # an early and a late block per slice: close to each other (whole 128-token tiles)
                assert max(cost.values()) <= (1.1 if world <= 8 else 1.25) * min(cost.values())
    with pytest.raises(ValueError):
        shard.plan_prefill(0, 3, 2048)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as ge
    ge.load_package()
    import oracle
    from qwen27_engine_b200 import shard, synth
    # one KV head group split by KV length over the two ranks (the 8-GPU layout with nkvh = 1)
    T, nkvh, nqh, n, n_ctx = 4, 1, 6, 700, 704
    qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n)
    sh = shard.plan_single_sequence(rank, world, nkvh)
    assert sh.nz == 2
    lo, hi = shard.kv_slice(n, sh.z, sh.nz)
    # each rank holds only its slice, as local rows 0 .. hi-lo-1
    kc, vc = oracle.fill_cache(kf[:, lo:hi], vf[:, lo:hi], n_ctx)
    full_k, full_v = oracle.fill_cache(kf, vf, n_ctx)
    part = oracle.attn_partial(qn, full_k, full_v, n - T, 1 / 16, nkvh, n_ctx, lo, hi)
    g = shard.peer_group(sh)
    allp = shard.gather_partials(torch.from_numpy(part.reshape(T * nqh, 258)), sh, g)
    merged = oracle.lse_merge(allp.numpy().reshape(2, T, nqh, 258), qg)
    whole = oracle.attn_ref(qn, qg, full_k, full_v, n - T, 1 / 16, nkvh, n_ctx)
    np.save(os.path.join(out_dir, "r%d.npy" % rank), np.stack([merged, whole]))
    dist.barrier()
    dist.destroy_process_group()


def test_kv_length_split_over_two_gloo_ranks(q27, tmp_path):
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a = np.load(tmp_path / "r0.npy")
    b = np.load(tmp_path / "r1.npy")
    assert np.array_equal(a[0], b[0])  # both ranks end with the same merged output
    assert_close(a[0], a[1], "2-rank merge", abs_tol=2e-4, rel_tol=2e-3)


def _prefill_rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as ge
    ge.load_package()
    import oracle
    from qwen27_engine_b200 import shard, synth
    # one chunk over two ranks that share ONE KV head (the 8-GPU layout with nkvh = 1): query-token ranges
    pos0, M, nkvh, nqh = 300, 400, 1, 6
    n, n_ctx = pos0 + M, pos0 + M + 8
    qn = synth.normal(synth.SEED_Q, (M, nqh, 256))
    qg = np.zeros((M, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (M, nqh, 256))
    kc, vc = oracle.fill_cache(synth.normal(synth.SEED_K, (nkvh, n, 256)), synth.normal(synth.SEED_V, (nkvh, n, 256)), n_ctx)
    plan = shard.plan_prefill(rank, world, M, pos0, nkvh)
    assert plan.n_kv_heads == 1 and plan.kv_head0 == 0
    mine = np.zeros((M, nqh, 256), np.float32)
    mask = np.zeros((M,), np.float32)
    for a, b in plan.ranges:  # one attn_prefill call per range at pos0 + a, the oracle standing in for the kernel
        mine[a:b] = oracle.attn_prefill_i8(qn[a:b], qg[a:b], kc, vc, pos0 + a, 1 / 16, nkvh, n_ctx)
        mask[a:b] = 1
    o = torch.from_numpy(mine)
    m = torch.from_numpy(mask)
    dist.all_reduce(o)   # disjoint slices: the sum is the concatenation
    dist.all_reduce(m)
    if rank == 0:
        whole = oracle.attn_prefill_i8(qn, qg, kc, vc, pos0, 1 / 16, nkvh, n_ctx)
        np.save(os.path.join(out_dir, "pf.npy"), np.stack([o.numpy(), whole]))
        np.save(os.path.join(out_dir, "mask.npy"), m.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_prefill_query_ranges_over_two_gloo_ranks(q27, tmp_path):
    """plan_prefill's query-token ranges on two ranks: every token computed exactly once, and a range
    computed as its own call at pos0 + a gives the rows of the whole-chunk call bit for bit."""
    port = _free_port()
    mp.spawn(_prefill_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got, whole = np.load(tmp_path / "pf.npy")
    assert np.array_equal(np.load(tmp_path / "mask.npy"), np.ones(400, np.float32))
    assert np.array_equal(got, whole)


class _FakeLib:
    """Stands in for the library in the set-up of the exchange buffers: 'device addresses' are small
    integers, a handle is the address plus an offset, rank `bad` fails where told to."""

    def __init__(self, rank, bad=None, where=None):
        self.rank, self.bad, self.where = rank, bad, where

    def _maybe(self, where):
        if self.rank == self.bad and self.where == where:
            raise RuntimeError("injected failure in %s on rank %d" % (where, self.rank))

    def sum_xbuf_bytes(self, world, rows, n):
        return 256 + 2 * world * rows * n * 4

    def xbuf_alloc_bytes(self, nbytes):
        self._maybe("alloc")
        return 1000 + self.rank

    def ipc_export(self, ptr):
        self._maybe("export")
        return ptr + 100000

    def ipc_open(self, handle):
        self._maybe("open")
        return handle - 100000 + 50  # the peer's buffer as mapped here


def _exchange_rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as ge
    ge.load_package()
    from qwen27_engine_b200 import shard
    res = []
    own, peers = shard.make_sum_exchange(_FakeLib(rank), rank, world, 4, 5120)
    res.append(("ok", own, peers))
    for where in ("alloc", "export", "open"):  # one rank fails: every rank raises, nobody is left in a collective
        try:
            shard.make_sum_exchange(_FakeLib(rank, bad=1, where=where), rank, world, 4, 5120)
            res.append(("no error", where))
        except RuntimeError as e:
            res.append(("raised", where, str(e)))
    dist.barrier()
    with open(os.path.join(out_dir, "x%d.txt" % rank), "w") as f:
        f.write(repr(res))
    dist.destroy_process_group()


def test_exchange_set_up_agrees_on_failures_over_two_gloo_ranks(q27, tmp_path):
    port = _free_port()
    mp.spawn(_exchange_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = eval((tmp_path / "x0.txt").read_text())
    r1 = eval((tmp_path / "x1.txt").read_text())
    assert r0[0] == ("ok", 1000, [1000, 1051]) and r1[0] == ("ok", 1001, [1050, 1001])  # own buffer as is, the peer's as mapped
    for a, b in zip(r0[1:], r1[1:]):
        assert a[0] == "raised" and b[0] == "raised" and a[1] == b[1]
        assert "injected failure" in a[2] and "rank 1" in a[2] and a[2] == b[2]


def test_c_abi_plans_agree_with_the_python_plans(q27):
    """q27b_plan_single_sequence / q27b_kv_slice / q27b_plan_prefill (host arithmetic behind the C ABI, for C++
    hosts) give what shard.py gives."""
    import ctypes
    from qwen27_engine_b200 import shard
    lib = ctypes.CDLL(q27.LIB_PATH)
    i = ctypes.c_int
    for world in (1, 2, 4, 8, 16):
        for rank in range(world):
            h0, nh, z, nz = i(), i(), i(), i()
            assert lib.q27b_plan_single_sequence(rank, world, 4, ctypes.byref(h0), ctypes.byref(nh), ctypes.byref(z), ctypes.byref(nz)) == 0
            s = shard.plan_single_sequence(rank, world, 4)
            assert (h0.value, nh.value, z.value, nz.value) == (s.kv_head0, s.n_kv_heads, s.z, s.nz)
            for n in (0, 1, 63, 64, 1000, 150000):
                lo, hi = i(), i()
                assert lib.q27b_kv_slice(n, s.z, s.nz, ctypes.byref(lo), ctypes.byref(hi)) == 0
                assert (lo.value, hi.value) == shard.kv_slice(n, s.z, s.nz)
            for M, pos0 in ((2048, 0), (2048, 32768), (300, 700), (128, 5), (1, 0), (2047, 148000)):
                rng = (i * 4)()
                nr = i()
                assert lib.q27b_plan_prefill(rank, world, M, pos0, 4, ctypes.byref(h0), ctypes.byref(nh), rng, ctypes.byref(nr)) == 0
                p = shard.plan_prefill(rank, world, M, pos0, 4)
                assert (h0.value, nh.value) == (p.kv_head0, p.n_kv_heads)
                assert tuple((rng[2 * k], rng[2 * k + 1]) for k in range(nr.value)) == tuple(p.ranges), (world, rank, M, pos0)
    assert lib.q27b_plan_single_sequence(0, 3, 4, ctypes.byref(i()), ctypes.byref(i()), ctypes.byref(i()), ctypes.byref(i())) == q27.BAD_SHAPE
