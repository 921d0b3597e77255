"""Host-side mirror of the reference's attention operators over the q27b_attn C ABI.

The functions carry the names, argument order and error behaviour of the reference's operator
layer (namespace q27, src/ops.h:50-77: kv_cache_bytes, attn_prep, attn_decode, attn_prefill,
attn_chunks), so that a test written against the reference reads the same here. Arguments are
torch CUDA tensors (torch is used for device memory and streams only); every call forwards the
raw device pointers to libq27b_attn.so and raises RuntimeError where the reference throws
std::runtime_error. There is no CPU path: if the library cannot be loaded the import fails.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# Q27B_LIB: path of another build of the same library (kernel tuning experiments)
LIB_PATH = os.environ.get("Q27B_LIB") or os.path.join(_HERE, "libq27b_attn.so")

HEAD_DIM = 256
GQA = 6
MAX_T = 4
PART_ROW = 258
PAGE = 256

OK, BAD_SHAPE, CUDA_ERROR, UNSUPPORTED, DEVICE_STATUS = 0, 1, 2, 3, 4

# Every symbol that include/q27b_attn.h declares.
SYMBOLS = [
    "q27b_last_error", "q27b_device_status", "q27b_kv_cache_bytes", "q27b_attn_chunks", "q27b_kv_append",
    "q27b_attn_prep", "q27b_attn_decode", "q27b_attn_decode_partial", "q27b_lse_merge", "q27b_attn_decode_paged",
    "q27b_kv_pool_bytes", "q27b_attn_prefill", "q27b_prefill_qk_debug", "q27b_debug_split_event", "q27b_debug_split_events", "q27b_debug_split_only", "q27b_debug_decode_trace", "q27b_set_decode_kernel", "q27b_set_decode_schedule", "q27b_set_prefill_kernel", "q27b_prefill_split_plan", "q27b_sum_xbuf_bytes", "q27b_xbuf_alloc_bytes",
    "q27b_sum_norm_q8", "q27b_sum_push", "q27b_sum_norm_q8_wait", "q27b_debug_expire_wait",
    "q27b_attn_prefill_q8_1", "q27b_xbuf_bytes", "q27b_attn_decode_partial_push", "q27b_lse_merge_wait",
    "q27b_xbuf_alloc", "q27b_xbuf_free", "q27b_ipc_export", "q27b_ipc_open", "q27b_ipc_close",
    "q27b_kv_wire_bytes", "q27b_kv_pages_to_wire", "q27b_kv_wire_to_pages", "q27b_kv_cache_to_wire", "q27b_kv_wire_to_cache",
    "q27b_attn_decode_noalloc", "q27b_attn_decode_ref", "q27b_attn_workspace_query", "q27b_attn_workspace_init",
    "q27b_attn_workspace_destroy", "q27b_debug_mma_peak", "q27b_xbuf_reset", "q27b_plan_single_sequence", "q27b_kv_slice", "q27b_plan_prefill",
    "q27b_attn_prep_paged", "q27b_pager_create", "q27b_pager_destroy", "q27b_pager_open", "q27b_pager_extend",
    "q27b_pager_cut", "q27b_pager_close", "q27b_pager_fork", "q27b_pager_free_pages", "q27b_pager_len",
    "q27b_pager_tables", "q27b_kv_page_copy", "q27b_pager_unshare", "q27b_attn_decode_exchange", "q27b_sum_exchange_norm_q8",
]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libq27b_attn.so is not built (run `python qwen27-engine_b200/build.py`); there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    lib.q27b_last_error.restype = ctypes.c_char_p
    lib.q27b_kv_cache_bytes.restype = ctypes.c_uint64
    lib.q27b_kv_pool_bytes.restype = ctypes.c_uint64
    lib.q27b_kv_wire_bytes.restype = ctypes.c_uint64
    lib.q27b_xbuf_bytes.restype = ctypes.c_uint64
    lib.q27b_sum_xbuf_bytes.restype = ctypes.c_uint64
    lib.q27b_pager_destroy.restype = None
    lib.q27b_pager_destroy.argtypes = [ctypes.c_void_p]
    return lib


_lib = _load()


class Q27Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("q27b_attn error %d: %s" % (code, msg))
        self.code = code


def _check(rc):
    if rc != 0:
        raise Q27Error(rc, _lib.q27b_last_error().decode())


def _ptr(t, dtype=None, optional=False):
    if isinstance(t, int):  # a raw device address (exchange buffers mapped from other processes)
        return ctypes.c_void_p(t)
    if t is None:
        if not optional:
            raise Q27Error(BAD_SHAPE, "null tensor")
        return ctypes.c_void_p(0)
    if not t.is_cuda or not t.is_contiguous():
        raise Q27Error(BAD_SHAPE, "tensors must be contiguous CUDA tensors")
    if dtype is not None and t.dtype != dtype:
        raise Q27Error(BAD_SHAPE, "expected dtype %s, got %s" % (dtype, t.dtype))
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f(x):
    return ctypes.c_float(x)


def kv_cache_bytes(nkvh, n_ctx, q8=True):
    """q27::kv_cache_bytes (src/ops.h:53)."""
    return int(_lib.q27b_kv_cache_bytes(int(nkvh), int(n_ctx), int(bool(q8))))


def kv_pool_bytes(nkvh, n_pages):
    return int(_lib.q27b_kv_pool_bytes(int(nkvh), int(n_pages)))


def kv_wire_bytes(nkvh, n_rows):
    """Bytes of rows [p0, p1) of one q8_0 cache in the reference's host layout (src/model.cu:1809-1830)."""
    return int(_lib.q27b_kv_wire_bytes(int(nkvh), int(n_rows)))


def kv_pages_to_wire(pool, pages, wire, nkvh, n_pages, p0, p1):
    """Rows [p0, p1) of one sequence of the page pool -> device buffer in the reference's host layout."""
    _check(_lib.q27b_kv_pages_to_wire(_ptr(pool), _ptr(pages, torch.int32), _ptr(wire), int(nkvh), int(n_pages),
                                      int(p0), int(p1), _stream()))


def kv_wire_to_pages(pool, pages, wire, nkvh, n_pages, p0, p1):
    _check(_lib.q27b_kv_wire_to_pages(_ptr(pool), _ptr(pages, torch.int32), _ptr(wire), int(nkvh), int(n_pages),
                                      int(p0), int(p1), _stream()))


def kv_cache_to_wire(cache, wire, nkvh, n_ctx, p0, p1):
    """Rows [p0, p1) of a contiguous cache -> the reference's host layout (Decoder::kv_copy)."""
    _check(_lib.q27b_kv_cache_to_wire(_ptr(cache), _ptr(wire), int(nkvh), int(n_ctx), int(p0), int(p1), _stream()))


def kv_wire_to_cache(cache, wire, nkvh, n_ctx, p0, p1):
    _check(_lib.q27b_kv_wire_to_cache(_ptr(cache), _ptr(wire), int(nkvh), int(n_ctx), int(p0), int(p1), _stream()))


def attn_chunks(nkvh):
    """q27::attn_chunks (src/ops.h:77)."""
    return int(_lib.q27b_attn_chunks(int(nkvh)))


def device_status():
    """Synchronises the device; returns the status word (0 = fine) and clears it."""
    st = ctypes.c_int(0)
    rc = _lib.q27b_device_status(ctypes.byref(st))
    if rc not in (OK, DEVICE_STATUS):
        _check(rc)
    return st.value


def debug_expire_wait():
    """Test hook: one warp waits on a barrier nobody arrives at; the bounded wait gives up (status bit 0)."""
    _check(_lib.q27b_debug_expire_wait(_stream()))


def xbuf_bytes(nz, rows):
    """Bytes of one rank's exchange buffer for the peer-memory merge of nz KV-length slices."""
    return int(_lib.q27b_xbuf_bytes(int(nz), ctypes.c_int64(int(rows))))


def xbuf_alloc(nz, rows):
    """Device address of a new zeroed exchange buffer (an allocation of its own, exportable over CUDA IPC)."""
    out = ctypes.c_void_p(0)
    _check(_lib.q27b_xbuf_alloc(int(nz), ctypes.c_int64(int(rows)), ctypes.byref(out)))
    return int(out.value)


def xbuf_free(ptr):
    _check(_lib.q27b_xbuf_free(ctypes.c_void_p(int(ptr))))


def ipc_export(ptr):
    """The 64-byte CUDA IPC handle of an allocation."""
    h = (ctypes.c_ubyte * 64)()
    _check(_lib.q27b_ipc_export(ctypes.c_void_p(int(ptr)), h))
    return bytes(h)


def ipc_open(handle):
    """Maps a peer's allocation into the current device's address space; returns the device address."""
    h = (ctypes.c_ubyte * 64).from_buffer_copy(handle)
    out = ctypes.c_void_p(0)
    _check(_lib.q27b_ipc_open(h, ctypes.byref(out)))
    return int(out.value)


def ipc_close(ptr):
    _check(_lib.q27b_ipc_close(ctypes.c_void_p(int(ptr))))


def attn_decode_partial_push(qn, kcache, vcache, pos0, T, kq_scale, nqh, nkvh, n_ctx, base_pos, n_local, peer_ptrs,
                             my_z, q8=True):
    """Split-K decode of one KV-length slice whose merged partial is stored into slot my_z of the
    exchange buffers of all ranks of the group (peer_ptrs: their device addresses as seen from here)."""
    arr = (ctypes.c_void_p * len(peer_ptrs))(*[ctypes.c_void_p(int(x)) for x in peer_ptrs])
    _check(_lib.q27b_attn_decode_partial_push(_ptr(qn, torch.float32), _ptr(kcache), _ptr(vcache), _ptr(pos0, torch.int32),
                                              int(T), _f(kq_scale), int(nqh), int(nkvh), int(n_ctx), int(bool(q8)),
                                              int(base_pos), int(n_local), arr, int(my_z), len(peer_ptrs), _stream()))


def lse_merge_wait(xbuf, nz, rows, qg, o):
    """Waits for the nz slices of this step in this rank's exchange buffer, merges them, applies the gate."""
    _check(_lib.q27b_lse_merge_wait(_ptr(xbuf), int(nz), ctypes.c_int64(int(rows)),
                                    _ptr(qg, torch.float32) if qg is not None else None, _ptr(o, torch.float32), _stream()))


def sum_xbuf_bytes(world, rows, n):
    return int(_lib.q27b_sum_xbuf_bytes(int(world), int(rows), int(n)))


def xbuf_alloc_bytes(nbytes):
    """Device address of a new zeroed exchange buffer of nbytes (an allocation of its own, exportable over CUDA IPC)."""
    out = ctypes.c_void_p(0)
    _check(_lib.q27b_xbuf_alloc_bytes(ctypes.c_uint64(int(nbytes)), ctypes.byref(out)))
    return int(out.value)


def sum_norm_q8(x, partial, n, rows, w, eps, h=None, xq=None, xd=None):
    """q27::sum_norm_q8 without an exchange (src/ops.h:101-104): x += partial, RMSNorm(x) * w -> h and q8_1."""
    _check(_lib.q27b_sum_norm_q8(_ptr(x, torch.float32), _ptr(partial, torch.float32), int(n), int(rows), _ptr(w, torch.float32),
                                 _f(eps), _ptr(h, torch.float32) if h is not None else None,
                                 _ptr(xq, torch.int8) if xq is not None else None,
                                 _ptr(xd, torch.float32) if xd is not None else None, _stream()))


def sum_push(partial, n, rows, rank, xbufs):
    """Stores this rank's partial rows into slot `rank` of the exchange buffers of all ranks (xbufs: their
    device addresses as seen from here, in rank order, this rank's own at index rank)."""
    arr = (ctypes.c_void_p * len(xbufs))(*[ctypes.c_void_p(int(x)) for x in xbufs])
    _check(_lib.q27b_sum_push(_ptr(partial, torch.float32), int(n), int(rows), int(rank), len(xbufs), arr, _stream()))


def sum_norm_q8_wait(x, xbuf, world, n, rows, w, eps, h=None, xq=None, xd=None):
    """Waits for the partial rows of all ranks of this step, x += their sum in rank order, RMSNorm -> h and q8_1."""
    _check(_lib.q27b_sum_norm_q8_wait(_ptr(x, torch.float32), _ptr(xbuf), int(world), int(n), int(rows), _ptr(w, torch.float32),
                                      _f(eps), _ptr(h, torch.float32) if h is not None else None,
                                      _ptr(xq, torch.int8) if xq is not None else None,
                                      _ptr(xd, torch.float32) if xd is not None else None, _stream()))


def sum_exchange_norm_q8(x, partial, n, rows, rank, xbufs, w, eps, h=None, xq=None, xd=None):
    """sum_push + sum_norm_q8_wait as one kernel (xbufs: the exchange buffers of all ranks as mapped here)."""
    arr = (ctypes.c_void_p * len(xbufs))(*[ctypes.c_void_p(int(b) if isinstance(b, int) else b.data_ptr()) for b in xbufs])
    _check(_lib.q27b_sum_exchange_norm_q8(_ptr(x, torch.float32), _ptr(partial, torch.float32), int(n), int(rows), int(rank),
                                          len(xbufs), arr, _ptr(w, torch.float32), _f(eps),
                                          _ptr(h, torch.float32) if h is not None else None,
                                          _ptr(xq, torch.int8) if xq is not None else None,
                                          _ptr(xd, torch.float32) if xd is not None else None, _stream()))


def set_decode_kernel(which):
    """0 default (= 3), 1 single-role warp-MMA kernel, 2 tcgen05 kernel, 3 warp-specialised kernel (q8_0 caches; see include/q27b_attn.h)."""
    _check(_lib.q27b_set_decode_kernel(int(which)))


def prefill_split_plan(M, nqh, n_sm, depth_hint):
    """(split_tiles, pieces) of an attn_prefill call: the first split_tiles query tiles are cut into
    `pieces` pieces over their positions, the others are not (host arithmetic only)."""
    ts, ns = ctypes.c_int(0), ctypes.c_int(0)
    _check(_lib.q27b_prefill_split_plan(int(M), int(nqh), int(n_sm), int(depth_hint), ctypes.byref(ts), ctypes.byref(ns)))
    return ts.value, ns.value


def set_prefill_kernel(which):
    """0 automatic, 1 int8 Q K^T, 2 f16 Q K^T on dequantised K and V (q8_0 caches; the reference's
    Q27_ATTN_I8 switch, src/attn.cu:933)."""
    _check(_lib.q27b_set_prefill_kernel(int(which)))


def debug_split_event(event):
    """event: a recorded-at-least-once torch.cuda.Event (timing enabled) or None."""
    _check(_lib.q27b_debug_split_event(ctypes.c_void_p(event.cuda_event if event is not None else 0)))


def attn_decode_exchange(qn, qg, kcache, vcache, o, pos0, T, kq_scale, nqh, nkvh, n_ctx, base_pos, n_local, peer_ptrs, my_z,
                         q8=True):
    """attn_decode_partial_push + lse_merge_wait as one call (one kernel after the split-K kernel where the shape allows)."""
    arr = (ctypes.c_void_p * len(peer_ptrs))(*[ctypes.c_void_p(int(x)) for x in peer_ptrs])
    _check(_lib.q27b_attn_decode_exchange(_ptr(qn, torch.float32), _ptr(qg, torch.float32, True), _ptr(kcache), _ptr(vcache),
                                          _ptr(o, torch.float32), _ptr(pos0, torch.int32), int(T), _f(kq_scale), int(nqh),
                                          int(nkvh), int(n_ctx), int(bool(q8)), int(base_pos), int(n_local), arr, int(my_z),
                                          len(peer_ptrs), _stream()))


def attn_decode_ref(qn, qg, kcache, vcache, o, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8=True):
    """q27::attn_decode_ref (src/ops.h:73-75): the simple slow kernel, for checks."""
    _check(_lib.q27b_attn_decode_ref(_ptr(qn, torch.float32), _ptr(qg, torch.float32), _ptr(kcache), _ptr(vcache),
                                     _ptr(o, torch.float32), _ptr(pos0, torch.int32), int(T), _f(kq_scale), int(nqh),
                                     int(nkvh), int(n_ctx), int(bool(q8)), _stream()))


def workspace_query():
    """(decode_bytes, prefill_bytes, paged_bytes, fixed) of the current device's workspace."""
    a, b, c, f = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_int(0)
    _check(_lib.q27b_attn_workspace_query(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(f)))
    return a.value, b.value, c.value, bool(f.value)


def workspace_init(prefill_bytes=0, paged_bytes=0):
    """Allocates the whole workspace now and fixes it: no later call allocates or frees."""
    _check(_lib.q27b_attn_workspace_init(ctypes.c_uint64(int(prefill_bytes)), ctypes.c_uint64(int(paged_bytes))))


def workspace_destroy():
    _check(_lib.q27b_attn_workspace_destroy())


def xbuf_reset(xbuf, nbytes=None):
    """Zeroes an exchange buffer (every rank of the group, after a step that reported status 1); nbytes is
    needed when xbuf is a raw address."""
    if nbytes is None:
        nbytes = xbuf.numel() * xbuf.element_size()
    _check(_lib.q27b_xbuf_reset(_ptr(xbuf), ctypes.c_uint64(int(nbytes)), _stream()))


def debug_mma_peak(kind, iters):
    """Launches the tensor-core peak microbenchmark (kind 0: int8, 1: f16); returns the ops of the launch."""
    ops = ctypes.c_double(0)
    _check(_lib.q27b_debug_mma_peak(int(kind), int(iters), _stream(), ctypes.byref(ops)))
    return ops.value


def set_decode_schedule(pool):
    """True: CTAs share a pool of tiles (default, faster); False: equal static shares (same bits every run)."""
    _check(_lib.q27b_set_decode_schedule(int(bool(pool))))


def debug_decode_trace(stamps):
    """stamps: int64 CUDA tensor of 8 values per CTA of the split-K grid, or None (see the header)."""
    _check(_lib.q27b_debug_decode_trace(_ptr(stamps, torch.int64, optional=True)))


def debug_split_only(on):
    """True: attn_decode launches its split-K kernel only (benchmarks time that kernel alone)."""
    _check(_lib.q27b_debug_split_only(int(bool(on))))


def debug_split_events(begin, end):
    """begin, end: torch.cuda.Event objects (timing enabled, each recorded at least once) or None, None."""
    h = lambda e: ctypes.c_void_p(e.cuda_event if e is not None else 0)
    _check(_lib.q27b_debug_split_events(h(begin), h(end)))


def new_cache(nkvh, n_ctx, q8=True, device="cuda", fill=0):
    """Zero-filled K (or V) cache of one layer, as the reference allocates it (src/model.cu:441-446)."""
    return torch.full((kv_cache_bytes(nkvh, n_ctx, q8),), fill, dtype=torch.uint8, device=device)


def kv_append(k, v, kcache, vcache, pos0, T, nkvh, n_ctx, q8=True):
    """K/V rows [T][nkvh][256] f32 -> cache rows *pos0 + t (the cache-write tail of q27::attn_prep)."""
    _check(_lib.q27b_kv_append(_ptr(k, torch.float32), _ptr(v, torch.float32), _ptr(kcache), _ptr(vcache),
                               _ptr(pos0, torch.int32), int(T), int(nkvh), int(n_ctx), int(bool(q8)), _stream()))


def attn_prep(qg, k, v, q_norm, k_norm, qn, kcache, vcache, pos0, T, eps, theta_scale, nqh, nkvh, n_ctx, q8=True,
              rope3=None, rdelta=None):
    """q27::attn_prep (src/ops.h:59-62)."""
    _check(_lib.q27b_attn_prep(_ptr(qg, torch.float32), _ptr(k, torch.float32), _ptr(v, torch.float32),
                               _ptr(q_norm, torch.float32), _ptr(k_norm, torch.float32), _ptr(qn, torch.float32),
                               _ptr(kcache), _ptr(vcache), _ptr(pos0, torch.int32), int(T), _f(eps), _f(theta_scale),
                               int(nqh), int(nkvh), int(n_ctx), int(bool(q8)), _stream(),
                               _ptr(rope3, torch.int32, True), _ptr(rdelta, torch.int32, True)))


def attn_decode(qn, qg, kcache, vcache, o, xq, xd, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8=True):
    """q27::attn_decode (src/ops.h:66-67). With xq given the result goes to q8_1 (xq, xd) instead of o."""
    _check(_lib.q27b_attn_decode(_ptr(qn, torch.float32), _ptr(qg, torch.float32), _ptr(kcache), _ptr(vcache),
                                 _ptr(o, torch.float32, True), _ptr(xq, torch.int8, True),
                                 _ptr(xd, torch.float32, True), _ptr(pos0, torch.int32), int(T), _f(kq_scale),
                                 int(nqh), int(nkvh), int(n_ctx), int(bool(q8)), _stream()))


def attn_decode_noalloc(qn, qg, kcache, vcache, o, xq, xd, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8=True):
    """attn_decode for hosts that may not allocate device memory (fixed memory budgets, several GPUs
    driven in lock step, runtimes that own the allocator): the split partials live in a 3.96 MB array
    inside the library image instead of a cudaMalloc'ed workspace. Same arguments and result as
    attn_decode; at most 160 chunk partials (nkvh * attn_chunks(nkvh)); calls of one device must not
    overlap on the GPU, and the first one should come before any stream capture."""
    _check(_lib.q27b_attn_decode_noalloc(_ptr(qn, torch.float32), _ptr(qg, torch.float32), _ptr(kcache),
                                         _ptr(vcache), _ptr(o, torch.float32, True), _ptr(xq, torch.int8, True),
                                         _ptr(xd, torch.float32, True), _ptr(pos0, torch.int32), int(T),
                                         _f(kq_scale), int(nqh), int(nkvh), int(n_ctx), int(bool(q8)), _stream()))


def attn_decode_partial(qn, kcache, vcache, part, pos0, T, kq_scale, nqh, nkvh, n_ctx, base_pos, n_local, q8=True):
    """Unnormalised (m, l, O) [T][nqh][258] over the local cache rows of a KV-length shard."""
    _check(_lib.q27b_attn_decode_partial(_ptr(qn, torch.float32), _ptr(kcache), _ptr(vcache),
                                         _ptr(part, torch.float32), _ptr(pos0, torch.int32), int(T), _f(kq_scale),
                                         int(nqh), int(nkvh), int(n_ctx), int(bool(q8)), int(base_pos), int(n_local),
                                         _stream()))


def lse_merge(part, nparts, part_stride, rows, qg, o, xq=None, xd=None):
    """Log-sum-exp merge of partials (attn_combine_kernel / attn_pf_combine_kernel of the reference)."""
    _check(_lib.q27b_lse_merge(_ptr(part, torch.float32), int(nparts), ctypes.c_int64(part_stride),
                               ctypes.c_int64(rows), _ptr(qg, torch.float32, True), _ptr(o, torch.float32, True),
                               _ptr(xq, torch.int8, True), _ptr(xd, torch.float32, True), _stream()))


def attn_decode_paged(qn, qg, kpool, vpool, page_table, seq_len, o, B, T, kq_scale, nqh, nkvh, n_pages, max_pages,
                      max_seq_len):
    """Batched decode over a paged q8_0 cache (256-position pages)."""
    _check(_lib.q27b_attn_decode_paged(_ptr(qn, torch.float32), _ptr(qg, torch.float32), _ptr(kpool), _ptr(vpool),
                                       _ptr(page_table, torch.int32), _ptr(seq_len, torch.int32),
                                       _ptr(o, torch.float32), int(B), int(T), _f(kq_scale), int(nqh), int(nkvh),
                                       int(n_pages), int(max_pages), int(max_seq_len), _stream()))


def attn_prep_paged(qg, k, v, q_norm, k_norm, qn, kpool, vpool, page_table, seq_len, B, T, eps, theta_scale, nqh, nkvh,
                    n_pages, max_pages, rope3=None, rdelta=None):
    """q27::attn_prep for B sequences over the page pool; with q_norm None it only appends K and V."""
    _check(_lib.q27b_attn_prep_paged(_ptr(qg, torch.float32, True), _ptr(k, torch.float32), _ptr(v, torch.float32),
                                     _ptr(q_norm, torch.float32, True), _ptr(k_norm, torch.float32, True),
                                     _ptr(qn, torch.float32, True), _ptr(kpool), _ptr(vpool),
                                     _ptr(page_table, torch.int32), _ptr(seq_len, torch.int32), int(B), int(T),
                                     _f(eps), _f(theta_scale), int(nqh), int(nkvh), int(n_pages), int(max_pages),
                                     _stream(), _ptr(rope3, torch.int32, True), _ptr(rdelta, torch.int32, True)))


def kv_page_copy(pool, src_page, dst_page, rows, nkvh, n_pages):
    """The first `rows` rows of one page into another, all heads, of one pool."""
    _check(_lib.q27b_kv_page_copy(_ptr(pool), int(src_page), int(dst_page), int(rows), int(nkvh), int(n_pages), _stream()))


class Pager:
    """Page bookkeeping of the paged cache (q27b_pager_*): host only, no device memory."""

    def __init__(self, n_pages, max_seqs, max_pages_per_seq):
        self._h = ctypes.c_void_p()
        self.n_pages, self.max_seqs, self.max_pages = int(n_pages), int(max_seqs), int(max_pages_per_seq)
        _check(_lib.q27b_pager_create(self.n_pages, self.max_seqs, self.max_pages, ctypes.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            _lib.q27b_pager_destroy(self._h)
            self._h = None

    def open(self):
        s = ctypes.c_int()
        _check(_lib.q27b_pager_open(self._h, ctypes.byref(s)))
        return s.value

    def extend(self, seq, new_len):
        _check(_lib.q27b_pager_extend(self._h, int(seq), int(new_len)))

    def cut(self, seq, new_len):
        _check(_lib.q27b_pager_cut(self._h, int(seq), int(new_len)))

    def close(self, seq):
        _check(_lib.q27b_pager_close(self._h, int(seq)))

    def fork(self, seq, prefix_len):
        """-> (new sequence, (src page, dst page, rows) to copy in both pools, or None)."""
        s, a, b, r = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        _check(_lib.q27b_pager_fork(self._h, int(seq), int(prefix_len), ctypes.byref(s), ctypes.byref(a), ctypes.byref(b),
                                    ctypes.byref(r)))
        return s.value, ((a.value, b.value, r.value) if r.value else None)

    def unshare(self, seq):
        """Gives the sequence its own copy of a shared, partly filled last page -> (src, dst, rows) to copy, or None."""
        a, b, r = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        _check(_lib.q27b_pager_unshare(self._h, int(seq), ctypes.byref(a), ctypes.byref(b), ctypes.byref(r)))
        return (a.value, b.value, r.value) if r.value else None

    def free_pages(self):
        return int(_lib.q27b_pager_free_pages(self._h))

    def length(self, seq):
        return int(_lib.q27b_pager_len(self._h, int(seq)))

    def tables(self, seqs):
        """-> (page_table int32 [B][max_pages], seq_len int32 [B]) as numpy arrays."""
        import numpy as np
        ids = (ctypes.c_int * len(seqs))(*[int(x) for x in seqs])
        table = np.empty((len(seqs), self.max_pages), np.int32)
        lens = np.empty((len(seqs),), np.int32)
        _check(_lib.q27b_pager_tables(self._h, ids, len(seqs), table.ctypes.data_as(ctypes.c_void_p),
                                      lens.ctypes.data_as(ctypes.c_void_p)))
        return table, lens


def attn_prefill(qn, qg, kcache, vcache, o, pos0, M, kq_scale, nqh, nkvh, n_ctx, q8=True, depth_hint=-1):
    """q27::attn_prefill (src/ops.h:71-72)."""
    _check(_lib.q27b_attn_prefill(_ptr(qn, torch.float32), _ptr(qg, torch.float32), _ptr(kcache), _ptr(vcache),
                                  _ptr(o, torch.float32), _ptr(pos0, torch.int32), int(M), _f(kq_scale), int(nqh),
                                  int(nkvh), int(n_ctx), int(bool(q8)), _stream(), int(depth_hint)))


def attn_prefill_q8_1(qn, qg, kcache, vcache, xq, xd, pos0, M, kq_scale, nqh, nkvh, n_ctx, q8=True, depth_hint=-1):
    """attn_prefill with the q8_1 quantisation of the output (src/model.cu:1230) done in the epilogue."""
    _check(_lib.q27b_attn_prefill_q8_1(_ptr(qn, torch.float32), _ptr(qg, torch.float32), _ptr(kcache), _ptr(vcache),
                                       _ptr(xq, torch.int8), _ptr(xd, torch.float32), _ptr(pos0, torch.int32), int(M),
                                       _f(kq_scale), int(nqh), int(nkvh), int(n_ctx), int(bool(q8)), _stream(),
                                       int(depth_hint)))


def prefill_qk_debug(x, rows, kq_scale, kcache, nkvh, n_ctx, kh, p0, npos, q_i8, q_scale, acc):
    """Integer stage of the prefill kernel on one tile (test hook)."""
    _check(_lib.q27b_prefill_qk_debug(_ptr(x, torch.float32), int(rows), _f(kq_scale), _ptr(kcache), int(nkvh),
                                      int(n_ctx), int(kh), int(p0), int(npos), _ptr(q_i8, torch.int8),
                                      _ptr(q_scale, torch.float32), _ptr(acc, torch.int32), _stream()))
