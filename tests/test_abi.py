"""The C-ABI library loads without a GPU, exports every symbol that include/q27b_attn.h declares,
and rejects bad shapes on the host with the reference's error behaviour (src/attn.cu:906,929)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "q27b_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q27b_[a-z0-9_]+)\s*\(", text)))


def test_exports_every_declared_symbol(q27):
    lib = ctypes.CDLL(q27.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), "missing export " + n
    assert sorted(q27.SYMBOLS) == names


def test_cache_sizes(q27):
    assert q27.kv_cache_bytes(4, 150008, True) == 4 * 150008 * 272
    assert q27.kv_cache_bytes(2, 1000, False) == 2 * 1000 * 512
    assert q27.kv_pool_bytes(4, 10) == 10 * 4 * 256 * 272


def test_bad_shapes_are_rejected_on_the_host(q27):
    lib = ctypes.CDLL(q27.LIB_PATH)
    lib.q27b_last_error.restype = ctypes.c_char_p
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)  # never dereferenced: the shape check comes first
    f = ctypes.c_float(0.0625)
    # T out of range, and nqh != 6 * nkvh
    for T, nqh, nkvh in [(0, 24, 4), (5, 24, 4), (4, 20, 4)]:
        rc = lib.q27b_attn_decode(one, one, one, one, one, null, null, one, T, f, nqh, nkvh, 1024, 1, null)
        assert rc == q27.BAD_SHAPE
        assert b"attn_decode: bad shape" in lib.q27b_last_error()
    rc = lib.q27b_attn_prefill(one, one, one, one, one, one, 0, f, 24, 4, 1024, 1, null, -1)
    assert rc == q27.BAD_SHAPE and b"attn_prefill: bad shape" in lib.q27b_last_error()
    rc = lib.q27b_attn_prefill(one, one, one, one, one, one, 16, f, 25, 4, 1024, 1, null, -1)
    assert rc == q27.BAD_SHAPE
    rc = lib.q27b_attn_decode(null, one, one, one, one, null, null, one, 4, f, 24, 4, 1024, 1, null)
    assert rc == q27.BAD_SHAPE and b"null pointer" in lib.q27b_last_error()
    rc = lib.q27b_kv_append(one, one, one, one, one, 0, 4, 1024, 1, null)
    assert rc == q27.BAD_SHAPE
    rc = lib.q27b_lse_merge(null, 2, ctypes.c_int64(0), ctypes.c_int64(1), null, one, null, null, null)
    assert rc == q27.BAD_SHAPE


def test_decode_kernel_selection_is_checked(q27):
    lib = ctypes.CDLL(q27.LIB_PATH)
    lib.q27b_last_error.restype = ctypes.c_char_p
    for which in (0, 1, 2, 3, 4, 0):
        assert lib.q27b_set_decode_kernel(which) == 0
    for which in (-1, 5):
        assert lib.q27b_set_decode_kernel(which) == q27.BAD_SHAPE
        assert b"set_decode_kernel" in lib.q27b_last_error()


def test_prefill_kernel_selection_is_checked(q27):
    lib = ctypes.CDLL(q27.LIB_PATH)
    lib.q27b_last_error.restype = ctypes.c_char_p
    for which in (0, 1, 2, 0):
        assert lib.q27b_set_prefill_kernel(which) == 0
    for which in (-1, 3):
        assert lib.q27b_set_prefill_kernel(which) == q27.BAD_SHAPE
        assert b"set_prefill_kernel" in lib.q27b_last_error()


def test_prefill_split_plan(q27, monkeypatch):
    """Host arithmetic of the prefill split: the reference's rule while the CTAs do not fill the GPU,
    the tail split on a deep prefix, nothing on a short one."""
    monkeypatch.delenv("Q27_ATTN_SPLIT", raising=False)
    monkeypatch.delenv("Q27B_PREFILL_TAIL_SPLIT", raising=False)
    assert q27.prefill_split_plan(2048, 24, 148, -1) == (0, 1)          # no hint: never split
    assert q27.prefill_split_plan(2048, 24, 148, 0) == (0, 1)           # short prefix
    ts, ns = q27.prefill_split_plan(2048, 24, 148, 32768)                # 384 CTAs = 2 rounds + 88
    assert ts == 4 and 2 <= ns <= 8
    ts2, ns2 = q27.prefill_split_plan(2048, 24, 148, 148000)
    assert ts2 == 4 and ns2 >= ns                                        # pieces get cheaper with depth
    assert q27.prefill_split_plan(70, 6, 148, 8000) == (1, 3)            # 6 CTAs: every tile, (8000 + 70) / 2048 pieces
    assert q27.prefill_split_plan(128 * 37, 4, 148, 10 ** 6) == (37, 2)  # 148 CTAs: the reference's rule, two per SM
    assert q27.prefill_split_plan(128 * 74, 4, 148, 10 ** 6) == (0, 1)   # 296 CTAs: two full rounds
    for M, nqh, depth in [(896, 24, 3600), (2048, 12, 32768), (1024, 24, 65536), (4096, 24, 200000)]:
        ts, ns = q27.prefill_split_plan(M, nqh, 148, depth)
        tiles = (M + 127) // 128
        assert 0 <= ts <= tiles and 1 <= ns <= 8 and (ts == 0) == (ns == 1)
        if 0 < ts < tiles:  # tail split: the unsplit CTAs fit in full rounds
            assert (tiles - ts) * nqh <= (tiles * nqh // 148) * 148
    monkeypatch.setenv("Q27_ATTN_SPLIT", "3")
    assert q27.prefill_split_plan(2048, 24, 148, 32768) == (16, 3)
    monkeypatch.setenv("Q27_ATTN_SPLIT", "1")
    assert q27.prefill_split_plan(2048, 24, 148, 32768) == (0, 1)


def test_sum_norm_entry_points_check_their_arguments(q27):
    """Argument checks of the sum_norm family come before any CUDA call."""
    lib = ctypes.CDLL(q27.LIB_PATH)
    lib.q27b_last_error.restype = ctypes.c_char_p
    lib.q27b_sum_xbuf_bytes.restype = ctypes.c_uint64
    assert lib.q27b_sum_xbuf_bytes(8, 4, 5120) == 256 + 2 * 8 * 4 * 5120 * 8  # 8-byte words {value, step tag}
    assert lib.q27b_sum_xbuf_bytes(0, 4, 5120) == 0
    null, one = ctypes.c_void_p(0), ctypes.c_void_p(16)
    f = ctypes.c_float(1e-6)
    assert lib.q27b_sum_norm_q8(null, one, 5120, 4, one, f, null, null, null, null) == q27.BAD_SHAPE
    assert lib.q27b_sum_norm_q8(one, one, 5100, 4, one, f, null, null, null, null) == q27.BAD_SHAPE   # n % 32
    assert lib.q27b_sum_norm_q8(one, one, 32768, 4, one, f, null, null, null, null) == q27.BAD_SHAPE  # n > 16384
    assert lib.q27b_sum_norm_q8(one, one, 5120, 4, one, f, null, one, null, null) == q27.BAD_SHAPE    # xq without xd
    assert lib.q27b_sum_push(one, 5120, 4, 2, 2, one, null) == q27.BAD_SHAPE                         # rank >= world
    assert lib.q27b_sum_push(one, 5120, 4, 0, 9, one, null) == q27.BAD_SHAPE                         # more than 8 ranks
    assert lib.q27b_sum_norm_q8_wait(one, null, 2, 5120, 4, one, f, null, null, null, null) == q27.BAD_SHAPE
    assert b"sum_norm_q8_wait" in lib.q27b_last_error()
    assert lib.q27b_xbuf_alloc_bytes(ctypes.c_uint64(8), ctypes.byref(ctypes.c_void_p(0))) == q27.BAD_SHAPE


def test_paged_and_exchange_entry_points_check_their_arguments(q27):
    """The entry points added around the paged cache and the peer-memory exchanges refuse bad arguments
    before any CUDA call."""
    lib = ctypes.CDLL(q27.LIB_PATH)
    lib.q27b_last_error.restype = ctypes.c_char_p
    null, one = ctypes.c_void_p(0), ctypes.c_void_p(16)
    f = ctypes.c_float(1.0)
    # q27b_attn_prep_paged: null pool; norm weights without the rest; bad shape
    args = lambda **kw: [kw.get("qg", null), one, one, kw.get("q_norm", null), null, null, kw.get("kpool", one), one, one, one,
                         kw.get("B", 2), 4, f, f, 24, 4, 16, 8, null, null, null]
    assert lib.q27b_attn_prep_paged(*args(kpool=null)) == q27.BAD_SHAPE
    assert lib.q27b_attn_prep_paged(*args(q_norm=one)) == q27.BAD_SHAPE
    assert lib.q27b_attn_prep_paged(*args(B=0)) == q27.BAD_SHAPE
    assert b"attn_prep_paged" in lib.q27b_last_error()
    # q27b_attn_decode_exchange: no output, bad slice index, null buffer list
    ex = lambda o=one, z=0, nz=2, bufs=one: [one, one, one, one, o, one, 4, f, 6, 1, 1000, 1, 0, 500, bufs, z, nz, null]
    assert lib.q27b_attn_decode_exchange(*ex(o=null)) == q27.BAD_SHAPE
    assert lib.q27b_attn_decode_exchange(*ex(z=2)) == q27.BAD_SHAPE
    assert lib.q27b_attn_decode_exchange(*ex(nz=9)) == q27.BAD_SHAPE
    assert lib.q27b_attn_decode_exchange(*ex(bufs=null)) == q27.BAD_SHAPE
    # q27b_sum_exchange_norm_q8
    assert lib.q27b_sum_exchange_norm_q8(one, null, 5120, 4, 0, 2, one, one, f, null, null, null, null) == q27.BAD_SHAPE
    assert lib.q27b_sum_exchange_norm_q8(one, one, 5120, 4, 2, 2, one, one, f, null, null, null, null) == q27.BAD_SHAPE
    assert lib.q27b_sum_exchange_norm_q8(one, one, 5100, 4, 0, 2, one, one, f, null, null, null, null) == q27.BAD_SHAPE
    # q27b_xbuf_reset: less than the header; q27b_kv_page_copy: a page onto itself
    assert lib.q27b_xbuf_reset(one, ctypes.c_uint64(8), null) == q27.BAD_SHAPE
    assert lib.q27b_kv_page_copy(one, 1, 1, 10, 4, 8, null) == q27.BAD_SHAPE
    assert lib.q27b_kv_page_copy(one, 0, 9, 10, 4, 8, null) == q27.BAD_SHAPE
    lib.q27b_xbuf_bytes.restype = ctypes.c_uint64
    assert lib.q27b_xbuf_bytes(2, ctypes.c_int64(24)) == 256 + 2 * 2 * 24 * 258 * 8


def test_python_mirror_raises(q27):
    with pytest.raises(RuntimeError):
        q27.kv_append(None, None, None, None, None, 1, 4, 16)


def test_shim_header_compiles():
    """The C++ shim with the reference's signatures compiles against the C ABI (host only): every operator
    of src/ops.h:50-77 is called with the reference's argument lists, default arguments included."""
    import subprocess
    import tempfile
    src = """#include "common.cuh"
#include "ops.h"
using namespace q27;
int main(int argc, char**) {
  if (argc > 100) {  // never taken: the calls only have to compile and link
    cudaStream_t s = nullptr;
    const float* f = nullptr; float* g = nullptr; void* c = nullptr; const int* p = nullptr; int8_t* q = nullptr;
    attn_prep(f, f, f, f, f, g, c, c, p, 4, 1e-6f, 0.5f, 24, 4, 64, true, s);
    attn_prep(f, f, f, f, f, g, c, c, p, 4, 1e-6f, 0.5f, 24, 4, 64, true, s, nullptr, 0, p, p);
    attn_decode(f, f, c, c, g, q, g, p, 4, 0.0625f, 24, 4, 64, true, s);
    attn_prefill(f, f, c, c, g, p, 128, 0.0625f, 24, 4, 64, true, s);
    attn_prefill(f, f, c, c, g, p, 128, 0.0625f, 24, 4, 64, true, s, 1000);
    attn_decode_ref(f, f, c, c, g, p, 4, 0.0625f, 24, 4, 64, true, s);
    CK(cudaStreamSynchronize(s));
    return attn_chunks(4);
  }
  return kv_cache_bytes(4, 16, true) == (size_t)4 * 16 * 272 && kv_cache_bytes(4, 16, false) == (size_t)4 * 16 * 512 ? 0 : 1;
}
"""
    with tempfile.TemporaryDirectory() as d:
        p = os.path.join(d, "t.cpp")
        open(p, "w").write(src)
        pkg = os.path.join(ROOT, "qwen27-engine_b200")
        exe = os.path.join(d, "t")
        subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(pkg, "shim"), "-I", "/usr/local/cuda/include", p,
                               "-L", pkg, "-lq27b_attn", "-Wl,-rpath," + pkg, "-L", "/usr/local/cuda/lib64", "-lcudart_static",
                               "-ldl", "-lrt", "-lpthread", "-o", exe])
        assert subprocess.call([exe]) == 0


def test_reference_bench_tool_builds_against_the_shim():
    """tools/bench_attn.cu of the reference compiles and links UNMODIFIED against the shim headers and the
    library (the -m gpu suite runs the result). Needs the reference checkout; elsewhere the prebuilt file
    must at least be there."""
    from oracle import build as ob
    if ob.ref_available():
        exe = ob.build_bench_attn(force=True)
        assert exe and os.path.exists(exe)
    else:
        exe = ob.build_bench_attn()
        if exe is None:
            pytest.skip("no reference checkout and no prebuilt oracle/_ref/bench_attn_shim")
        assert os.access(exe, os.X_OK)


def test_sum_push_refuses_a_null_buffer_before_any_cuda_call(q27):
    lib = ctypes.CDLL(q27.LIB_PATH)
    lib.q27b_last_error.restype = ctypes.c_char_p
    bufs = (ctypes.c_void_p * 2)(ctypes.c_void_p(16), ctypes.c_void_p(0))
    assert lib.q27b_sum_push(ctypes.c_void_p(16), 5120, 4, 0, 2, bufs, ctypes.c_void_p(0)) == q27.BAD_SHAPE
    assert b"null exchange buffer" in lib.q27b_last_error()
