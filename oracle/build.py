"""Build recipes for the checker code (test infrastructure, never shipped).

build_oracle(): oracle/attn_oracle.cpp -> oracle/liboracle.so (g++ -fopenmp).
build_ref():    the reference's own src/attn.cu + src/ops.cu, compiled where they lie in the
                reference checkout together with oracle/ref_wrap.cu, for sm_100a with the
                reference's flags (CMakeLists.txt:17-21) -> oracle/_ref/libq27ref.so.
                Only possible where the reference checkout is present; elsewhere the
                prebuilt file is used as it is.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libq27ref.so")
# Where the reference checkout lies: the environment variable Q27_REFERENCE_DIR, or the first command-line
# argument that is a directory; without either, the prebuilt files under oracle/_ref are used as they are.
REF_SRC = os.environ.get("Q27_REFERENCE_DIR") or next((a for a in sys.argv[1:] if os.path.isdir(a)), "") or \
    (os.path.join(os.sep, "root", "reference") if os.path.isdir(os.path.join(os.sep, "root", "reference", "src")) else "")
BENCH_ATTN = os.path.join(REF_DIR, "bench_attn_shim")
BENCH_ATTN_REF = os.path.join(REF_DIR, "bench_attn_ref")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "attn_oracle.cpp")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    cmd = ["g++", "-std=c++17", "-O3", "-mavx2", "-mf16c", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
           src, "-o", ORACLE_SO]
    subprocess.check_call(cmd)
    return ORACLE_SO


def ref_available():
    return bool(REF_SRC) and os.path.isdir(os.path.join(REF_SRC, "src"))


def build_ref(force=False):
    """Returns the path of libq27ref.so, or None when it is neither built nor buildable."""
    wrap = os.path.join(HERE, "ref_wrap.cu")
    if not ref_available():
        return REF_SO if os.path.exists(REF_SO) else None
    srcs = [wrap, os.path.join(REF_SRC, "src", "attn.cu"), os.path.join(REF_SRC, "src", "ops.cu")]
    if not force and _newer(REF_SO, srcs):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-use_fast_math",
           "--expt-relaxed-constexpr", "-lineinfo", "-I", os.path.join(REF_SRC, "src"), "-shared", "-Xcompiler",
           "-fPIC", "-cudart", "shared"] + srcs + ["-o", REF_SO]
    subprocess.check_call(cmd)
    return REF_SO


def build_bench_attn(force=False):
    """The reference's own check-and-bench tool, tools/bench_attn.cu, compiled UNMODIFIED where it lies
    against this repository's shim headers (qwen27-engine_b200/shim: ops.h, common.cuh) and linked with
    libq27b_attn.so -> oracle/_ref/bench_attn_shim. It is the most direct test of the drop-in boundary:
    the reference's program running on the new kernels. Returns the path, or None when it is neither
    built nor buildable here."""
    pkg = os.path.join(os.path.dirname(HERE), "qwen27-engine_b200")
    lib = os.path.join(pkg, "libq27b_attn.so")
    if not ref_available() or not os.path.exists(lib):
        return BENCH_ATTN if os.path.exists(BENCH_ATTN) else None
    src = os.path.join(REF_SRC, "tools", "bench_attn.cu")
    shim = os.path.join(pkg, "shim")
    deps = [src, lib] + [os.path.join(shim, f) for f in os.listdir(shim)]
    if not force and _newer(BENCH_ATTN, deps):
        return BENCH_ATTN
    os.makedirs(REF_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I", shim, src, "-L", pkg,
           "-lq27b_attn", "-Xlinker", "-rpath=$ORIGIN/../../qwen27-engine_b200", "-cudart", "static", "-o", BENCH_ATTN]
    subprocess.check_call(cmd)
    return BENCH_ATTN


def build_bench_attn_ref(force=False):
    """The same tool linked with the reference's own kernels (oracle/_ref/libq27ref.so) ->
    oracle/_ref/bench_attn_ref: what the reference prints about itself on the same GPU, to set the new
    kernels' numbers against."""
    so = build_ref()
    if not ref_available() or so is None:
        return BENCH_ATTN_REF if os.path.exists(BENCH_ATTN_REF) else None
    src = os.path.join(REF_SRC, "tools", "bench_attn.cu")
    if not force and _newer(BENCH_ATTN_REF, [src, so]):
        return BENCH_ATTN_REF
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr", "-I",
           os.path.join(REF_SRC, "src"), src, "-L", REF_DIR, "-lq27ref", "-Xlinker", "-rpath=$ORIGIN", "-cudart", "shared",
           "-o", BENCH_ATTN_REF]
    subprocess.check_call(cmd)
    return BENCH_ATTN_REF


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(build_bench_attn(force="--force" in sys.argv))
    print(build_bench_attn_ref(force="--force" in sys.argv))
