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
REF_SRC = os.environ.get("Q27_REFERENCE_DIR", "/root/reference")


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
    return os.path.isdir(os.path.join(REF_SRC, "src"))


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


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
