"""Generates tests/golden/ref_sum_norm_b200.npz: output of the REFERENCE's own sum_norm_q8 kernel
(src/ops.cu:129-260, no exchange) on seeded inputs.

Needs a B200 and oracle/_ref/libq27ref.so (oracle/build.py); nothing of the reference is read at run
time. tests/test_golden.py recomputes the case with the oracle's numpy statement from the same seeds.

Usage (GPU box): python tests/golden/make_golden_sum_norm.py
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import __graft_entry__ as ge  # noqa: E402
from golden_cases import sum_norm_inputs, SUM_NORM_EPS  # noqa: E402


def main():
    ge.load_package()
    ref = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libq27ref.so"))
    ref.ref_last_error.restype = ctypes.c_char_p
    x, part, w = sum_norm_inputs()
    rows, n = x.shape
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    dx, dp, dw = (torch.from_numpy(a).cuda() for a in (x, part, w))
    h = torch.zeros((rows, n), device="cuda")
    xq = torch.zeros((rows, n), dtype=torch.int8, device="cuda")
    xd = torch.zeros((rows * n // 32,), device="cuda")
    rc = ref.ref_sum_norm_q8(p(dx), p(dp), n, rows, p(dw), ctypes.c_float(SUM_NORM_EPS), p(h), p(xq), p(xd), None)
    if rc:
        raise RuntimeError(ref.ref_last_error().decode())
    torch.cuda.synchronize()
    out = os.path.join(ROOT, "tests", "golden", "ref_sum_norm_b200.npz")
    np.savez_compressed(out, x=dx.cpu().numpy(), h=h.cpu().numpy(), xq=xq.cpu().numpy(), xd=xd.cpu().numpy())
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
