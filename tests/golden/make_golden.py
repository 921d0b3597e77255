"""Generates tests/golden/ref_b200.npz: outputs of the REFERENCE's own kernels on seeded inputs.

Needs a B200 and oracle/_ref/libq27ref.so (the reference's src/attn.cu + src/ops.cu compiled for
sm_100a by oracle/build.py; nothing of the reference is read at run time). The reference holds no
golden vectors for this path, so these outputs are what pins the CPU oracle: tests/test_golden.py
recomputes every case with the oracle from the same seeds.

Usage (GPU box): python tests/golden/make_golden.py [--out tests/golden/ref_b200.npz]
                 python tests/golden/make_golden.py --deep [--out tests/golden/ref_b200_deep.npz]
--deep runs the cases at depth (DEEP_CASES of tests/golden_cases.py) and keeps only the rows the tests compare.
"""
import argparse
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import __graft_entry__ as ge  # noqa: E402
import oracle  # noqa: E402
from golden_cases import CASES, DEEP_CASES, case_inputs  # noqa: E402

AD = 256


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--deep", action="store_true")
    args = ap.parse_args()
    cases = DEEP_CASES if args.deep else CASES
    args.out = args.out or os.path.join(ROOT, "tests", "golden", "ref_b200_deep.npz" if args.deep else "ref_b200.npz")
    ge.load_package()
    ref = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libq27ref.so"))
    ref.ref_last_error.restype = ctypes.c_char_p

    def ck(rc):
        if rc != 0:
            raise RuntimeError(ref.ref_last_error().decode())

    def p(t):
        return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)

    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    f = ctypes.c_float
    out = {}
    for name, c in cases.items():
        x = case_inputs(name)
        kind = c["kind"]
        if kind == "prep":
            T, nqh, nkvh, n_ctx, pos0, q8 = c["T"], c["nqh"], c["nkvh"], c["n_ctx"], c["pos0"], c["q8"]
            qn = torch.zeros((T, nqh, AD), device="cuda")
            nbytes = oracle.kv_cache_bytes(nkvh, n_ctx, q8)
            kc = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
            vc = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
            pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
            keep = [d(x[k]) for k in ("qg", "k", "v", "q_norm", "k_norm")]  # stay alive until the kernel has run
            rope3 = d(np.array(c["rope3"], np.int32)) if c.get("rope3") else None
            ck(ref.ref_attn_prep(p(keep[0]), p(keep[1]), p(keep[2]), p(keep[3]), p(keep[4]), p(qn),
                                 p(kc), p(vc), p(pos), T, f(c["eps"]), f(c["theta_scale"]), nqh, nkvh, n_ctx, int(q8),
                                 None, p(rope3), None))
            torch.cuda.synchronize()
            if T <= 8:
                out[name + "/qn"] = qn.cpu().numpy()
            if c.get("rows_only"):  # the rows just written: values [nkvh][T][256] and scales [nkvh][T][8]
                for key, cache in (("k", kc), ("v", vc)):
                    vals = cache[: nkvh * n_ctx * AD].view(nkvh, n_ctx, AD)[:, pos0:pos0 + T]
                    sc = cache[nkvh * n_ctx * AD:].view(torch.float16).view(nkvh, n_ctx, 8)[:, pos0:pos0 + T]
                    out[name + "/%srows" % key] = vals.cpu().numpy()
                    out[name + "/%sscales" % key] = sc.cpu().numpy()
            else:
                out[name + "/kcache"] = kc.cpu().numpy()
                out[name + "/vcache"] = vc.cpu().numpy()
        elif kind == "decode":
            T, nkvh, n, n_ctx, q8 = c["T"], c["nkvh"], c["n"], c["n_ctx"], c["q8"]
            nqh = nkvh * 6
            kc, vc = oracle.fill_cache(x["k"], x["v"], n_ctx, q8)
            pos = torch.tensor([n - T], dtype=torch.int32, device="cuda")
            qn, qg, kcd, vcd = d(x["qn"]), d(x["qg"]), d(kc), d(vc)
            for fn, key in ((ref.ref_attn_decode_ref, "slow"), (None, "fast")):
                o = torch.zeros((T, nqh, AD), device="cuda")
                if fn is not None:
                    ck(fn(p(qn), p(qg), p(kcd), p(vcd), p(o), p(pos), T, f(c["scale"]), nqh, nkvh, n_ctx, int(q8), None))
                else:
                    ck(ref.ref_attn_decode(p(qn), p(qg), p(kcd), p(vcd), p(o), None, None, p(pos), T, f(c["scale"]), nqh,
                                           nkvh, n_ctx, int(q8), None))
                torch.cuda.synchronize()
                out[name + "/" + key] = o.cpu().numpy()
            if c.get("q8_1"):
                xq = torch.zeros((T, nqh, AD), dtype=torch.int8, device="cuda")
                xd = torch.zeros(T * nqh * 8, device="cuda")
                ck(ref.ref_attn_decode(p(qn), p(qg), p(kcd), p(vcd), None, p(xq), p(xd), p(pos), T, f(c["scale"]), nqh,
                                       nkvh, n_ctx, int(q8), None))
                torch.cuda.synchronize()
                out[name + "/xq"] = xq.cpu().numpy()
                out[name + "/xd"] = xd.cpu().numpy()
        elif kind == "prefill":
            M, nkvh, pos0, n_ctx = c["M"], c["nkvh"], c["pos0"], c["n_ctx"]
            nqh = nkvh * 6
            kc, vc = oracle.fill_cache(x["k"], x["v"], n_ctx, True)
            pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
            o = torch.zeros((M, nqh, AD), device="cuda")
            qn, qg, kcd, vcd = d(x["qn"]), d(x["qg"]), d(kc), d(vc)
            ck(ref.ref_attn_prefill(p(qn), p(qg), p(kcd), p(vcd), p(o), p(pos), M, f(c["scale"]), nqh,
                                    nkvh, n_ctx, 1, None, -1))
            torch.cuda.synchronize()
            if c.get("keep"):  # sampled token ranges only
                for a, b in c["keep"]:
                    out[name + "/i8_%d_%d" % (a, b)] = o[a:b].cpu().numpy()
                continue
            out[name + "/i8"] = o.cpu().numpy()
            o2 = torch.zeros((M, nqh, AD), device="cuda")
            ck(ref.ref_attn_decode_ref(p(qn), p(qg), p(kcd), p(vcd), p(o2), p(pos), M, f(c["scale"]),
                                       nqh, nkvh, n_ctx, 1, None))
            torch.cuda.synchronize()
            out[name + "/slow_f16q"] = o2.cpu().numpy()
    out["meta/gpu"] = np.array(torch.cuda.get_device_name(0))
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
