"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras]

One step = one decode-attention call (split-K kernel + log-sum-exp merge kernel) for a
4-token speculative-verify block, 24 Q / 4 KV heads, head dim 256, over a q8_0 KV cache of
150,000 positions. Metric: algorithmic KV bytes streamed per second,
2 * nkvh * n * 272 B / step time, the reference's own accounting (tools/bench_attn.cu:148).
Inputs are resident in HBM for `value`; `e2e` goes through the C ABI with host buffers (query,
gate, the new K/V rows in pinned host memory -> device, KV append, decode, result -> host).
With N > 1 (torchrun, one rank per GPU) every rank decodes its own sequence (batched decode
sharded by sequence, no exchange): value is the aggregate. The same run also reports, as extra
keys, one sequence sharded over the ranks by KV-head group and then KV length with the NCCL
gather + log-sum-exp merge ("strong"), the other context depths, the prefill TOPS and the
reference's own kernels on the same GPU.

Timing: `value` is taken the way the reference times this operator (tools/bench_attn.cu:131-147): the
steps are captured in CUDA graphs of 20 calls and replayed, so that host launch time does not count;
the call-by-call figure is kept beside it (eager_*). The split-K kernel alone (roofline) is timed with
CUDA events recorded inside such a graph, on the launching stream, around each launch of the kernel.

--impl reference runs the reference's kernels (oracle/_ref/libq27ref.so: its src/attn.cu compiled
for sm_100a, called through its own q27::attn_decode) on the same workload, timed the same way; that
process loads nothing of this repository's library (the caches are written with torch). The reference
has no CPU implementation of this path. If that library is missing, the CPU oracle is timed instead.
"""
import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

AD, GQA, T, NKVH, NQH = 256, 6, 4, 4, 24
N_POS = 150000
N_CTX = 150056
SCALE = 1.0 / 16.0
NBUF = 3  # rotating caches: the reuse distance (3 x 326 MB) is far beyond the 126 MB L2


def env_int(name, default):
    return int(os.environ.get(name, default))


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cool_down(seconds=0.4):
    """Lets the GPU leave the power-capped state that tens of milliseconds of back-to-back launches of these
    kernels put it in (SM clock 1965 -> 1830 MHz with sw_power_cap active, the same launches 10 % slower):
    the copy peak that the roofline is quoted against is a burst figure (best of ten 0.7 ms copies), so the
    kernels are timed as bursts too, each after a short idle."""
    torch.cuda.synchronize()
    time.sleep(seconds)


def graph_us(fn, calls=20, replays=5):
    """Microseconds per call of fn(i), from `calls` calls captured in one CUDA graph and replayed."""
    fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls):
            fn(i)
    cool_down()
    g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (calls * replays)


def torch_q8_cache(nkvh, n, n_ctx, gen):
    """One q8_0 cache in the reference's layout (int8 values [nkvh][n_ctx][256], then f16 scales
    [nkvh][n_ctx][8]) holding n positions of N(0,1) rows, quantised with torch operations (d = amax / 127
    per 32 values, q = round(x / d)): synthetic data of the metric's distribution that neither arm's
    library has touched."""
    buf = torch.zeros(nkvh * n_ctx * 272, dtype=torch.uint8, device="cuda")
    vals = buf[: nkvh * n_ctx * AD].view(torch.int8).view(nkvh, n_ctx, AD)
    sc = buf[nkvh * n_ctx * AD:].view(torch.float16).view(nkvh, n_ctx, 8)
    step = 16384
    for p0 in range(0, n, step):
        m = min(step, n - p0)
        x = torch.randn((nkvh, m, 8, 32), generator=gen, device="cuda")
        d = x.abs().amax(-1, keepdim=True) / 127.0
        vals[:, p0:p0 + m] = (x / d).round_().clamp_(-127, 127).to(torch.int8).view(nkvh, m, AD)
        sc[:, p0:p0 + m] = d.squeeze(-1).to(torch.float16)
    return buf


def torch_caches(nkvh, n, n_ctx, seed, q8=True):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    if q8:
        return torch_q8_cache(nkvh, n, n_ctx, g), torch_q8_cache(nkvh, n, n_ctx, g)

    def f16():  # f16 cache [nkvh][n_ctx][256] halves
        c = torch.zeros((nkvh, n_ctx, AD), dtype=torch.float16, device="cuda")
        for p0 in range(0, n, 16384):
            m = min(16384, n - p0)
            c[:, p0:p0 + m] = torch.randn((nkvh, m, AD), generator=g, device="cuda").to(torch.float16)
        return c.view(torch.uint8).view(-1)
    return f16(), f16()


def kv_bytes(nkvh, n):
    return 2.0 * nkvh * n * 272


def time_steps(fn, steps, warmup, dist=None):
    """W untimed calls, then K calls between two events; barrier + synchronize on both sides;
    returns ms per step (max over ranks)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


def time_graph_steps(fn, steps, warmup, dist=None, calls=20):
    """The same contract with the steps captured in CUDA graphs: W untimed calls issued one by one, then
    graphs of `calls` steps (one graph of all K steps when K is not a multiple of it), one untimed replay,
    then exactly K steps of replays between two events; returns ms per step (max over ranks)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if steps % calls != 0:
        calls = steps
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls):
            fn(warmup + i)
    g.replay()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # One untimed replay goes first and is not waited for: while the GPU runs it the host queues the first event
    # and the timed replays, so the events bracket exactly K steps of device time and not the host's launch
    # latency of the first timed replay (with K = 20 that is the only one: 0.6 us per step on one GPU, 3 to 4 us
    # with several ranks launching from one host).
    g.replay()
    e0.record()
    for _ in range(steps // calls):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    return ms


class RefLib:
    """The reference's kernels (oracle/_ref/libq27ref.so) behind its own operator API."""

    def __init__(self):
        path = os.path.join(ROOT, "oracle", "_ref", "libq27ref.so")
        self.lib = ctypes.CDLL(path)
        self.lib.ref_last_error.restype = ctypes.c_char_p

    @staticmethod
    def _p(t):
        return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)

    def _ck(self, rc):
        if rc:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def decode(self, qn, qg, kc, vc, o, pos, T_, nqh, nkvh, n_ctx):
        s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._ck(self.lib.ref_attn_decode(self._p(qn), self._p(qg), self._p(kc), self._p(vc), self._p(o), None, None,
                                          self._p(pos), T_, ctypes.c_float(SCALE), nqh, nkvh, n_ctx, 1, s))

    def prefill(self, qn, qg, kc, vc, o, pos, M, nqh, nkvh, n_ctx, hint, q8=True):
        s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._ck(self.lib.ref_attn_prefill(self._p(qn), self._p(qg), self._p(kc), self._p(vc), self._p(o), self._p(pos), M,
                                           ctypes.c_float(SCALE), nqh, nkvh, n_ctx, int(q8), s, hint))


def cpu_baseline(n=N_POS):
    """The CPU oracle (C++/OpenMP restatement of the reference numerics) on the full decode workload."""
    import oracle
    rng = np.random.default_rng(7)
    nkvh, nqh = NKVH, NQH
    kc = oracle.new_cache(nkvh, n)
    vc = oracle.new_cache(nkvh, n)
    for c in (kc, vc):  # random int8 values and scales around 1/127: the cost does not depend on the values
        c[: nkvh * n * AD] = rng.integers(0, 256, nkvh * n * AD, dtype=np.uint8)
        c[nkvh * n * AD:].view(np.float16)[:] = (rng.random(nkvh * n * 8) * 0.02 + 0.005).astype(np.float16)
    qn = rng.standard_normal((T, nqh, AD)).astype(np.float32)
    qg = rng.standard_normal((T, nqh, 512)).astype(np.float32)
    oracle.attn_ref(qn, qg, kc, vc, n - T, SCALE, nkvh, n)  # warm
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 8 and reps < 20):
        oracle.attn_ref(qn, qg, kc, vc, n - T, SCALE, nkvh, n)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": kv_bytes(nkvh, n) / dt / 1e9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": "%d full calls of the same workload (T=4, 24q/4kv, n=%d) on the host cores" % (reps, n),
            "ms_per_step": dt * 1e3}


def measure_mma_peak(q, kind, iters=4000, reps=3):
    """TOPS (kind 0: tcgen05.mma kind::i8) or TFLOP/s (kind 1: kind::f16) of the library's tensor-core peak
    microbenchmark: back-to-back 128 x 256 tiles from operands resident in shared memory, one CTA per SM,
    timed with CUDA events around the launch; best of `reps`."""
    q.debug_mma_peak(kind, 200)
    torch.cuda.synchronize()
    best = 0.0
    for _ in range(reps):
        cool_down(0.5)  # a peak is a burst figure: not taken in the power-capped state that earlier timings leave
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops = q.debug_mma_peak(kind, iters)
        e1.record()
        torch.cuda.synchronize()
        best = max(best, ops / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--ref-cpu", action="store_true", help="reference arm: time the CPU oracle instead of the reference's GPU kernels")
    ap.add_argument("--n", type=int, default=N_POS)
    ap.add_argument("--mode", default="decode", help="decode (the headline), prefill (second half of the metric), paged (config 5: the batched decode over pages) or sum_norm (N > 1: the exchange after the output projection)")
    ap.add_argument("--prefix", type=int, default=32768, help="prefill mode: tokens already in the cache")
    ap.add_argument("--seqs", type=int, default=64, help="paged mode: sequences in the batch")
    ap.add_argument("--max-len", type=int, default=131072, help="paged mode: lengths are uniform in 1024 .. this")
    ap.add_argument("--kv", default="q8", help="prefill mode: q8 (int8 Q K^T on the q8_0 cache) or f16 (f16 Q K^T on an f16 cache)")
    args = ap.parse_args()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    world = env_int("WORLD_SIZE", 1)
    rank = env_int("RANK", 0)
    local = env_int("LOCAL_RANK", 0)
    n = args.n
    n_ctx = max(N_CTX, n + 2048 + 8)

    if args.impl == "reference" and rank != 0:
        return  # the reference arm is a single-GPU program: rank 0 alone runs it
    dist = None
    if world > 1 and args.impl != "reference":
        import torch.distributed as dist_
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist_.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_
    else:
        torch.cuda.set_device(local)

    if args.impl == "reference":
        q = None  # the reference arm loads nothing of this repository's library
    else:
        q = ge.load_package()
    if args.mode == "prefill":
        prefill_mode(q, args, steps, warmup, dist, rank, world)
        return
    if args.mode == "paged":  # config 5 alone (or a smaller batch of the same kind: --seqs, --max-len)
        out = batched_paged(q, rank, world, dist, args.seqs, args.max_len)
        if rank == 0:
            print(json.dumps({"metric": "batched paged q8_0 decode-attn HBM GB/s", "value": out["value"], "unit": "GB/s",
                              "n_gpus": world, "steps": 20, "warmup": 3, "ms_per_step": out["ms_per_step"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                              "data": "synthetic", "config": {"workload": out["what"]}, "gpu_launches": 40,
                              "roofline": {"bound": "hbm", "achieved": out["value"] / world, "peak": peaks()[0]["hbm_gbs"],
                                           "unit": "GB/s", "frac": out["value"] / world / peaks()[0]["hbm_gbs"],
                                           "what": "the whole step (split-K kernel + merge) against the measured copy peak"},
                              "detail": out}))
        if dist is not None:
            dist.barrier()
        return
    if args.mode == "sum_norm":  # the exchange after the output projection alone (needs N > 1)
        if dist is None:
            raise SystemExit("--mode sum_norm needs torchrun with at least 2 ranks")
        out = sum_norm_scaling(q, dist, rank, world, steps, warmup)
        if rank == 0:
            print(json.dumps({"metric": "sum_norm_q8 us/step (x[4][5120] += sum over GPUs, RMSNorm, q8_1)", "value": out["us_per_step"],
                              "unit": "us", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": out["us_per_step"] / 1e3,
                              "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                              "config": {"workload": out["what"]}, "gpu_launches": 2 * steps, "detail": out}))
        dist.barrier()
        return
    line = {
        "metric": "q8_0 decode-attn HBM GB/s @150k ctx (4-token verify block, 24q/4kv heads, head dim 256)",
        "unit": "GB/s", "n_gpus": world if args.impl != "reference" else 1, "steps": steps, "warmup": warmup,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "verify-decode T=4, 24 Q / 4 KV heads, head_dim 256, q8_0 KV length %d" % n,
                   "per_gpu": "one sequence per GPU (batched decode sharded by sequence, no exchange)",
                   "bytes_per_step_per_gpu": kv_bytes(NKVH, n),
                   "l2": "%.0f MB of KV per step, %d caches in rotation: inputs larger than L2" % (kv_bytes(NKVH, n) / 1e6, NBUF),
                   "timing": "steps captured in CUDA graphs of 20 calls and replayed (tools/bench_attn.cu:131-147), after 0.4 s of "
                             "idle and one untimed replay that is still running when the first event is queued; "
                             "eager_* = the same calls issued one by one"},
    }

    # ---- inputs resident in HBM: q8_0 caches of N(0,1) rows written with torch (the same for both arms)
    caches = [torch_caches(NKVH, n, n_ctx, 1002 + 10 * rank + i) for i in range(NBUF)]
    g = torch.Generator(device="cuda")
    g.manual_seed(1001 + rank)
    qn = torch.randn((T, NQH, AD), generator=g, device="cuda")
    qg = torch.randn((T, NQH, 512), generator=g, device="cuda")
    o = torch.empty((T, NQH, AD), device="cuda")
    pos = torch.tensor([n - T], dtype=torch.int32, device="cuda")

    if args.impl == "reference":
        run_reference(args, line, caches, qn, qg, o, pos, n, n_ctx, steps, warmup)
        return

    def step(i):
        kc, vc = caches[i % NBUF]
        q.attn_decode(qn, qg, kc, vc, o, None, None, pos, T, SCALE, NQH, NKVH, n_ctx)

    cool_down()  # (the cache build above is tens of milliseconds of load)
    sampler = ClockSampler(local)
    sampler.start()
    ms = time_graph_steps(step, steps, warmup, dist)
    clocks = sampler.stop()
    assert q.device_status() == 0, "a kernel reported a device-side problem"
    ms_eager = time_steps(step, steps, warmup, dist)
    line["value"] = world * kv_bytes(NKVH, n) / (ms * 1e-3) / 1e9
    line["ms_per_step"] = ms
    line["us_per_step"] = ms * 1e3
    line["eager_ms_per_step"] = ms_eager
    line["eager_value"] = world * kv_bytes(NKVH, n) / (ms_eager * 1e-3) / 1e9
    line["gpu_launches"] = 2 * steps
    line["clocks"] = clocks

    # ---- the dominant kernel alone (split-K decode kernel): CUDA events recorded on the launching stream
    # around every launch of it, inside a replayed graph of 20 calls (event nodes of the graph)
    line["roofline"] = split_kernel_roofline(q, step, n)

    # ---- end to end through the C ABI with host buffers
    line["e2e"] = e2e(q, caches, n, n_ctx, steps, warmup, dist, world)

    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(n)
    if world > 1:
        line["strong"] = strong_scaling(q, dist, rank, world, n, steps, warmup)
        del caches
        torch.cuda.empty_cache()
        line["batched_paged"] = batched_paged(q, rank, world, dist)
        try:
            line["sum_norm"] = sum_norm_scaling(q, dist, rank, world, steps, warmup)
        except Exception as e:  # report, do not hide (every rank raises or none: the set-up agrees on errors)
            line["sum_norm"] = {"error": str(e)}
    if rank == 0 and world == 1 and not args.no_extras:
        line["extras"] = extras(q, caches, qn, qg, o, n_ctx)
        # the second half of the metric, last in the line: int8 prefill TOPS of a 2048-token chunk per prefix depth
        line["prefill_int8_tops"] = {k: round(v["tops"], 1) for k, v in line["extras"]["prefill"].items() if "tops" in v}
        i8 = line["extras"].get("mma_peak", {}).get("int8_tops")
        if i8:
            line["prefill_int8_tops"]["int8_peak_measured"] = round(i8, 1)
            line["prefill_int8_tops"]["frac_of_int8_peak"] = {k: round(v / i8, 3) for k, v in line["prefill_int8_tops"].items()
                                                              if k.isdigit()}
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


BURSTS = 5


def split_kernel_roofline(q, step, n, calls=20, replays=3):
    """Average duration of one launch of the split-K kernel: a CUDA graph of `calls` decode calls that stop
    after the split-K kernel (q27b_debug_split_only), replayed between two CUDA events on the launching
    stream; against the measured copy peak. (With event nodes around every launch inside the graph the
    figure comes out 3-5 us higher than the whole two-kernel step: event_nodes_us, kept for the record.)"""
    step(0)
    torch.cuda.synchronize()
    q.debug_split_only(True)
    try:
        gs = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gs):
            for i in range(calls):
                step(i)
    finally:
        q.debug_split_only(False)
    bursts = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(BURSTS):  # each burst: idle, one untimed replay, `replays` timed ones (a few ms)
        cool_down()
        gs.replay()
        e0.record()
        for _ in range(replays):
            gs.replay()
        e1.record()
        torch.cuda.synchronize()
        bursts.append(e0.elapsed_time(e1) * 1e3 / (calls * replays))
    kus = sorted(bursts)[len(bursts) // 2]
    ev0 = [torch.cuda.Event(enable_timing=True) for _ in range(calls)]
    ev1 = [torch.cuda.Event(enable_timing=True) for _ in range(calls)]
    for e in ev0 + ev1:
        e.record()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls):
            q.debug_split_events(ev0[i], ev1[i])
            step(i)
    q.debug_split_events(None, None)
    g.replay()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    ev_us = sum(a.elapsed_time(b) for a, b in zip(ev0, ev1)) / calls * 1e3
    pk, pk_kind = peaks()
    ach = kv_bytes(NKVH, n) / (kus * 1e-6) / 1e9
    return {"bound": "hbm", "kernel": "decode_ws_kernel<3,false> (q8_0, T=4)", "achieved": ach, "peak": pk["hbm_gbs"],
            "unit": "GB/s", "frac": ach / pk["hbm_gbs"], "peak_kind": pk_kind + " copy bandwidth (burst)",
            "frac_of_8TBs_nominal": ach / 8000.0, "kernel_us": kus, "launches_timed": calls * replays * BURSTS,
            "kernel_us_bursts": [round(x, 2) for x in bursts],
            "how": "median of %d bursts of %d launches (a replayed CUDA graph of %d), 0.4 s idle before each" % (BURSTS, calls * replays, calls),
            "event_nodes_us": ev_us, "traffic": env_float("Q27B_NCU_TRAFFIC_BYTES")}


def env_float(name):
    v = os.environ.get(name)
    return float(v) if v else NCU_TRAFFIC_BYTES


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the decode kernel at the bench workload,
# from an ncu capture at 60,000 positions scaled to 150,000: the reads (130.82 MB) grow in proportion to
# the positions, the writes (3.62 MB: the partials) do not.
NCU_TRAFFIC_BYTES = 330.7e6


def e2e(q, caches, n, n_ctx, steps, warmup, dist, world):
    """Host buffers in, host buffer out, every step: query + gate + the 4 new K/V rows from pinned
    memory, KV append at the tail of the cache, decode, result back to pinned memory."""
    # one pinned staging buffer and one device buffer for all inputs of a step: a single H2D copy
    sizes = [T * NQH * AD, T * NQH * 512, T * NKVH * AD, T * NKVH * AD]
    h_in = torch.randn((sum(sizes),)).pin_memory()
    d_in = torch.empty((sum(sizes),), device="cuda")
    offs = [0, sizes[0], sizes[0] + sizes[1], sizes[0] + sizes[1] + sizes[2]]
    d_qn = d_in[offs[0]:offs[0] + sizes[0]].view(T, NQH, AD)
    d_qg = d_in[offs[1]:offs[1] + sizes[1]].view(T, NQH, 512)
    d_k = d_in[offs[2]:offs[2] + sizes[2]].view(T, NKVH, AD)
    d_v = d_in[offs[3]:offs[3] + sizes[3]].view(T, NKVH, AD)
    h_o = torch.empty((T, NQH, AD)).pin_memory()
    d_o = torch.empty((T, NQH, AD), device="cuda")
    pos = torch.tensor([n - T], dtype=torch.int32, device="cuda")

    def step(i):
        kc, vc = caches[i % NBUF]
        d_in.copy_(h_in, non_blocking=True)
        q.kv_append(d_k, d_v, kc, vc, pos, T, NKVH, n_ctx)
        q.attn_decode(d_qn, d_qg, kc, vc, d_o, None, None, pos, T, SCALE, NQH, NKVH, n_ctx)
        h_o.copy_(d_o, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result before the next step

    ms_eager = time_steps(step, steps, warmup, dist)

    # The same step the way the reference's engine issues a decode step: captured once in a CUDA graph
    # (src/model.cu:910-955), one graph per cache of the rotation; a step is one replay plus the
    # synchronise before the host reads the result. The copies are memcpy nodes of the graph. (A graph with
    # the gate's 196 KB on a branch of its own, joined before the merge kernel, was measured too: 130 us
    # against 107 us per step - three copy nodes and a join cost more than the overlap returns.)
    def body(i):
        kc, vc = caches[i % NBUF]
        d_in.copy_(h_in, non_blocking=True)
        q.kv_append(d_k, d_v, kc, vc, pos, T, NKVH, n_ctx)
        q.attn_decode(d_qn, d_qg, kc, vc, d_o, None, None, pos, T, SCALE, NQH, NKVH, n_ctx)
        h_o.copy_(d_o, non_blocking=True)
    graphs = []
    for i in range(NBUF):
        body(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            body(i)
        graphs.append(g)

    def gstep(i):
        graphs[i % NBUF].replay()
        torch.cuda.current_stream().synchronize()
    ms = time_steps(gstep, steps, warmup, dist)
    h2d = h_in.numel() * 4
    return {"value": world * kv_bytes(NKVH, n) / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": h_o.numel() * 4,
            "eager_ms_per_step": ms_eager, "eager_value": world * kv_bytes(NKVH, n) / (ms_eager * 1e-3) / 1e9,
            "what": "every step: pinned host q/gate/new K,V rows -> device (one copy), kv_append, attn_decode, result -> "
                    "pinned host, synchronise; the step is captured in a CUDA graph as the reference's engine does "
                    "(value), and also issued call by call (eager_*)"}


def strong_scaling(q, dist, rank, world, n, steps, warmup):
    """One sequence over all ranks: KV-head groups up to 4 ranks, then KV length with the NCCL
    gather of (m, l, O) partials and the log-sum-exp merge on every rank."""
    from qwen27_engine_b200 import shard
    sh = shard.plan_single_sequence(rank, world, NKVH)
    group = shard.peer_group(sh)
    lo, hi = shard.kv_slice(n, sh.z, sh.nz)
    nk, nq = sh.n_kv_heads, sh.n_kv_heads * GQA
    n_ctx = hi - lo + 64
    caches = [torch_caches(nk, hi - lo, n_ctx, 5000 + 10 * rank + i) for i in range(NBUF)]
    g = torch.Generator(device="cuda")
    g.manual_seed(77 + sh.kv_head0)
    qn = torch.randn((T, nq, AD), generator=g, device="cuda")
    qg = torch.randn((T, nq, 512), generator=g, device="cuda")
    o = torch.empty((T, nq, AD), device="cuda")
    pos = torch.tensor([n - T], dtype=torch.int32, device="cuda")
    part = torch.empty((T * nq, 258), device="cuda")

    def step(i):
        kc, vc = caches[i % NBUF]
        if sh.nz == 1:
            q.attn_decode(qn, qg, kc, vc, o, None, None, pos, T, SCALE, nq, nk, n_ctx)
        else:
            q.attn_decode_partial(qn, kc, vc, part, pos, T, SCALE, nq, nk, n_ctx, lo, hi - lo)
            allp = shard.gather_partials(part, sh, group)
            q.lse_merge(allp, sh.nz, T * nq * 258, T * nq, qg, o)

    # no exchange: graph-timed like the headline; with the NCCL all-gather the steps are issued one by one
    ms = time_graph_steps(step, steps, warmup, dist) if sh.nz == 1 else time_steps(step, steps, warmup, dist)
    out = {"what": "one 150k sequence sharded over %d GPUs: %d KV head(s) per GPU x %d KV-length slice(s)%s" % (
               world, nk, sh.nz, ", NCCL all-gather of partials + LSE merge" if sh.nz > 1 else ", no exchange"),
           "us_per_step": ms * 1e3, "value": kv_bytes(NKVH, n) / (ms * 1e-3) / 1e9, "unit": "GB/s", "scaling": "strong",
           "timing": "CUDA graphs of 20 steps" if sh.nz == 1 else "steps issued one by one"}
    if sh.nz == 1:
        ms_e = time_steps(step, steps, warmup, dist)
        out["eager_us_per_step"] = ms_e * 1e3
    if sh.nz > 1 and os.environ.get("Q27B_P2P_MERGE", "1") != "0":
        # the same exchange over peer memory: the merge kernel of each slice stores its rows (tagged words) into
        # the other ranks' exchange buffers, waits for theirs in its own buffer and writes the output
        ok = torch.ones(1, device="cuda")
        try:  # raises on every rank of the head group or on none
            own, peers = shard.make_exchange(q, sh, group, T * nq)
        except RuntimeError as e:  # report, do not hide: the NCCL figure above stands
            out["p2p_error"] = str(e)
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)  # every rank of the job takes the same path
        if ok.item() == 0:
            return out
        o2 = torch.empty((T, nq, AD), device="cuda")

        def step_p2p(i):  # split-K kernel, then one kernel that pushes this rank's slice and merges all of them
            kc, vc = caches[i % NBUF]
            q.attn_decode_exchange(qn, qg, kc, vc, o2, pos, T, SCALE, nq, nk, n_ctx, lo, hi - lo, peers, sh.z)
        step(0)
        step_p2p(0)
        torch.cuda.synchronize()
        same = bool(torch.equal(o, o2))
        ms2_e = time_steps(step_p2p, steps, warmup, dist)
        ms2 = time_graph_steps(step_p2p, steps, warmup, dist)  # the whole step of every rank replayed from a CUDA graph
        assert q.device_status() == 0, "a kernel reported a device-side problem"
        out["nccl_us_per_step"] = out["us_per_step"]
        out["eager_us_per_step"] = ms2_e * 1e3
        out["timing"] = "CUDA graphs of 20 steps per rank (nccl_us_per_step: steps issued one by one)"
        out["us_per_step"] = ms2 * 1e3
        out["value"] = kv_bytes(NKVH, n) / (ms2 * 1e-3) / 1e9
        out["what"] = out["what"].replace("NCCL all-gather of partials + LSE merge",
                                          "the merge kernel stores its slice into the peers' exchange buffers over NVLink, waits for "
                                          "theirs and writes the output (nccl_us_per_step: the same with an NCCL all-gather)")
        out["p2p_equals_nccl_bitwise"] = same
    return out


def sum_norm_scaling(q, dist, rank, world, steps, warmup):
    """The step after the attention output projection: x [4][5120] += the sum of the ranks' partial rows,
    RMSNorm, q8_1 (the reference's sum_norm_q8 with its two-card exchange). Peer-memory form (each rank
    stores its rows as tagged words into every rank's exchange buffer and waits for the others') against an
    NCCL all-reduce followed by the single-GPU kernel."""
    from qwen27_engine_b200 import shard
    rows, n, eps = T, 5120, 1e-6
    g = torch.Generator(device="cuda")
    g.manual_seed(4242)
    x0 = torch.randn((rows, n), generator=g, device="cuda")
    w = 1.0 + 0.1 * torch.randn((n,), generator=g, device="cuda")
    g.manual_seed(4243 + rank)
    partial = 0.3 * torch.randn((rows, n), generator=g, device="cuda")
    x = x0.clone()
    buf = torch.empty_like(partial)
    xq = torch.zeros((rows, n), dtype=torch.int8, device="cuda")
    xd = torch.zeros((rows * n // 32,), dtype=torch.float32, device="cuda")

    def step_nccl(i):
        buf.copy_(partial)
        dist.all_reduce(buf)
        q.sum_norm_q8(x, buf, n, rows, w, eps, None, xq, xd)

    ms_nccl = time_steps(step_nccl, steps, warmup, dist)
    x.copy_(x0)
    step_nccl(0)
    x_ref = x.clone()
    own, peers = shard.make_sum_exchange(q, rank, world, rows, n)
    xq2, xd2 = torch.zeros_like(xq), torch.zeros_like(xd)

    def step_p2p(i):
        q.sum_exchange_norm_q8(x, partial, n, rows, rank, peers, w, eps, None, xq2, xd2)  # push + waiting norm, one kernel

    x.copy_(x0)
    step_p2p(0)
    torch.cuda.synchronize()
    bad = torch.tensor([float(q.device_status())], device="cuda")
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)  # every rank takes the same path
    if bad.item() != 0:  # e.g. a wait that ran out: do not time hundreds of bounded waits
        return {"error": "device status %d after the first peer-memory step" % int(bad.item()), "nccl_us_per_step": ms_nccl * 1e3}
    diff = float((x - x_ref).abs().max().item())
    ms_e = time_steps(step_p2p, steps, warmup, dist)
    ms = time_graph_steps(step_p2p, steps, warmup, dist)
    assert q.device_status() == 0, "a kernel reported a device-side problem"
    return {"timing": "CUDA graphs of 20 steps per rank (eager_us_per_step, nccl_us_per_step: issued one by one)",
            "eager_us_per_step": ms_e * 1e3,
            "what": "x[4][5120] += sum over %d GPUs of their partial rows, RMSNorm, q8_1: rows stored into every rank's exchange "
                    "buffer over NVLink + waiting norm kernel (nccl_us_per_step: NCCL all-reduce + the single-GPU kernel)" % world,
            "us_per_step": ms * 1e3, "nccl_us_per_step": ms_nccl * 1e3, "max_abs_diff_vs_nccl_sum": diff,
            "bytes_pushed_per_rank": rows * n * 4 * world}


def batched_paged(q, rank, world, dist=None, n_seqs=64, max_len=131072):
    """Config 5: 64 sequences, 4 query tokens each, lengths ~U{1,024..131,072} (seed 1005), q8_0 KV in
    256-token pages behind a random page table; sequences sharded over the ranks (greedy by length,
    no exchange). The pool holds random int8 values and scales of the size q8_0 gives N(0,1) rows:
    timing does not depend on the values. One step = one q27b_attn_decode_paged call per rank."""
    from qwen27_engine_b200 import shard
    PAGE, B_ALL = 256, n_seqs
    rng = np.random.default_rng(1005)
    lengths = rng.integers(1024, max_len + 1, size=B_ALL)
    mine = shard.shard_sequences(lengths, world)[rank]
    lens = [int(lengths[i]) for i in mine]
    B = len(lens)
    max_pages = (max_len + PAGE - 1) // PAGE
    need = [(n + PAGE - 1) // PAGE for n in lens]
    n_pages = sum(need)
    perm = rng.permutation(n_pages).astype(np.int32)
    table = np.full((B, max_pages), -1, np.int32)
    at = 0
    for b in range(B):
        table[b, :need[b]] = perm[at:at + need[b]]
        at += need[b]
    g = torch.Generator(device="cuda")
    g.manual_seed(1005 + rank)
    nval = n_pages * NKVH * PAGE * AD
    nsc = n_pages * NKVH * PAGE * 8

    def pool():
        buf = torch.empty(q.kv_pool_bytes(NKVH, n_pages), dtype=torch.uint8, device="cuda")
        buf[:nval] = torch.randint(0, 256, (nval,), generator=g, device="cuda", dtype=torch.uint8)
        sc = (torch.rand((nsc,), generator=g, device="cuda") * 0.01 + 0.02).to(torch.float16)
        buf[nval:nval + 2 * nsc] = sc.view(torch.uint8)
        return buf
    kpool, vpool = pool(), pool()
    qn = torch.randn((B, T, NQH, AD), generator=g, device="cuda")
    qg = torch.randn((B, T, NQH, 512), generator=g, device="cuda")
    o = torch.empty((B, T, NQH, AD), device="cuda")
    d_table = torch.from_numpy(table).cuda()
    d_len = torch.tensor(lens, dtype=torch.int32, device="cuda")

    def step(i):
        q.attn_decode_paged(qn, qg, kpool, vpool, d_table, d_len, o, B, T, SCALE, NQH, NKVH, n_pages, max_pages, max(lens))
    cool_down(1.0)
    ms_e = time_steps(step, 10, 3, dist)
    cool_down(1.0)
    ms = time_graph_steps(step, 20, 3, dist, calls=5)
    assert q.device_status() == 0, "a kernel reported a device-side problem"
    total = float(sum(2.0 * NKVH * int(n) * 272 for n in lengths))
    return {"what": "%d sequences x 4 query tokens, lengths U{1024..%d} (seed 1005), 256-token pages, random page "
                    "table; %d sequence(s) on rank 0 of %d" % (n_seqs, max_len, B, world),
            "positions_total": int(lengths.sum()), "kv_bytes_total": total, "ms_per_step": ms, "eager_ms_per_step": ms_e,
            "timing": "CUDA graphs of 5 steps, 4 replays timed",
            "value": total / (ms * 1e-3) / 1e9, "unit": "GB/s", "scaling": "strong (sequences sharded by KV length)"}


def kv_wire_bench(q):
    """Rows of one 131,072-position sequence (4 KV heads) from the page pool into the reference's host
    layout on the device and back (q27b_kv_pages_to_wire / q27b_kv_wire_to_pages): a copy kernel,
    272 B read + 272 B written per (head, position)."""
    PAGE, n = 256, 131072
    need = n // PAGE
    n_pages = need + 8
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    pool = torch.randint(0, 256, (q.kv_pool_bytes(NKVH, n_pages),), generator=g, device="cuda", dtype=torch.uint8)
    table = torch.randperm(n_pages, generator=g, device="cuda")[:need].to(torch.int32)
    wire = torch.empty(q.kv_wire_bytes(NKVH, n), dtype=torch.uint8, device="cuda")
    moved = 2.0 * NKVH * n * 272
    us_out = graph_us(lambda i: q.kv_pages_to_wire(pool, table, wire, NKVH, n_pages, 0, n))
    us_in = graph_us(lambda i: q.kv_wire_to_pages(pool, table, wire, NKVH, n_pages, 0, n))
    pk, _ = peaks()
    return {"what": "131,072 positions x 4 KV heads, q8_0, page pool <-> reference host layout (device side)",
            "bytes_moved": moved, "pages_to_wire_us": us_out, "wire_to_pages_us": us_in,
            "pages_to_wire_gbs": moved / (us_out * 1e-6) / 1e9, "wire_to_pages_gbs": moved / (us_in * 1e-6) / 1e9,
            "frac_of_measured_copy_peak": moved / (us_out * 1e-6) / 1e9 / pk["hbm_gbs"]}


def extras(q, caches, qn, qg, o, n_ctx):
    """Other depths of the metric, the prefill TOPS, the batched paged decode and the reference's kernels."""
    out = {"decode_us": {}, "prefill": {}}
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    # the other depths of the metric, timed as the reference times them (tools/bench_attn.cu:131-147):
    # 20 calls captured in one CUDA graph, replayed 5 times, so that host launch time does not count
    for depth in (1024, 30000, 100000, 150000):
        pos.fill_(depth - T)

        def step(i):
            kc, vc = caches[i % NBUF]
            q.attn_decode(qn, qg, kc, vc, o, None, None, pos, T, SCALE, NQH, NKVH, n_ctx)
        us = graph_us(step)
        out["decode_us"][str(depth)] = {"us": us, "gbs": kv_bytes(NKVH, depth) / (us * 1e-6) / 1e9}
    # spec-verify decode at 32,768 positions with the q8_0 and with the f16 KV cache
    n2 = 32768
    pos.fill_(n2 - T)
    f16c = [torch_caches(NKVH, n2, n2 + 64, 2002 + i, q8=False) for i in range(NBUF)]
    us_q8 = graph_us(lambda i: q.attn_decode(qn, qg, caches[i % NBUF][0], caches[i % NBUF][1], o, None, None, pos, T,
                                             SCALE, NQH, NKVH, n_ctx))
    us_f16 = graph_us(lambda i: q.attn_decode(qn, qg, f16c[i % NBUF][0], f16c[i % NBUF][1], o, None, None, pos, T,
                                              SCALE, NQH, NKVH, n2 + 64, False))
    out["spec_verify_32768"] = {"q8_0": {"us": us_q8, "gbs": kv_bytes(NKVH, n2) / (us_q8 * 1e-6) / 1e9},
                                "f16": {"us": us_f16, "gbs": 2.0 * NKVH * n2 * 512 / (us_f16 * 1e-6) / 1e9}}
    del f16c
    # prefill chunk: 2048 new tokens on a prefix of P tokens (int8 Q K^T, f16 P V); ops as the reference counts them
    M = 2048
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    pqn = torch.randn((M, NQH, AD), generator=g, device="cuda")
    pqg = torch.randn((M, NQH, 512), generator=g, device="cuda")
    po = torch.empty((M, NQH, AD), device="cuda")
    kc, vc = caches[0]
    for P in (0, 32768, 148000):
        pos.fill_(P)
        ops = NQH * 1024.0 * (M * P + M * (M + 1) / 2)
        try:
            ms = time_steps(lambda i: q.attn_prefill(pqn, pqg, kc, vc, po, pos, M, SCALE, NQH, NKVH, n_ctx, True, P), 3, 3)
            out["prefill"][str(P)] = {"ms": ms, "tops": ops / (ms * 1e-3) / 1e12}
        except Exception as e:  # report, do not hide
            out["prefill"][str(P)] = {"error": str(e)}
    # the same chunk and cache through the f16-QK kernel (the reference's Q27_ATTN_I8=0: K and V dequantised to f16)
    out["prefill_f16_qk_on_q8_0"] = {}
    try:
        q.set_prefill_kernel(2)
        for P in (0, 32768, 148000):
            pos.fill_(P)
            ops = NQH * 1024.0 * (M * P + M * (M + 1) / 2)
            ms = time_steps(lambda i: q.attn_prefill(pqn, pqg, kc, vc, po, pos, M, SCALE, NQH, NKVH, n_ctx, True, P), 3, 3)
            out["prefill_f16_qk_on_q8_0"][str(P)] = {"ms": ms, "tops": ops / (ms * 1e-3) / 1e12}
    except Exception as e:  # report, do not hide
        out["prefill_f16_qk_on_q8_0"]["error"] = str(e)
    finally:
        q.set_prefill_kernel(0)
    # the same chunk on an f16 KV cache (f16 Q K^T and P V, no per-block scale arithmetic)
    out["prefill_f16_cache"] = {}
    try:
        Pmax = 148000
        f16c = torch_caches(NKVH, Pmax + M, Pmax + M + 64, 3002, q8=False)
        for P in (0, 32768, Pmax):
            pos.fill_(P)
            ops = NQH * 1024.0 * (M * P + M * (M + 1) / 2)
            ms = time_steps(lambda i: q.attn_prefill(pqn, pqg, f16c[0], f16c[1], po, pos, M, SCALE, NQH, NKVH, Pmax + M + 64, False, P), 3, 3)
            out["prefill_f16_cache"][str(P)] = {"ms": ms, "tflops": ops / (ms * 1e-3) / 1e12}
        del f16c
    except Exception as e:  # report, do not hide
        out["prefill_f16_cache"]["error"] = str(e)
    out["device_status"] = q.device_status()
    try:  # the tensor-pipe denominators, measured in this run
        out["mma_peak"] = {"int8_tops": measure_mma_peak(q, 0), "f16_tflops": measure_mma_peak(q, 1),
                           "what": "tcgen05.mma kind::i8 / kind::f16, 128 x 256 tiles back to back from shared memory, one CTA per SM"}
    except Exception as e:  # report, do not hide
        out["mma_peak"] = {"error": str(e)}
    try:
        out["batched_paged"] = batched_paged(q, 0, 1)
    except Exception as e:  # report, do not hide
        out["batched_paged"] = {"error": str(e)}
    try:
        out["kv_wire"] = kv_wire_bench(q)
    except Exception as e:  # report, do not hide
        out["kv_wire"] = {"error": str(e)}
    try:
        ref = RefLib()
        pos.fill_(N_POS - T)
        ms = time_steps(lambda i: ref.decode(qn, qg, caches[i % NBUF][0], caches[i % NBUF][1], o, pos, T, NQH, NKVH, n_ctx), 100, 5)
        out["reference_kernels_same_gpu"] = {"decode_150k_us": ms * 1e3, "decode_150k_gbs": kv_bytes(NKVH, N_POS) / (ms * 1e-3) / 1e9}
        out["reference_kernels_same_gpu"]["decode_us_graph"] = {}
        for depth in (1024, 30000, 100000, 150000):
            pos.fill_(depth - T)
            us = graph_us(lambda i: ref.decode(qn, qg, caches[i % NBUF][0], caches[i % NBUF][1], o, pos, T, NQH, NKVH, n_ctx))
            out["reference_kernels_same_gpu"]["decode_us_graph"][str(depth)] = us
        for P in (32768,):
            pos.fill_(P)
            ops = NQH * 1024.0 * (M * P + M * (M + 1) / 2)
            ms = time_steps(lambda i: ref.prefill(pqn, pqg, kc, vc, po, pos, M, NQH, NKVH, n_ctx, P), 2, 3)
            out["reference_kernels_same_gpu"]["prefill_%d_tops" % P] = ops / (ms * 1e-3) / 1e12
    except Exception as e:
        out["reference_kernels_same_gpu"] = {"unavailable": str(e)}
    return out


def prefill_mode(q, args, steps, warmup, dist=None, rank=0, world=1):
    """Second half of the metric: one 2048-token prefill chunk on a q8_0 prefix of --prefix tokens
    (int8 Q K^T, f16 P V). One step = one attn_prefill call; ops as the reference counts them
    (tools/bench_attn.cu:104): nqh * 1024 * (M * P + M (M + 1) / 2)."""
    M, P = 2048, args.prefix
    n_ctx = P + M + 8
    q8 = args.kv != "f16"
    use_ref = args.impl == "reference"
    ref = RefLib() if use_ref else None
    # N > 1: the one chunk is shared out (strong scaling): KV-head groups, then query-token ranges within a
    # group (shard.plan_prefill); every rank holds the K and V rows of its heads, nothing is exchanged
    if use_ref:  # one GPU, the whole chunk in one call
        import collections
        plan = collections.namedtuple("Plan", "kv_head0 n_kv_heads ranges")(0, NKVH, [(0, M)])
    else:
        from qwen27_engine_b200 import shard
        plan = shard.plan_prefill(rank, world, M, P, NKVH)
    nkvh, nqh = plan.n_kv_heads, plan.n_kv_heads * GQA
    kc, vc = torch_caches(nkvh, P + M, n_ctx, 1002 + plan.kv_head0, q8=q8)
    g = torch.Generator(device="cuda")
    g.manual_seed(3 + plan.kv_head0)
    qn = torch.randn((M, nqh, AD), generator=g, device="cuda")
    qg = torch.randn((M, nqh, 512), generator=g, device="cuda")
    o = torch.empty((M, nqh, AD), device="cuda")
    calls = [(a, b, torch.tensor([P + a], dtype=torch.int32, device="cuda")) for a, b in plan.ranges]

    def step(i):
        for a, b, pos in calls:
            if use_ref:
                ref.prefill(qn[a:b], qg[a:b], kc, vc, o[a:b], pos, b - a, nqh, nkvh, n_ctx, P + a, q8)
            else:
                q.attn_prefill(qn[a:b], qg[a:b], kc, vc, o[a:b], pos, b - a, SCALE, nqh, nkvh, n_ctx, q8, P + a)

    sampler = ClockSampler(env_int("LOCAL_RANK", 0))
    sampler.start()
    ms = time_steps(step, steps, warmup, dist)
    clocks = sampler.stop()
    if rank != 0:
        return
    ops = NQH * 1024.0 * (M * P + M * (M + 1) / 2)
    tops = ops / (ms * 1e-3) / 1e12
    pk, pk_kind = peaks()
    f16 = pk["bf16_tflops_sustained"]
    sm_mhz = clocks.get("sm_mhz") or 1965.0
    line = {"metric": "int8 prefill-attn TOPS (2048-token chunk, 24q/4kv heads, head dim 256, q8_0 prefix)",
            "value": tops, "unit": "TOPS", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "s8 x s8 -> s32 (QK), f16 -> f32 (PV)",
            "data": "synthetic", "config": {"workload": "prefill chunk M=2048 on a q8_0 prefix of %d tokens" % P},
            "gpu_launches": steps * len(calls), "clocks": clocks}
    if use_ref:
        i8_peak, f16_peak, peak_kind = 2 * f16, f16, "2 x %s bf16 GEMM rate (sustained) as the int8 peak" % pk_kind
    else:
        # the denominators measured on this GPU, in this process: tcgen05.mma kind::i8 and kind::f16 back to back
        i8_peak, f16_peak = measure_mma_peak(q, 0), measure_mma_peak(q, 1)
        peak_kind = "tcgen05.mma kind::i8 microbenchmark of this run (kind::f16: %.0f TFLOP/s; %s bf16 GEMM: %.0f sustained)" % (
            f16_peak, pk_kind, f16)
    # half of the ops run on the int8 pipe, half on the f16 pipe
    t_min_ms = (ops / 2 / (i8_peak * 1e12) + ops / 2 / (f16_peak * 1e12)) * 1e3
    # the exact per-block numerics cost ~22 SIMT instructions per score (8 blocks x (int -> float, scale
    # product, FMA) + softmax): what 128 lanes per SM can issue at the sampled clock, as TOPS of the same ops
    alu_bound_tops = 1024.0 * 128 * n_sm_of_device() * sm_mhz * 1e6 / 22.0 / 1e12 * world
    line["roofline"] = {"bound": "tensor", "achieved": tops, "peak": i8_peak * world, "unit": "TOP/s",
                        "frac": tops / (i8_peak * world), "peak_kind": peak_kind, "int8_tops_measured": i8_peak,
                        "f16_tflops_measured": f16_peak, "frac_of_mixed_int8_f16_bound": t_min_ms / ms / world,
                        "fp32_alu_bound_tops": alu_bound_tops, "frac_of_fp32_alu_bound": tops / alu_bound_tops,
                        "traffic": None}
    if not use_ref and world == 1:
        line["e2e"] = prefill_e2e(q, kc, vc, M, P, n_ctx, q8, steps, warmup)
        if q8:
            line["cpu_baseline"] = prefill_cpu_baseline(kc, vc, qn, qg, M, P, n_ctx)
    if not q8:  # all of the ops on the f16 pipe
        line["metric"] = "f16 prefill-attn TFLOPS (2048-token chunk, 24q/4kv heads, head dim 256, f16 prefix)"
        line["unit"] = "TFLOP/s"
        line["dtype"] = "f16 -> f32 (QK and PV)"
        line["config"] = {"workload": "prefill chunk M=2048 on an f16 prefix of %d tokens" % P}
        line["roofline"] = {"bound": "tensor", "achieved": tops, "peak": f16_peak * world, "unit": "TFLOP/s",
                            "frac": tops / (f16_peak * world), "peak_kind": peak_kind, "traffic": None}
    if q8 and os.environ.get("Q27_ATTN_I8", "1")[:1] == "0":  # the library reads the same switch
        line["metric"] = "f16-QK prefill-attn TOPS on a q8_0 prefix (Q27_ATTN_I8=0: K and V dequantised to f16; 2048-token chunk, 24q/4kv heads, head dim 256)"
        line["dtype"] = "f16 -> f32 (QK and PV), q8_0 K/V dequantised on the way"
        line["roofline"] = {"bound": "tensor", "achieved": tops, "peak": f16_peak * world, "unit": "TFLOP/s",
                            "frac": tops / (f16_peak * world), "peak_kind": peak_kind, "traffic": None}
    if world > 1:
        line["config"]["sharding"] = "KV-head groups x %d query-token slices per group, no exchange; rank 0: heads %d..%d, tokens %s" % (
            max(1, world // NKVH), plan.kv_head0, plan.kv_head0 + nkvh - 1, list(plan.ranges))
    if use_ref:
        line["impl"] = "reference"
    if not use_ref:
        assert q.device_status() == 0
    print(json.dumps(line))


def n_sm_of_device():
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def prefill_e2e(q, kc, vc, M, P, n_ctx, q8, steps, warmup):
    """The prefill chunk through the operator API with host buffers: every step copies the chunk's query +
    gate rows and its new K and V rows from pinned host memory, appends the rows to the cache, runs
    attn_prefill and copies the result back to pinned host memory."""
    sizes = [M * NQH * AD, M * NQH * 512, M * NKVH * AD, M * NKVH * AD]
    h_in = torch.randn((sum(sizes),)).pin_memory()
    d_in = torch.empty((sum(sizes),), device="cuda")
    o0, o1, o2 = sizes[0], sizes[0] + sizes[1], sizes[0] + sizes[1] + sizes[2]
    d_qn, d_qg = d_in[:o0].view(M, NQH, AD), d_in[o0:o1].view(M, NQH, 512)
    d_k, d_v = d_in[o1:o2].view(M, NKVH, AD), d_in[o2:].view(M, NKVH, AD)
    h_o = torch.empty((M, NQH, AD)).pin_memory()
    d_o = torch.empty((M, NQH, AD), device="cuda")
    pos = torch.tensor([P], dtype=torch.int32, device="cuda")

    def step(i):
        d_in.copy_(h_in, non_blocking=True)
        q.kv_append(d_k, d_v, kc, vc, pos, M, NKVH, n_ctx, q8)
        q.attn_prefill(d_qn, d_qg, kc, vc, d_o, pos, M, SCALE, NQH, NKVH, n_ctx, q8, P)
        h_o.copy_(d_o, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    ms = time_steps(step, steps, warmup)
    ops = NQH * 1024.0 * (M * P + M * (M + 1) / 2)
    return {"value": ops / (ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": ms, "h2d_bytes_per_step": h_in.numel() * 4,
            "d2h_bytes_per_step": h_o.numel() * 4,
            "what": "every step: pinned host q|gate and new K, V rows of the chunk -> device, kv_append, attn_prefill, "
                    "result -> pinned host, synchronise"}


def prefill_cpu_baseline(kc, vc, qn, qg, M, P, n_ctx):
    """The CPU oracle's int8-QK prefill on a subset of the chunk's query tokens (the first, a middle and the
    last 8 tokens, all 24 heads, their whole causal range), timed on the host cores; the rate is per op of
    what it computed, as for the GPU figure."""
    import oracle
    hk, hv = kc.cpu().numpy(), vc.cpu().numpy()
    hq, hg = qn.cpu().numpy(), qg.cpu().numpy()
    ranges = [(0, 8), (M // 2 - 4, M // 2 + 4), (M - 8, M)]
    oracle.attn_prefill_i8(hq, hg, hk, hv, P, SCALE, NKVH, n_ctx, 0, 1)  # warm
    t0 = time.perf_counter()
    for a, b in ranges:
        oracle.attn_prefill_i8(hq, hg, hk, hv, P, SCALE, NKVH, n_ctx, a, b)
    dt = time.perf_counter() - t0
    ops = sum(NQH * 1024.0 * (P + t + 1) for a, b in ranges for t in range(a, b))
    return {"value": ops / dt / 1e12, "unit": "TOPS", "cores": oracle.num_threads(), "kind": "port",
            "sample": "%d of the %d query tokens (tokens %s, all heads, whole causal range): %.2f s on the host cores; "
                      "the whole chunk would take %.0f s at that rate" % (
                          sum(b - a for a, b in ranges), M, ranges, dt, NQH * 1024.0 * (M * P + M * (M + 1) / 2) / (ops / dt))}


def run_reference(args, line, caches, qn, qg, o, pos, n, n_ctx, steps, warmup):
    line["impl"] = "reference"
    use_cpu = args.ref_cpu
    ref = None
    if not use_cpu:
        try:
            ref = RefLib()
        except OSError:
            use_cpu = True
    if use_cpu:
        cb = cpu_baseline(n)
        line.update({"value": cb["value"], "ms_per_step": cb["ms_per_step"], "cpu_baseline": cb,
                     "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                     "reference_arm": "CPU oracle (C++/OpenMP port of the reference numerics)"})
        print(json.dumps(line))
        return

    def step(i):
        kc, vc = caches[i % NBUF]
        ref.decode(qn, qg, kc, vc, o, pos, T, NQH, NKVH, n_ctx)

    cool_down()  # as in the other arm
    sampler = ClockSampler(env_int("LOCAL_RANK", 0))
    sampler.start()
    ms = time_graph_steps(step, steps, warmup)
    line["clocks"] = sampler.stop()
    ms_eager = time_steps(step, steps, warmup)
    v = kv_bytes(NKVH, n) / (ms * 1e-3) / 1e9
    line.update({"value": v, "ms_per_step": ms, "us_per_step": ms * 1e3, "gpu_launches": 2 * steps,
                 "eager_ms_per_step": ms_eager, "eager_value": kv_bytes(NKVH, n) / (ms_eager * 1e-3) / 1e9,
                 "reference_arm": "the reference's own CUDA kernels (src/attn.cu, mma.sync + cp.async) compiled for "
                                  "sm_100a and called through q27::attn_decode on the same GPU, timed the same way "
                                  "(CUDA graphs of 20 calls); the reference has no CPU implementation of this path; "
                                  "this process loads oracle/_ref/libq27ref.so only",
                 "cpu_baseline": {"value": v, "unit": "GB/s", "cores": 0, "kind": "reference",
                                  "sample": "%d full steps on the GPU (not host cores)" % steps},
                 "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(line))


if __name__ == "__main__":
    main()
