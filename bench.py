#!/usr/bin/env python
"""Benchmark of the GEMM hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one GEMM call through the library's C ABI on synthetic seeded operands:

  N = 1  HGEMM NT, M=N=K=8192, alpha=1, beta=0.5, A/B/C ~ N(0, 0.5^2) rounded to fp16
         (the configuration the headline metric is quoted on).  The same line also carries,
         each timed on the device outside the headline's timed region: `sgemm` (fp32 8192^3 NN on
         the CUDA-core FFMA kernel and on the 3xTF32 tensor-core kernel, 4096^3 in all four
         transpose modes, the ragged padded configuration), `config5_1gpu` (HGEMM NN 32768^3 on
         this one GPU: the T1 of the multi-GPU curve) and `vendor` (cuBLAS through torch on the
         identical operands, run after ours).
  N > 1  HGEMM NN, M=N=K=32768, alpha=1, beta=0, U[-1,1): B and C split into N column
         blocks, A replicated, one rank per GPU, no communication in the contraction: `value`.
         `exchange` then times the same step followed by the one optional exchange -- every rank
         ends with the whole C -- three ways (one multimem store per piece through NVSwitch; one
         store per peer; NCCL all-gather through mmbo_gemm_f16_sharded), each checked against
         binary64 dot products of elements RECEIVED from another rank.

`value` is whole-job TFLOP/s (2*M*N*K per step over the slowest rank's device time) with
operands resident in HBM; `e2e` is the same metric with pinned host operands copied to
the device and the result copied back inside the timed region (N > 1: each rank uploads 1/N
of A and the GPUs exchange the shares over NVLink).  `--impl reference` times the CPU
restatement of the reference's arithmetic (oracle/) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "hgemm_tflops"
UNIT = "TFLOP/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the N=1 workload, from the ncu capture
# summarised in profiles/ (a profiler figure cannot be taken inside this run)
TRAFFIC_8192_NT = {  # by kernel id of the fp16 table
    6: {"bytes": 1.327e9, "source": "profiles/hgemm_tcgen05_MT512x256x64_CG2_8192cubed.md"},
    3: {"bytes": 1.805e9, "source": "profiles/hgemm_tcgen05_MT256x256x64_CG2_8192cubed.md"},
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--kernel", type=int, default=-1, help="force a kernel id of the fp16 table")
    ap.add_argument("--size", type=int, default=0, help="override M=N=K (debugging / profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline step (no sgemm / config5_1gpu / vendor / exchange legs): profiling runs")
    return ap.parse_args()


def workload(n_gpus: int, size: int):
    if n_gpus == 1:
        s = size or 8192
        return dict(name=f"HGEMM NT {s}^3 alpha=1 beta=0.5 normal(0,0.5) fp16", ta=False, tb=True, m=s, n=s,
                    k=s, alpha=1.0, beta=0.5, dist=1, scale=0.5)
    return config5(size)


def config5(size: int = 0):
    s = size or 32768
    return dict(name=f"HGEMM NN {s}^3 alpha=1 beta=0 uniform[-1,1) fp16, B/C column blocks", ta=False,
                tb=False, m=s, n=s, k=s, alpha=1.0, beta=0.0, dist=0, scale=1.0)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(burst=float(d["bf16_tflops"]), sustained=float(d["bf16_tflops_sustained"]),
                    hbm=float(d["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


# ------------------------------------------------------------------ clocks ------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------ CPU baseline ------
def cpu_panel_time(O, w, pm: int, pn: int, repeats: int = 1) -> float:
    """Seconds for one pm x pn x K panel of the workload on all host cores."""
    k = w["k"]
    ta, tb = w["ta"], w["tb"]
    ra, rb = (k if ta else pm), (pn if tb else k)
    ca, cb = (pm if ta else k), (k if tb else pn)
    A = O.fill("f16", ra, ca, ra, mat=O.MAT_A, dist=w["dist"], scale=w["scale"])
    B = O.fill("f16", rb, cb, rb, mat=O.MAT_B, dist=w["dist"], scale=w["scale"])
    C = O.fill("f16", pm, pn, pm, mat=O.MAT_C, dist=w["dist"], scale=w["scale"])
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.gemm("f16", ta, tb, pm, pn, k, w["alpha"], A, ra, B, rb, w["beta"], C, pm)
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_baseline(w, target_s: float = 12.0):
    from oracle import oracle as O
    O.set_num_threads(0)  # every host core, even when the launcher exported OMP_NUM_THREADS=1
    t = cpu_panel_time(O, w, 512, 512)
    rate = 2.0 * 512 * 512 * w["k"] / t  # flop/s
    # panel edge for ~target_s of work, multiple of 256, within the problem
    edge = int((rate * target_s / (2.0 * w["k"])) ** 0.5) // 256 * 256
    edge = max(512, min(edge, w["m"], w["n"], 8192))
    t = cpu_panel_time(O, w, edge, edge)
    tflops = 2.0 * edge * edge * w["k"] / t / 1e12
    full_s = 2.0 * w["m"] * w["n"] * w["k"] / (tflops * 1e12)
    return {"value": tflops, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
            "sample": f"{edge}x{edge}x{w['k']} panel of the workload, {t:.2f} s measured; "
                      f"full problem extrapolated to {full_s:.0f} s"}


def run_reference(args, rank: int):
    """CPU arm: the oracle (restatement of the reference's arithmetic) on host cores."""
    if rank != 0:
        return
    from oracle import oracle as O
    O.set_num_threads(0)  # every host core, even when the launcher exported OMP_NUM_THREADS=1
    w = workload(args.gpus, args.size)
    t_probe = cpu_panel_time(O, w, 512, 512)
    rate = 2.0 * 512 * 512 * w["k"] / t_probe
    per_step_s = max(0.05, min(1.0, 120.0 / max(1, args.steps + args.warmup)))
    edge = int((rate * per_step_s / (2.0 * w["k"])) ** 0.5) // 128 * 128
    edge = max(256, min(edge, w["m"], w["n"]))
    for _ in range(args.warmup):
        cpu_panel_time(O, w, edge, edge)
    times = [cpu_panel_time(O, w, edge, edge) for _ in range(args.steps)]  # GEMM time only
    mean_t = sum(times) / len(times)
    val = 2.0 * edge * edge * w["k"] / mean_t / 1e12
    line = {
        "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": mean_t * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "impl": "reference",
        "config": {"workload": w["name"], "m": w["m"], "n": w["n"], "k": w["k"],
                   "panel": [edge, edge, w["k"]], "l2": "inputs larger than L2 (126 MB)", "accumulate": "fp64"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                         "sample": f"each step = one {edge}x{edge}x{w['k']} panel of the workload, "
                                   "fp64 accumulation, all host threads"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ helpers (GPU arm) --
def shapes(w, ncols):
    """(rows A, rows B, cols A, cols B) of the stored operands of a rank that owns ncols columns."""
    m, k, ta, tb = w["m"], w["k"], w["ta"], w["tb"]
    return (k if ta else m), (ncols if tb else k), (m if ta else k), (k if tb else ncols)


def make_operands(torch, mm, w, col0, ncols, want_c=True):
    m, n, k, tb = w["m"], w["n"], w["k"], w["tb"]
    ra, rb, ca, cb = shapes(w, ncols)
    A = torch.empty((ca, ra), dtype=torch.float16, device="cuda")
    B = torch.empty((cb, rb), dtype=torch.float16, device="cuda")
    mm.fill("f16", A, ra, ca, ra, mat=0, dist=w["dist"], scale=w["scale"])
    if tb:   # B stored n x k: the block is a row window
        mm.fill("f16", B, rb, cb, rb, mat=1, dist=w["dist"], scale=w["scale"], row0=col0, total_rows=n)
    else:    # B stored k x n: the block is a column window
        mm.fill("f16", B, rb, cb, rb, mat=1, dist=w["dist"], scale=w["scale"], col0=col0, total_rows=k)
    C = None
    if want_c:
        C = torch.empty((ncols, m), dtype=torch.float16, device="cuda")
        fill_c(mm, w, C, col0, ncols)
    return A, B, C


def fill_c(mm, w, C, col0, ncols):
    mm.fill("f16", C, w["m"], ncols, w["m"], mat=2, dist=w["dist"], scale=w["scale"], col0=col0, total_rows=w["m"])


def sampled_rel_err(O, w, got_fn, col_lo, col_hi, nsamp=48, seed=7):
    """Relative error over `nsamp` elements C(i, j), j in [col_lo, col_hi) (global column indices), of ONE
    application of the GEMM to freshly generated operands, against binary64 dot products of the same seeded
    operand values (the oracle's generator).  got_fn(rows, cols) returns the computed values."""
    import numpy as np
    rng = np.random.default_rng(seed)
    m, n, k, ta, tb = w["m"], w["n"], w["k"], w["ta"], w["tb"]
    rows = rng.integers(0, m, nsamp)
    cols = rng.integers(col_lo, col_hi, nsamp)
    want = np.empty(nsamp)
    for t in range(nsamp):
        i, j = int(rows[t]), int(cols[t])
        if ta:   # A stored k x m
            a = O.fill("f16", k, 1, k, mat=0, dist=w["dist"], scale=w["scale"], col0=i, total_rows=k)
        else:    # A stored m x k
            a = O.fill("f16", 1, k, 1, mat=0, dist=w["dist"], scale=w["scale"], row0=i, total_rows=m)
        if tb:   # B stored n x k
            b = O.fill("f16", 1, k, 1, mat=1, dist=w["dist"], scale=w["scale"], row0=j, total_rows=n)
        else:    # B stored k x n
            b = O.fill("f16", k, 1, k, mat=1, dist=w["dist"], scale=w["scale"], col0=j, total_rows=k)
        v = w["alpha"] * float(a.astype(np.float64).reshape(-1) @ b.astype(np.float64).reshape(-1))
        if w["beta"] != 0.0:
            c = O.fill("f16", 1, 1, 1, mat=2, dist=w["dist"], scale=w["scale"], row0=i, col0=j, total_rows=m)
            v += w["beta"] * float(c.reshape(-1)[0])
        want[t] = v
    got = np.asarray(got_fn(rows, cols), dtype=np.float64)
    return float(np.linalg.norm(got - want) / np.linalg.norm(want))


def vendor_mm(torch, w, A, B, C):
    """cuBLAS through torch on the identical operands (column-major operands are row-major transposes)."""
    opb_t = B.t() if w["tb"] else B          # (ncols, k)
    opa_t = A.t() if w["ta"] else A          # (k, m)
    if w["beta"] != 0.0:
        C.addmm_(opb_t, opa_t, beta=w["beta"], alpha=w["alpha"])
    else:
        torch.mm(opb_t, opa_t, out=C)


def sgemm_legs(torch, mm, O, steps, sm_max_mhz):
    """fp32 figures of the metric ("% of FP32 peak"): exact fp32 on the CUDA cores and 3xTF32 on the tensor cores."""
    import numpy as np
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    fp32_peak = sms * 128 * 2 * (sm_max_mhz or 1965) * 1e6 / 1e12
    out = {"fp32_ffma_peak_tflops": fp32_peak, "peak_formula": "SMs x 128 lanes x 2 x max SM clock"}

    def run(ta, tb, m, n, k, kid, alpha, beta, pad, iters):
        ra, rb = (k if ta else m), (n if tb else k)
        ca, cb = (m if ta else k), (k if tb else n)
        lda, ldb, ldc = ra + pad, rb + pad, m + pad
        A = torch.empty((ca, lda), dtype=torch.float32, device="cuda")
        B = torch.empty((cb, ldb), dtype=torch.float32, device="cuda")
        C = torch.zeros((n, ldc), dtype=torch.float32, device="cuda")
        mm.fill("f32", A, ra, ca, lda, mat=0)
        mm.fill("f32", B, rb, cb, ldb, mat=1)
        mm.fill("f32", C, m, n, ldc, mat=2)
        C0 = C.clone() if beta != 0.0 else None
        kern = kid if kid >= 0 else mm.select_kernel("f32", ta, tb, m, n, k, A, lda, B, ldb, C, ldc)
        mm.gemm("f32", ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kid)
        # sampled check against binary64 dot products of the device operands
        rng = np.random.default_rng(3)
        rows, cols = rng.integers(0, m, 32), rng.integers(0, n, 32)
        want, got = np.empty(32), np.empty(32)
        for t, (i, j) in enumerate(zip(rows.tolist(), cols.tolist())):
            a = (A[i, :k] if ta else A[:k, i]).double().cpu().numpy()
            b = (B[:k, j] if tb else B[j, :k]).double().cpu().numpy()
            want[t] = alpha * float(a @ b) + (beta * float(C0[j, i]) if beta != 0.0 else 0.0)
            got[t] = float(C[j, i])
        err = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        for _ in range(2):
            mm.gemm("f32", ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kid)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            mm.gemm("f32", ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kid)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        tf = 2.0 * m * n * k / ms / 1e9
        return {"tflops": tf, "ms": ms, "kernel": mm.kernel_name("f32", kern), "rel_err": err}

    s = 8192
    mm.set_option("f32_exact", 1)
    try:
        r = run(False, False, s, s, s, -1, 1.0, 0.0, 0, min(steps, 10))
        r["frac_of_fp32_peak"] = r["tflops"] / fp32_peak
        out["ffma"] = {"workload": f"SGEMM NN {s}^3 alpha=1 beta=0, exact fp32 (FFMA)", **r}
        modes = {}
        for name, (ta, tb) in {"NN": (False, False), "NT": (False, True), "TN": (True, False), "TT": (True, True)}.items():
            q = run(ta, tb, 4096, 4096, 4096, -1, 1.0, 0.0, 0, min(steps, 10))
            modes[name] = {"tflops": q["tflops"], "frac_of_fp32_peak": q["tflops"] / fp32_peak, "kernel": q["kernel"],
                           "rel_err": q["rel_err"]}
        out["ffma_4096_modes"] = modes
        c3 = {}
        for name, (ta, tb) in {"NN": (False, False), "NT": (False, True), "TN": (True, False), "TT": (True, True)}.items():
            q = run(ta, tb, 4095, 4097, 1023, -1, 1.5, -0.25, 3, min(steps, 10))
            c3[name] = {"tflops": q["tflops"], "kernel": q["kernel"], "rel_err": q["rel_err"]}
        out["ffma_config3_ragged_ld_plus_3"] = c3
    finally:
        mm.set_option("f32_exact", 0)
    r = run(False, False, s, s, s, -1, 1.0, 0.0, 0, min(steps, 20))
    out["tf32x3"] = {"workload": f"SGEMM NN {s}^3 alpha=1 beta=0, 3xTF32 on tcgen05 (split passes included)", **r,
                     "x_fp32_ffma_peak": r["tflops"] / fp32_peak}
    return out


# ------------------------------------------------------------------ GPU arm -----------
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import numpy as np
    import torch
    import gemm_mmbo_b200 as mm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the library has no CPU path")
    torch.cuda.set_device(local_rank)
    host_affinity = None
    if world > 1:  # several ranks share the host: keep each one's pinned buffers on its GPU's NUMA node
        from gemm_mmbo_b200.sharded import bind_host_to_device
        host_affinity = bind_host_to_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    P = world if world > 1 else 1
    w = workload(args.gpus if world == 1 else world, args.size)
    m, n, k, ta, tb = w["m"], w["n"], w["k"], w["ta"], w["tb"]
    col0, ncols = mm.shard_columns(n, P, rank, 256) if P > 1 else (0, n)
    ra, rb, ca, cb = shapes(w, ncols)
    A, B, C = make_operands(torch, mm, w, col0, ncols)
    O = None
    if not args.no_extras or not args.no_cpu_baseline:
        from oracle import oracle as O  # the checker: sampled binary64 dot products, CPU baseline

    def step():
        mm.gemm("f16", ta, tb, m, ncols, k, w["alpha"], A, ra, B, rb, w["beta"], C, m, args.kernel)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warm):
        """ms per step of `fn`: barrier + synchronize on both sides, CUDA events on the launching stream,
        max over ranks."""
        for _ in range(warm):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        mine = e0.elapsed_time(e1)
        worst = mine
        if dist is not None:
            t = torch.tensor([mine], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            worst = float(t.item())
        return worst / steps, mine / steps

    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    for _ in range(warm):
        step()
    barrier()
    sampler.start()
    launches0 = mm.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    launches = mm.launch_count() - launches0
    clocks = sampler.stop()
    my_ms = ev0.elapsed_time(ev1)
    ms = my_ms
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    status = mm.device_status()
    if status:
        raise SystemExit(f"bench.py: device fault word {status:#x}")
    ms_per_step = ms / args.steps
    flops = 2.0 * m * n * k
    value = flops / (ms_per_step * 1e-3) / 1e12
    per_rank = [{"rank": rank, "ms_per_step": my_ms / args.steps, "sm_mhz_median": clocks["sm_mhz"],
                 "reasons": clocks["reasons"],
                 "tflops_per_sampled_ghz": (2.0 * m * ncols * k / (my_ms / args.steps * 1e-3) / 1e12 /
                                            (clocks["sm_mhz"] / 1e3)) if clocks["sm_mhz"] else None}]
    if dist is not None:
        gathered = [None] * P
        dist.all_gather_object(gathered, per_rank[0])
        per_rank = gathered

    # correctness of one application of the headline step, on fresh C (sampled binary64 oracle)
    rel_err = None
    if O is not None and not args.no_extras:
        fill_c(mm, w, C, col0, ncols)
        step()
        torch.cuda.synchronize()
        rel_err = sampled_rel_err(O, w, lambda r, c: C[torch.as_tensor(c - col0), torch.as_tensor(r)].double().cpu().numpy(),
                                  col0, col0 + ncols)

    # kernel-only duration (events around each launch) for the roofline of one launch
    kern_ms = []
    for _ in range(min(args.steps, 20)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        kern_ms.append(a.elapsed_time(b))
    isolated_ms = sum(kern_ms) / len(kern_ms)
    kern_avg = my_ms / args.steps  # average launch duration over the timed region (back-to-back launches of this rank)
    peaks = measured_peaks()
    # the timed region is a loop of back-to-back launches: sustained when it lasts seconds, burst otherwise
    peak = peaks["sustained"] if ms > 2000.0 else peaks["burst"]
    achieved = 2.0 * m * ncols * k / (kern_avg * 1e-3) / 1e12
    kid = args.kernel if args.kernel >= 0 else mm.select_kernel("f16", ta, tb, m, ncols, k, A, ra, B, rb, C, m)
    traffic = TRAFFIC_8192_NT.get(kid) if (P == 1 and (m, n, k) == (8192, 8192, 8192)) else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic["bytes"] if traffic else None,
                "traffic_source": traffic["source"] if traffic else None,
                "algorithmic_bytes": 2.0 * (m * k + k * ncols + m * ncols * (2 if w["beta"] else 1)),
                "peak_source": f"{peaks['source']} cuBLAS bf16 "
                               f"({'sustained' if ms > 2000.0 else 'burst'}); nominal dense fp16 2250",
                "frac_of_nominal": achieved / 2250.0,
                "kernel": mm.kernel_name("f16", kid),
                "kernel_ms": kern_avg, "isolated_launch_ms": isolated_ms}

    # cuBLAS (through torch) on the identical operands, same steps, after ours; never on the product path
    vendor = None
    if not args.no_extras:
        v_ms, _ = timed(lambda: vendor_mm(torch, w, A, B, C), args.steps, 3)
        vendor = {"library": "cuBLAS via torch.mm / addmm_", "ms_per_step": v_ms,
                  "tflops": flops / (v_ms * 1e-3) / 1e12, "ours_over_vendor": v_ms / ms_per_step}

    # ---------------- the exchange step of the sharded configuration (N > 1) ----------------
    exchange = None
    if P > 1 and not args.no_extras:
        exchange = exchange_legs(torch, dist, mm, O, w, args, rank, P, col0, ncols, A, B, ra, rb, timed, barrier,
                                 ms_per_step)

    # ---------------- end to end: pinned host operands -> device -> GEMM -> host ----------------
    e2e = None
    if not args.no_e2e:
        hA = torch.empty(A.shape, dtype=A.dtype).pin_memory()
        hB = torch.empty(B.shape, dtype=B.dtype).pin_memory()
        hC = torch.empty(C.shape, dtype=C.dtype).pin_memory()
        fill_c(mm, w, C, col0, ncols)
        hA.copy_(A)
        hB.copy_(B)
        hC.copy_(C)
        hC0 = hC.clone() if w["beta"] != 0.0 else None
        use_c = w["beta"] != 0.0
        e2e_steps = max(3, min(args.steps, 10 if P == 1 else 5))
        comm = None
        if P > 1:
            from gemm_mmbo_b200.sharded import ColumnShard, nccl_comm_ptr
            shard = ColumnShard(n, P, rank)
            try:
                comm = nccl_comm_ptr()
                have = torch.ones(1, device="cuda")
            except Exception as e:  # a torch without access to the communicator: every rank uploads all of A itself
                have = torch.zeros(1, device="cuda")
                if rank == 0:
                    print(f"bench.py: no ncclComm_t from torch ({type(e).__name__}: {e}); e2e without sharing A", file=sys.stderr)
            dist.all_reduce(have, op=dist.ReduceOp.MIN)
            if float(have.item()) == 0.0:
                comm = None
        if comm is not None:
            a_share = mm.shard_columns(ca, P, rank, 8)[1] * ra

            def e2e_step():
                # one library call per rank: 1/N of A host -> device, shares exchanged over NVLink, B / C
                # column panels copied in, multiplied and copied out on overlapping streams
                shard.gemm_sharded_host(ta, tb, m, k, w["alpha"], hA, ra, hB, rb, w["beta"], hC, m, comm, args.kernel)
            api = "mmbo_gemm_f16_sharded_host (pinned host A, B block, C block; A shares exchanged by NCCL over NVLink)"
        else:
            a_share = hA.numel()

            def e2e_step():
                # one library call on host operands: A staged once, B/C column panels copied in,
                # multiplied and copied out on overlapping streams; returns when hC is complete
                mm.gemm_host("f16", ta, tb, m, ncols, k, w["alpha"], hA, ra, hB, rb, w["beta"], hC, m, args.kernel)
            api = "mmbo_gemm_f16_host (pinned host A, B, C)"
        ems, _ = timed(e2e_step, e2e_steps, 2)
        e2e_err = None
        if O is not None and not args.no_extras:
            if hC0 is not None:
                hC.copy_(hC0)
            e2e_step()
            e2e_err = sampled_rel_err(O, w, lambda r, c: hC[torch.as_tensor(c - col0), torch.as_tensor(r)].double().numpy(),
                                      col0, col0 + ncols, seed=11)
        h2d = (a_share + hB.numel() + (hC.numel() if use_c else 0)) * 2
        e2e = {"value": flops / (ems * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": hC.numel() * 2, "steps": e2e_steps,
               "ms_per_step": ems, "api": api, "rel_err": e2e_err}
        del hA, hB, hC

    extras = {}
    if P == 1 and not args.no_extras:
        del A, B, C
        torch.cuda.empty_cache()
        extras["sgemm"] = sgemm_legs(torch, mm, O, args.steps, clocks["sm_max_mhz"])
        torch.cuda.empty_cache()
        # the T1 of the multi-GPU curve: the sharded configuration on this one GPU (3 x 2 GiB)
        w5 = config5(args.size)
        A5, B5, C5 = make_operands(torch, mm, w5, 0, w5["n"])
        s5 = max(3, min(args.steps, 6))
        samp5 = ClockSampler(local_rank)
        samp5.start()
        t5, _ = timed(lambda: mm.gemm("f16", False, False, w5["m"], w5["n"], w5["k"], 1.0, A5, w5["m"], B5, w5["k"], 0.0,
                                      C5, w5["m"], args.kernel), s5, 2)
        c5 = samp5.stop()
        err5 = sampled_rel_err(O, w5, lambda r, c: C5[torch.as_tensor(c), torch.as_tensor(r)].double().cpu().numpy(),
                               0, w5["n"], nsamp=24)
        f5 = 2.0 * w5["m"] * w5["n"] * w5["k"]
        v5, _ = timed(lambda: vendor_mm(torch, w5, A5, B5, C5), s5, 2)
        extras["config5_1gpu"] = {"workload": w5["name"], "ms_per_step": t5, "tflops": f5 / (t5 * 1e-3) / 1e12,
                                  "steps": s5, "rel_err": err5, "sm_mhz_median": c5["sm_mhz"], "reasons": c5["reasons"],
                                  "vendor_ms_per_step": v5, "vendor_tflops": f5 / (v5 * 1e-3) / 1e12}
        del A5, B5, C5

    cpu = None
    if rank == 0 and P == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(w)

    status = mm.device_status()
    if status:
        raise SystemExit(f"bench.py: device fault word {status:#x}")
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": P, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if P > 1 else "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": w["name"], "m": m, "n": n, "k": k, "columns_per_gpu": ncols,
                       "gather_c": False, "l2": "inputs larger than L2 (126 MB)", "accumulate": "fp32",
                       "host_affinity_rank0": host_affinity},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline, "rel_err": rel_err,
            "per_rank": per_rank, "vendor": vendor, "exchange": exchange, **extras,
            "cpu_baseline": cpu, "impl": "ours",
        }
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()


def exchange_legs(torch, dist, mm, O, w, args, rank, P, col0, ncols, A, B, ra, rb, timed, barrier, base_ms):
    """The optional exchange of the sharded configuration (every rank ends a step with the whole C), three ways.
    Each leg: `steps` timed steps (max over ranks), then one step on poisoned C whose result is checked on
    elements of a block this rank RECEIVED (the next rank's), against binary64 dot products."""
    from gemm_mmbo_b200.sharded import ColumnShard, SymmetricC, nccl_comm_ptr
    m, n, k, ta, tb = w["m"], w["n"], w["k"], w["ta"], w["tb"]
    shard = ColumnShard(n, P, rank)
    steps = max(3, min(args.steps, 10))
    flops = 2.0 * m * n * k
    peer_c0, peer_nc = shard.block_of((rank + 1) % P)
    out = {"steps": steps, "no_exchange_ms_per_step": base_ms}
    token = torch.zeros(1, device="cuda")  # a one-element all-reduce: the stream-ordered meeting point of the NCCL leg

    def leg(name, fn, Cfull, note, sync):
        ok = torch.ones(1, device="cuda")
        try:
            # The same GEMM without the exchange, into the same buffer, timed right before the leg: under the power
            # cap the clock of a long run drifts, so a ratio against a figure taken minutes earlier says little.
            own = Cfull[col0:col0 + ncols]

            def plain():
                mm.gemm("f16", ta, tb, m, ncols, k, w["alpha"], A, ra, B, rb, w["beta"], own, m, args.kernel)

            def plain_lockstep():  # ... and with the ranks meeting after every step, as every exchange makes them do
                plain()
                sync()
            near_ms, _ = timed(plain, steps, 2)
            lock_ms, _ = timed(plain_lockstep, steps, 2)
            ms, _ = timed(fn, steps, 2)
            Cfull.fill_(float("nan"))
            barrier()
            fn()
            barrier()
            err = sampled_rel_err(O, w, lambda r, c: Cfull[torch.as_tensor(c), torch.as_tensor(r)].double().cpu().numpy(),
                                  peer_c0, peer_c0 + peer_nc, nsamp=24, seed=100 + rank)
            finite = bool(torch.isfinite(Cfull).all().item())
            res = {"ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12, "no_exchange_ms_just_before": near_ms,
                   "no_exchange_lockstep_ms_just_before": lock_ms,
                   "x_no_exchange": ms / near_ms, "x_no_exchange_lockstep": ms / lock_ms, "x_first_timed_region": ms / base_ms,
                   "rel_err": err, "whole_c_finite": finite, "how": note}
        except Exception as e:  # a rank that cannot run a leg says so; the others learn it below
            ok.zero_()
            res = {"error": f"{type(e).__name__}: {e}"}
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0 and "error" not in res:
            res = {"error": "another rank failed this leg"}
        out[name] = res

    Csym = None
    try:
        Csym = SymmetricC(n, m)
        have = torch.ones(1, device="cuda")
    except Exception as e:
        have = torch.zeros(1, device="cuda")
        out["symmetric_memory"] = f"unavailable: {type(e).__name__}: {e}"
    dist.all_reduce(have, op=dist.ReduceOp.MIN)
    if float(have.item()) == 1.0:
        mc = torch.tensor([1.0 if Csym.multicast_ptr else 0.0], device="cuda")
        dist.all_reduce(mc, op=dist.ReduceOp.MIN)
        if float(mc.item()) == 1.0:
            leg("fused_multicast",
                lambda: shard.gemm_and_multicast(ta, tb, m, k, w["alpha"], A, ra, B, rb, w["beta"], Csym, kernelId=args.kernel),
                Csym.tensor, "mmbo_gemm_f16_mcast: epilogue writes each piece once with multimem.st, NVSwitch "
                             "delivers it to every GPU; stream-ordered barrier ends the step", Csym.barrier)
        else:
            out["fused_multicast"] = {"error": "no NVLink multicast mapping on this system"}
        leg("fused_peer_stores",
            lambda: shard.gemm_and_broadcast(ta, tb, m, k, w["alpha"], A, ra, B, rb, w["beta"], Csym, kernelId=args.kernel),
            Csym.tensor, "mmbo_gemm_f16_bcast: epilogue issues one TMA store per GPU for each piece; barrier ends the step",
            Csym.barrier)
    barrier()
    Cfull = Csym.tensor if Csym is not None else torch.empty((n, m), dtype=torch.float16, device="cuda")
    comm = None
    try:
        comm = nccl_comm_ptr()
    except Exception as e:
        out["nccl_all_gather"] = {"error": f"no ncclComm_t from torch: {type(e).__name__}: {e}"}
    if comm is not None:
        leg("nccl_all_gather",
            lambda: shard.gemm_sharded(ta, tb, m, k, w["alpha"], A, ra, B, rb, w["beta"], Cfull, True, comm, args.kernel),
            Cfull, "mmbo_gemm_f16_sharded(gatherC=1): GEMM, then ncclAllGather in place on the same stream",
            lambda: dist.all_reduce(token))
    barrier()
    # every rank leaves the multicast object together, with nothing in flight
    del Cfull
    Csym = None
    barrier()
    return out


if __name__ == "__main__":
    main()
