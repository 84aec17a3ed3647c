#!/usr/bin/env python
"""Benchmark of the GEMM hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one GEMM call through the library's C ABI on synthetic seeded operands:

  N = 1  HGEMM NT, M=N=K=8192, alpha=1, beta=0.5, A/B/C ~ N(0, 0.5^2) rounded to fp16
         (the configuration the headline metric is quoted on);
  N > 1  HGEMM NN, M=N=K=32768, alpha=1, beta=0, U[-1,1): B and C split into N column
         blocks, A replicated, one rank per GPU, no communication in the contraction
         (--gather: the GEMM's epilogue also stores each rank's block into every rank's copy of
         C over NVLink, so that each step ends with the whole C on every GPU; --gather-nccl: the
         same through an overlapped NCCL all-gather).

`value` is whole-job TFLOP/s (2*M*N*K per step over the slowest rank's device time) with
operands resident in HBM; `e2e` is the same metric with pinned host operands copied to
the device and the result copied back inside the timed region.  `--impl reference`
times the CPU restatement of the reference's arithmetic (oracle/) on the host cores.
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


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--gather", action="store_true",
                    help="N>1: every rank ends each step with the whole C (the GEMM's epilogue stores its block "
                         "into all ranks' copies over NVLink)")
    ap.add_argument("--gather-nccl", action="store_true",
                    help="N>1: the same result through an NCCL all-gather overlapped with the GEMM in 4 panels")
    ap.add_argument("--kernel", type=int, default=-1, help="force a kernel id of the fp16 table")
    ap.add_argument("--size", type=int, default=0, help="override M=N=K (debugging / profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def workload(n_gpus: int, size: int):
    if n_gpus == 1:
        s = size or 8192
        return dict(name=f"HGEMM NT {s}^3 alpha=1 beta=0.5 normal(0,0.5) fp16", ta=False, tb=True, m=s, n=s,
                    k=s, alpha=1.0, beta=0.5, dist=1, scale=0.5)
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
        "config": {"workload": w["name"], "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                         "sample": f"each step = one {edge}x{edge}x{w['k']} panel of the workload, "
                                   "fp64 accumulation, all host threads"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ GPU arm -----------
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import gemm_mmbo_b200 as mm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    P = world if world > 1 else 1
    w = workload(args.gpus if world == 1 else world, args.size)
    m, n, k, ta, tb = w["m"], w["n"], w["k"], w["ta"], w["tb"]
    col0, ncols = mm.shard_columns(n, P, rank, 256) if P > 1 else (0, n)

    # Operands, generated on the device from the shared seeded generator.
    ra, rb = (k if ta else m), (ncols if tb else k)
    ca, cb = (m if ta else k), (k if tb else ncols)
    A = torch.empty((ca, ra), dtype=torch.float16, device="cuda")
    B = torch.empty((cb, rb), dtype=torch.float16, device="cuda")
    C = torch.empty((ncols, m), dtype=torch.float16, device="cuda")
    mm.fill("f16", A, ra, ca, ra, mat=0, dist=w["dist"], scale=w["scale"])
    if tb:   # B stored n x k: the block is a row window
        mm.fill("f16", B, rb, cb, rb, mat=1, dist=w["dist"], scale=w["scale"], row0=col0, total_rows=n)
    else:    # B stored k x n: the block is a column window
        mm.fill("f16", B, rb, cb, rb, mat=1, dist=w["dist"], scale=w["scale"], col0=col0, total_rows=k)
    mm.fill("f16", C, m, ncols, m, mat=2, dist=w["dist"], scale=w["scale"], col0=col0, total_rows=m)
    Cfull = torch.empty((n, m), dtype=torch.float16, device="cuda") if (args.gather_nccl and P > 1) else None
    Csym = None
    shard = None
    if P > 1 and (args.gather or args.gather_nccl):
        from gemm_mmbo_b200.sharded import ColumnShard, SymmetricC
        shard = ColumnShard(n, P, rank)
        if Cfull is None:
            try:
                Csym = SymmetricC(n, m)  # every rank's copy of the whole C, mapped into every rank
                ok = torch.ones(1, device="cuda")
            except Exception as e:  # no symmetric memory on this system: all ranks fall back together
                if rank == 0:
                    print(f"bench.py: symmetric memory unavailable ({type(e).__name__}: {e}); using the NCCL all-gather",
                          file=sys.stderr)
                ok = torch.zeros(1, device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok.item()) == 0.0:
                Csym = None
                Cfull = torch.empty((n, m), dtype=torch.float16, device="cuda")

    def step():
        if Csym is not None:  # the epilogue stores this rank's block into every rank's C, then a barrier
            shard.gemm_and_broadcast(ta, tb, m, k, w["alpha"], A, ra, B, rb, w["beta"], Csym, kernelId=args.kernel)
        elif shard is not None:  # GEMM in column panels, each panel's all-gather overlapped
            shard.gemm_and_gather("f16", ta, tb, m, k, w["alpha"], A, ra, B, rb, w["beta"], C, Cfull,
                                  panels=4, kernelId=args.kernel)
        else:
            mm.gemm("f16", ta, tb, m, ncols, k, w["alpha"], A, ra, B, rb, w["beta"], C, m, args.kernel)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
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

    # kernel-only duration (events around each launch) for the roofline of one launch
    kern_ms = []
    for _ in range(min(args.steps, 20)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        mm.gemm("f16", ta, tb, m, ncols, k, w["alpha"], A, ra, B, rb, w["beta"], C, m, args.kernel)
        b.record()
        torch.cuda.synchronize()
        kern_ms.append(a.elapsed_time(b))
    isolated_ms = sum(kern_ms) / len(kern_ms)
    # average launch duration over the timed region (back-to-back launches of this rank)
    kern_avg = ev0.elapsed_time(ev1) / args.steps if shard is None else isolated_ms
    peaks = measured_peaks()
    # the timed region is a loop of back-to-back launches: sustained when it lasts
    # seconds, burst otherwise
    peak = peaks["sustained"] if ms > 2000.0 else peaks["burst"]
    achieved = 2.0 * m * ncols * k / (kern_avg * 1e-3) / 1e12
    # DRAM bytes per launch from the ncu capture of this workload (dram__bytes_read.sum +
    # dram__bytes_write.sum; summary under profiles/): known for the default N=1 case only
    traffic = 1.805e9 if (P == 1 and (m, n, k) == (8192, 8192, 8192) and args.kernel in (-1, 3)) else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic,
                "algorithmic_bytes": 2.0 * (m * k + k * ncols + m * ncols * (2 if w["beta"] else 1)),
                "peak_source": f"{peaks['source']} cuBLAS bf16 "
                               f"({'sustained' if ms > 2000.0 else 'burst'}); nominal dense fp16 2250",
                "frac_of_nominal": achieved / 2250.0,
                "kernel": mm.kernel_name("f16", args.kernel if args.kernel >= 0 else mm.select_kernel(
                    "f16", ta, tb, m, ncols, k, A, ra, B, rb, C, m)),
                "kernel_ms": kern_avg, "isolated_launch_ms": isolated_ms}

    # end to end: pinned host operands -> device -> GEMM -> host, inside the timed region
    e2e = None
    if not args.no_e2e:
        hA = torch.empty(A.shape, dtype=A.dtype).pin_memory()
        hB = torch.empty(B.shape, dtype=B.dtype).pin_memory()
        hC = torch.empty(C.shape, dtype=C.dtype).pin_memory()
        hA.copy_(A)
        hB.copy_(B)
        hC.copy_(C)
        use_c = w["beta"] != 0.0
        e2e_steps = max(3, min(args.steps, 10 if P == 1 else 3))

        def e2e_step():
            # one library call on host operands: A staged once, B/C column panels copied in,
            # multiplied and copied out on overlapping streams; returns when hC is complete
            mm.gemm_host("f16", ta, tb, m, ncols, k, w["alpha"], hA, ra, hB, rb, w["beta"], hC, m, args.kernel)

        for _ in range(2):
            e2e_step()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(e2e_steps):
            e2e_step()
        b.record()
        barrier()
        ems = a.elapsed_time(b)
        if dist is not None:
            t = torch.tensor([ems], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t.item())
        h2d = (hA.numel() + hB.numel() + (hC.numel() if use_c else 0)) * 2
        e2e = {"value": flops / (ems / e2e_steps * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": hC.numel() * 2, "steps": e2e_steps,
               "ms_per_step": ems / e2e_steps, "api": "mmbo_gemm_f16_host (pinned host A, B, C)"}

    cpu = None
    if rank == 0 and P == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(w)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": P, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if P > 1 else "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": w["name"], "m": m, "n": n, "k": k, "columns_per_gpu": ncols,
                       "gather_c": ("fused: epilogue stores to every GPU's C" if Csym is not None else
                                    "NCCL all-gather, 4 panels" if Cfull is not None else False),
                       "l2": "inputs larger than L2 (126 MB)",
                       "accumulate": "fp32"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps, "roofline": roofline,
            "cpu_baseline": cpu, "impl": "ours",
        }
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
