#!/usr/bin/env python
"""Benchmark of the hot path through the C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cg|jacobi2d|jacobi3d|chain|matvec]
    python bench.py --impl reference ...      # the CPU restatement of the reference path

One step = one pass of the hot path: one CG iteration (default workload, configuration C3:
matrix-free CG on the 2-D Poisson 5-point operator, 8192 x 8192 unknowns per GPU), one Jacobi
sweep, one fused-chain repeat or one power-iteration step.  Inputs are synthetic, generated on
the device from a seed; the working set (five 537 MB arrays for CG) is far larger than L2.

Timed quantities
  value     K steps enqueued back to back, CUDA events on the library's own stream, barrier and
            device synchronisation on both sides, maximum over ranks.
  e2e       the same K steps, each one submitted from the host as a DAG blob through
            cn_receive_dag and followed by a device->host read of the step's scalar result
            through cn_get (host buffers on both sides, one synchronisation per step).
  roofline  the dominant kernel's algorithmic bytes / its mean launch duration, taken from the
            library's per-kernel CUDA-event records over a further K profiled steps.
  cpu_baseline  the oracle's C loops (reference-structured, OpenMP) on this box's host cores,
            a bounded number of steps of the same workload (rank 0, N = 1 only).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

PEAKS_FALLBACK_GBS = 6650.0


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return PEAKS_FALLBACK_GBS, "fallback"


def dram_traffic(kernel, wl):
    """DRAM bytes per launch of the dominant kernel, from the committed ncu capture of that
    kernel (profiles/dram_traffic.json: measured dram read+write bytes per algorithmic byte on a
    reduced-size case; traffic of these streaming kernels grows in proportion to the points
    processed).  None when no capture covers the kernel."""
    try:
        table = json.loads((ROOT / "profiles" / "dram_traffic.json").read_text())
    except Exception:
        return None
    label = kernel["kernel"]
    for entry in table.get("kernels", []):
        if entry["match"] in label:
            algorithmic = kernel["gbs"] * 1e9 * kernel["ms_per_launch"] * 1e-3
            return entry["dram_bytes_per_algorithmic_byte"] * algorithmic
    return None


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 100 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.device)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        try:
            self.proc.terminate()
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            return None
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return None
        busy = [v for v in sm if v > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(smax),
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(world):
    if world == 1:
        return None
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group(backend="gloo", rank=int(os.environ["RANK"]), world_size=world)
    return dist


def barrier(dist):
    if dist is not None:
        dist.barrier()


def max_over_ranks(dist, value):
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def sum_over_ranks(dist, value):
    if dist is None:
        return value
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t[0])


def share_unique_id(dist, rank):
    import torch
    import charmnumeric_b200 as cnp
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = torch.frombuffer(bytearray(cnp.comm_unique_id()), dtype=torch.uint8).clone()
    dist.broadcast(buf, src=0)
    return bytes(buf.tolist())


# ---- CPU baseline (oracle; never on the product path) -------------------------------------------

def cpu_baseline(workload, scale, steps, threads):
    """Time the oracle's reference-structured C loops on the host: `steps` steps of the same
    workload.  Returns (steps_per_second, description)."""
    import numpy as np
    from oracle import oracle as O
    lib = O.clib()
    O.build()
    lib.cno_set_threads(int(threads))
    if workload == "cg":
        n = max(8, int(8192 * scale))
        m = n + 2
        b = np.zeros((m, m))
        b[1:-1, 1:-1] = O.randu((m, m), 0x5EED + 3)[1:-1, 1:-1]
        x, r, p, Ap = (np.empty((m, m)) for _ in range(4))
        hist = np.zeros(steps)
        tile = O.ref_tile(m * m, 1)
        t0 = time.perf_counter()
        lib.cno_cg_poisson(O._ptr(b), O._ptr(x), O._ptr(r), O._ptr(p), O._ptr(Ap), m, steps,
                           O._ptr(hist), tile)
        dt = time.perf_counter() - t0
        return steps / dt, f"{steps} CG iterations on the full {n}x{n} grid"
    if workload == "jacobi2d":
        n = max(8, int(2048 * scale))
        u = O.randu((n, n), 0x5EED + 1)
        scratch = np.zeros_like(u)
        res = np.zeros(steps // 10 + 1)
        t0 = time.perf_counter()
        lib.cno_jacobi2d(O._ptr(u), O._ptr(scratch), n, n, 0.25, steps, 10, O._ptr(res),
                         O.ref_tile(n, 2))
        dt = time.perf_counter() - t0
        return steps / dt, f"{steps} sweeps of the full {n}x{n} grid"
    if workload == "jacobi3d":
        n = max(8, int(1024 * scale))
        u = O.randu((n, n, n), 0x5EED + 5)
        scratch = np.zeros_like(u)
        res = np.zeros(steps // 10 + 1)
        t0 = time.perf_counter()
        lib.cno_jacobi3d(O._ptr(u), O._ptr(scratch), n, n, n, 1.0 / 6.0, steps, 10, O._ptr(res),
                         O.ref_tile(n, 3))
        dt = time.perf_counter() - t0
        return steps / dt, f"{steps} sweeps of the full {n}^3 grid"
    if workload == "chain":
        n = max(8, int((1 << 28) * scale))
        a = O.randu((n,), 0x5EED + 2, -1.0, 1.0)
        b = O.randu((n,), 0x5EED + 22, -1.0, 1.0)
        t0 = time.perf_counter()
        for _ in range(steps):
            lib.cno_chain_sum(O._ptr(a), O._ptr(b), n, O.ref_tile(n, 1))
        dt = time.perf_counter() - t0
        return steps / dt, f"{steps} repeats over the full vectors of length {n}"
    if workload == "matvec":
        full = max(8, int(65536 * scale))
        n = min(full, 16384)  # 2 GiB of matrix on the host; scaled by bytes to the full size
        A = O.randu((n, n), 0x5EED + 4, -1.0 / 256, 1.0 / 256)
        x = O.randu((n,), 0x5EED + 44, -1.0, 1.0)
        y = np.empty(n)
        hist = np.zeros(steps)
        t0 = time.perf_counter()
        lib.cno_power_iteration(O._ptr(A), O._ptr(x), O._ptr(y), n, steps, O._ptr(hist),
                                O.ref_tile(n, 2))
        dt = time.perf_counter() - t0
        ratio = (full / n) ** 2
        return steps / dt / ratio, (f"{steps} power-iteration steps on a {n}x{n} matrix, time scaled "
                                    f"by {ratio:.0f}x (bytes) to {full}x{full}")
    raise ValueError(workload)


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    steps = max(1, args.steps)
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(args.workload, args.scale, 1, threads)
    value, sample = cpu_baseline(args.workload, args.scale, steps, threads)
    from charmnumeric_b200.workloads import WORKLOADS
    w = WORKLOADS[args.workload]
    line = {
        "impl": "reference", "metric": w.metric, "value": value, "unit": w.unit,
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": 1000.0 / value, "higher_is_better": True, "scaling": w.scaling,
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": args.workload, "note": "CPU restatement of the reference path "
                   "(the reference's own Charm++/MLIR binary cannot be built on this box); one "
                   "rank-0 process, per-GPU problem size of the N=1 run"},
        "cpu_baseline": {"value": value, "unit": w.unit, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm ----------------------------------------------------------------------------------------

def run_gpu(args, rank, world, local_rank):
    import charmnumeric_b200 as cnp
    from charmnumeric_b200.workloads import WORKLOADS

    dist = dist_setup(world)
    uid = share_unique_id(dist, rank) if world > 1 else None
    itf = cnp.CharmNumericInterface(device=local_rank, rank=rank, nranks=world, unique_id=uid)
    ctx = itf.context
    cnp.reset_frontend_state()
    # halo depth: sweeps without a fused reduction also update the halo rows they can, so a
    # deeper halo means fewer exchanges (Jacobi2D: one per 8 sweeps; measured no gain for the
    # 8 MiB planes of Jacobi3D, whose exchange is bandwidth, not latency)
    halo = args.halo if args.halo > 0 else {"jacobi2d": 8}.get(args.workload, 1)
    if world > 1:
        ctx.set_option("halo", halo)
    wl = WORKLOADS[args.workload](itf, nranks=world, scale=args.scale)
    K, W = max(1, args.steps), max(3, args.warmup)

    # every distinct step blob once, so that no run-time compilation lands in a timed region
    for i in range(len(wl.blobs)):
        ctx.receive_dag(wl.blobs[i])
    ctx.synchronize()
    step_index = 0
    for _ in range(W):
        wl.run_step(step_index)
        step_index += 1
    ctx.synchronize()

    # ---- device-timed region ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    stats0 = ctx.stats()
    barrier(dist)
    ctx.synchronize()
    ctx.timer_start()
    for _ in range(K):
        wl.run_step(step_index)
        step_index += 1
    ms = ctx.timer_stop()
    barrier(dist)
    stats1 = ctx.stats()
    ms = max_over_ranks(dist, ms)
    launches = sum_over_ranks(dist, stats1["kernel_launches"] - stats0["kernel_launches"])

    # ---- end to end: host blob in, scalar result out, every step ----
    blob_bytes = max(len(b) for b in wl.blobs)
    barrier(dist)
    ctx.synchronize()
    t0 = time.perf_counter()
    last = None
    for _ in range(K):
        wl.run_step(step_index)
        step_index += 1
        last = wl.read_result()
    ctx.synchronize()
    e2e_s = max_over_ranks(dist, time.perf_counter() - t0)

    # ---- per-kernel profile over K more steps (event pairs around every launch) ----
    ctx.profile(True)
    for _ in range(K):
        wl.run_step(step_index)
        step_index += 1
    prof = ctx.profile_report()
    ctx.profile(False)
    # The sampler runs through the device-timed, end-to-end and profiled passes (same workload).
    # nvidia-smi needs a few hundred ms before its first sample: when the three passes together
    # were shorter than 1.5 s, the same steps keep running under the sampler until that much
    # load has been seen.  The count derives from the rank-maximum time, so all ranks agree.
    extra = 0
    if 3.0 * ms < 1500.0:
        extra = min(500000, int((1500.0 - 3.0 * ms) / max(ms / K, 1e-4)) + 1)
        for _ in range(extra):
            wl.run_step(step_index)
            step_index += 1
        ctx.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = ("timed + end-to-end + profiled passes" if not extra else
                            f"timed + end-to-end + profiled passes + {extra} more steps of the same workload")

    if rank == 0:
        peak, peak_kind = measured_peak()
        roofline = None
        kernels = []
        if prof:
            total_ms = sum(r["ms"] for r in prof) or 1.0
            for r in sorted(prof, key=lambda r: -r["ms"]):
                gbs = r["bytes"] / (r["ms"] * 1e-3) / 1e9 if r["ms"] > 0 else 0.0
                kernels.append({"kernel": r["label"], "launches": r["launches"],
                                "ms_per_launch": r["ms"] / max(1, r["launches"]),
                                "share": r["ms"] / total_ms, "gbs": gbs})
            top = kernels[0]
            roofline = {"bound": "hbm", "achieved": top["gbs"], "peak": peak, "unit": "GB/s",
                        "frac": top["gbs"] / peak, "traffic": dram_traffic(top, wl), "kernel": top["kernel"],
                        "peak_kind": peak_kind, "nominal_frac": top["gbs"] / 8000.0}
        # weak scaling: every GPU iterates its own slab of the (N times larger) global grid, so the
        # whole-job figure is GPUs x iterations/s; strong scaling: one fixed problem, steps/s
        agg = world if wl.scaling == "weak" else 1
        value = agg * K / (ms * 1e-3)
        step_gbs = wl.bytes_per_step / world / (ms / K * 1e-3) / 1e9
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": wl.scaling,
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": wl.description, "l2": "working set far larger than L2; no flush",
                       "parallelism": f"slab{world}", "scale": args.scale,
                       "halo_depth": halo if world > 1 else 0,
                       "aggregate": ("value = GPUs x iterations/s of the per-GPU slab" if agg > 1
                                     else "value = steps/s of the whole problem")},
            "roofline": roofline,
            "step_hbm": {"algorithmic_bytes_per_step_per_gpu": wl.bytes_per_step / world,
                         "gbs_per_gpu": step_gbs, "frac_of_" + peak_kind: step_gbs / peak,
                         "frac_of_nominal_8000": step_gbs / 8000.0},
            "kernels": kernels,
            "e2e": {"value": agg * K / e2e_s, "unit": wl.unit, "h2d_bytes_per_step": blob_bytes,
                    "d2h_bytes_per_step": 8, "last_result": last},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            try:
                budget_steps = {"cg": 12, "jacobi2d": 200, "jacobi3d": 3, "chain": 3, "matvec": 5}
                v, sample = cpu_baseline(args.workload, args.scale, budget_steps[args.workload], threads)
                line["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": threads, "kind": "port",
                                        "sample": sample}
                if threads > 4:
                    # the reference's own test set-up runs on four PEs (charmrun +p4)
                    v4, _ = cpu_baseline(args.workload, args.scale, max(1, budget_steps[args.workload] // 2), 4)
                    line["cpu_baseline"]["p4"] = {"value": v4, "cores": 4}
            except Exception as exc:  # the baseline is a report, never a gate
                line["cpu_baseline"] = {"error": repr(exc)}
        print(json.dumps(line), flush=True)
    barrier(dist)
    itf.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cg", choices=["cg", "jacobi2d", "jacobi3d", "chain", "matvec"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scale", type=float, default=1.0, help="linear problem-size factor (1 = the configured size)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--halo", type=int, default=0, help="halo rows per side for N > 1 (0: per-workload default)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
