#!/usr/bin/env python
"""Benchmark of the hot path through the C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cg|jacobi2d|jacobi3d|chain|matvec]
    python bench.py --impl reference ...      # the CPU restatement of the reference path

One step = one pass of the hot path: one CG iteration (default workload, configuration C3:
matrix-free CG on the 2-D Poisson 5-point operator, 8192 x 8192 unknowns per GPU), one Jacobi
sweep, one fused-chain repeat or one power-iteration step.  Inputs are synthetic, generated on
the device from a seed; every working set but Jacobi2D's (64 MiB, which the configuration
fixes) is far larger than L2.

The JSON line carries the named workload at the top level and, under "workloads", the same
figures for the other four configurations at the same number of GPUs.

Before anything is timed, an untimed check leg runs small seeded problems (Jacobi 2-D / 3-D at
two halo depths, CG, the chain, a matvec) through the C ABI on all N ranks and through the CPU
oracle on the same DAG, and compares them ("check" in the JSON line); the process exits
non-zero when a case fails.

Timed quantities, per workload
  value     K steps enqueued back to back, CUDA events on the library's own stream, barrier and
            device synchronisation on both sides, maximum over ranks; that burst is repeated at
            least five times (and for at least a second, so that the clock sampler sees it) and
            the median burst is reported, with the fastest and slowest beside it.
  e2e       the same K steps, each one submitted from the host as a DAG blob through
            cn_receive_dag and followed by a device->host read of the step's scalar result
            through cn_get (host buffers on both sides, one synchronisation per step).
  e2e_solve (CG) a whole solve through the C ABI: the right-hand side goes up from pinned host
            memory (cn_put_local), K iterations run, the solution comes back (cn_get_local).
  roofline  the dominant kernel's algorithmic bytes / its mean launch duration, taken from the
            library's per-kernel CUDA-event records over a further K profiled steps.
  cpu_baseline  the oracle's C loops (OpenMP) on this box's host cores, a bounded number of
            steps of the same workload (rank 0, N = 1 only).
"""
import argparse
import datetime
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
ALL_WORKLOADS = ["cg", "jacobi2d", "jacobi3d", "chain", "matvec"]
DEFAULT_HALO = {"jacobi2d": 64}  # rows per side at N > 1; every other workload uses 1


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return PEAKS_FALLBACK_GBS, "fallback"


def dram_traffic(kernel):
    """(DRAM bytes per launch, where the figure comes from) of a kernel, from the committed ncu
    capture of that kernel (profiles/dram_traffic.json: measured dram read+write bytes per
    algorithmic byte on a reduced-size case; traffic of these streaming kernels grows in
    proportion to the points processed).  An entry names the code digest of the kernel it was
    captured from (the `#xxxxxxxx` the library puts at the end of a kernel's label: source,
    device header and tile configuration); a capture of another version of the kernel is not
    used.  (None, reason) when no capture covers the running kernel."""
    try:
        table = json.loads((ROOT / "profiles" / "dram_traffic.json").read_text())
    except Exception:
        return None, "profiles/dram_traffic.json not readable"
    label = kernel["kernel"]
    for entry in table.get("kernels", []):
        if entry["match"] in label:
            if entry.get("code") and entry["code"] not in label:
                return None, (f"{entry['source']} was captured from another version of this kernel "
                              f"({entry['code']})")
            algorithmic = kernel["gbs"] * 1e9 * kernel["ms_per_launch"] * 1e-3
            return entry["dram_bytes_per_algorithmic_byte"] * algorithmic, "profiles/" + entry["source"]
    return None, "no capture of this kernel"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 100 ms; stop() keeps the samples
    whose time stamp falls inside the window it is given."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
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

    def stop(self, window=None):
        if self.proc is None:
            return None
        try:
            self.proc.terminate()
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            return None
        rows = []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm, smax = float(f[1]), float(f[2])
            except ValueError:
                continue
            try:
                stamp = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
            except ValueError:
                stamp = None
            try:
                power = float(f[3])
            except ValueError:
                power = 0.0
            active = [n for n, v in zip(names, f[5:9]) if v.lower().startswith("active")]
            rows.append((stamp, sm, smax, power, active))
        if not rows:
            return None
        inside = rows
        if window is not None:
            inside = [r for r in rows if r[0] is not None and window[0] <= r[0] <= window[1]] or rows
        sm = [r[1] for r in inside]
        reasons = sorted({n for r in inside for n in r[4]})
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(r[2] for r in inside),
                "power_w_max": max(r[3] for r in inside), "reasons": reasons,
                "samples": len(inside), "samples_outside_window": len(rows) - len(inside)}


def dist_setup(world):
    if world == 1:
        return None
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    # The library's NCCL communicator carries set-up traffic, operand rows of stepped views and
    # one-value collectives; halos and reduction totals go through the peer mailboxes.  NVLink
    # multicast buffers are not worth their set-up for that (an explicit setting is respected).
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
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


def min_over_ranks(dist, value):
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return float(t[0])


def sum_over_ranks(dist, value):
    if dist is None:
        return value
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t[0])


def gather_bytes_fn(dist, world):
    """Every rank's byte string, on every rank (the check leg compares reduction results
    across ranks with it)."""
    if dist is None:
        return None

    def gather(b):
        out = [None] * world
        dist.all_gather_object(out, bytes(b))
        return out
    return gather


def share_unique_id(dist, rank):
    import torch
    import charmnumeric_b200 as cnp
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = torch.frombuffer(bytearray(cnp.comm_unique_id()), dtype=torch.uint8).clone()
    dist.broadcast(buf, src=0)
    return bytes(buf.tolist())


def pinned_array(shape):
    """float64 host array in page-locked memory (plain numpy when pinning is not possible)."""
    import numpy as np
    try:
        import torch
        n = 1
        for s in shape:
            n *= int(s)
        return torch.empty(n, dtype=torch.float64, pin_memory=True).numpy().reshape(shape), True
    except Exception:
        return np.empty(shape, dtype=np.float64), False


def config_for(name, world, scale, halo):
    """The configuration block of a JSON line; the GPU arm and the CPU arm print the same one."""
    from charmnumeric_b200.workloads import WORKLOADS
    w = WORKLOADS[name]
    weak = w.scaling == "weak"
    return {"workload": w.describe(world, scale)["description"],
            "l2": ("64 MiB working set, fixed by the configuration: served from L2 once warm; no flush"
                   if name == "jacobi2d" and scale <= 1.0
                   else "working set far larger than L2; no flush"),
            "parallelism": f"slab{world}", "scale": scale, "halo_depth": halo if world > 1 else 0,
            "aggregate": ("value = GPUs x iterations/s of the per-GPU slab" if weak and world > 1
                          else "value = steps/s of the whole problem")}


# ---- CPU baseline (oracle; never on the product path) -------------------------------------------

def cpu_baseline(workload, scale, steps, threads):
    """Time the oracle's OpenMP C loops on the host: `steps` steps of the same workload.
    Returns (steps_per_second, description)."""
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


def cpu_baseline_tiled(workload, scale, steps, pes):
    """The reference-structured variant of the CPU baseline (CG and Jacobi2D): every array a
    grid of separately allocated tiles (tile size by the reference's rule for `pes` PEs and an
    overdecomposition factor of 4), one worker thread per PE, halo rows and columns packed
    into messages and copied on receive, every node into a result buffer and copied back, dot
    products as passes of their own.  Returns a dict for the JSON line, or None."""
    import numpy as np
    from oracle import oracle as O
    lib = O.clib()
    secs = np.zeros(1)
    if workload == "cg":
        n = max(8, int(8192 * scale))
        m = n + 2
        b = np.zeros((m, m))
        b[1:-1, 1:-1] = O.randu((m, m), 0x5EED + 3)[1:-1, 1:-1]
        hist = np.zeros(steps)
        lib.cno_cg_poisson_tiled(O._ptr(b), None, m, steps, O._ptr(hist), 0, int(pes), O._ptr(secs))
        extent = m
    elif workload == "jacobi2d":
        n = max(8, int(2048 * scale))
        u = O.randu((n, n), 0x5EED + 1)
        res = np.zeros(steps // 10 + 1)
        lib.cno_jacobi2d_tiled(O._ptr(u), n, 0.25, steps, 10, O._ptr(res), 0, int(pes), O._ptr(secs))
        extent = n
    else:
        return None
    tile = int(lib.cno_tile(extent, 2, 4 * int(pes)))
    per_dim = (extent + tile - 1) // tile
    return {"value": steps / float(secs[0]), "cores": int(pes), "tile": tile, "tiles": per_dim * per_dim,
            "what": ("tiles as separate allocations, one worker per PE, packed halo messages, "
                     "result buffer + copy per node, separate dot passes")}


def run_reference(args, rank, world):
    """The CPU arm: the oracle's loops for the named workload on all host cores, rank 0 only.
    It runs the per-GPU problem of the N = 1 run once; its configuration block and its step
    and warm-up counts are the GPU arm's."""
    if rank != 0:
        return
    from charmnumeric_b200.workloads import WORKLOADS
    threads = os.cpu_count() or 1
    K, W = max(1, args.steps), max(3, args.warmup)
    halo = args.halo if args.halo > 0 else DEFAULT_HALO.get(args.workload, 1)
    cpu_baseline(args.workload, args.scale, W, threads)  # warm-up steps, untimed
    value, sample = cpu_baseline(args.workload, args.scale, K, threads)
    w = WORKLOADS[args.workload]
    line = {
        "impl": "reference", "metric": w.metric, "value": value, "unit": w.unit,
        "n_gpus": args.gpus, "steps": K, "warmup": W,
        "ms_per_step": 1000.0 / value, "higher_is_better": True, "scaling": w.scaling,
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": config_for(args.workload, world, args.scale, halo),
        "note": ("CPU restatement of the reference path (the reference's own Charm++/MLIR binary "
                 "cannot be built on this box); one rank-0 process runs the per-GPU problem size "
                 "of the N = 1 run on all host cores"),
        "cpu_baseline": {"value": value, "unit": w.unit, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    tiled = cpu_baseline_tiled(args.workload, args.scale, max(1, K // 2), threads)
    if tiled:
        line["cpu_baseline"]["tiled"] = tiled
    print(json.dumps(line), flush=True)


# ---- GPU arm ----------------------------------------------------------------------------------------

def timed_bursts(ctx, dist, wl, K, step_index, min_bursts, min_total_ms, max_bursts=400):
    """Bursts of K steps, each bracketed by a barrier and a device synchronisation and timed
    with CUDA events on the library's stream (maximum over ranks).  Every rank sees the same
    maxima, so all ranks run the same number of bursts.  On several ranks a device-side barrier
    (one allreduce of one value) is enqueued in front of each burst's start event."""
    times = []
    total = 0.0
    align = wl.align_blob() if dist is not None else None
    while len(times) < min_bursts or (total < min_total_ms and len(times) < max_bursts):
        barrier(dist)
        ctx.synchronize()
        if align is not None:
            # a one-value allreduce in front of the start event: the ranks leave the host barrier
            # tens of microseconds apart, which a burst of 13 us steps would otherwise count
            ctx.receive_dag(align)
        ctx.timer_start()
        for _ in range(K):
            wl.run_step(step_index)
            step_index += 1
        ms = max_over_ranks(dist, ctx.timer_stop())
        times.append(ms)
        total += ms
    barrier(dist)
    return times, step_index


def e2e_solve(ctx, dist, wl, K, rank):
    """A whole CG solve through the C ABI with host buffers on both ends: this rank's slab of
    the right-hand side goes up from pinned host memory, K iterations run, this rank's slab of
    the solution comes back into pinned host memory."""
    import numpy as np
    info = ctx.array_info(wl.b.name)
    rb, re = info["rows"]
    m0, m1 = wl.shape
    host_b, pinned = pinned_array((re - rb, m1))
    host_x, _ = pinned_array((re - rb, m1))
    rng = np.random.default_rng(0x5EED + 33 + rank)
    host_b[...] = rng.random((re - rb, m1))
    host_b[:, 0] = 0.0
    host_b[:, -1] = 0.0
    if rb == 0:
        host_b[0, :] = 0.0
    if re == m0:
        host_b[-1, :] = 0.0
    seconds = []
    for _ in range(3):
        barrier(dist)
        ctx.synchronize()
        t0 = time.perf_counter()
        ctx.put_local(wl.b.name, wl.shape, host_b)
        ctx.receive_dag(wl.init_blob)
        for i in range(K):
            wl.run_step(i)
        ctx.get_local_into(wl.x.name, host_x)  # waits for the stream
        seconds.append(max_over_ranks(dist, time.perf_counter() - t0))
    finite = bool(np.isfinite(host_x).all())
    return {"seconds": statistics.median(seconds), "h2d_bytes": int(host_b.nbytes), "d2h_bytes": int(host_x.nbytes),
            "pinned": pinned, "solution_finite": finite}


def measure(name, args, itf, dist, rank, world, local_rank, primary):
    """Everything that is measured for one workload; returns the dict that goes into the JSON
    line (rank 0) or None (other ranks)."""
    import charmnumeric_b200 as cnp
    from charmnumeric_b200.workloads import WORKLOADS

    ctx = itf.context
    cnp.reset_frontend_state()
    halo = args.halo if args.halo > 0 else DEFAULT_HALO.get(name, 1)
    if world > 1:
        ctx.set_option("halo", halo)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a few hundred ms before its first sample
    extra = {}
    if args.res_every >= 0 and name in ("jacobi2d", "jacobi3d"):
        extra["res_every"] = args.res_every  # diagnostic: how much of a step the residual costs
    wl = WORKLOADS[name](itf, nranks=world, scale=args.scale, **extra)
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

    # ---- device-timed region: repeated bursts of K steps ----
    stats0 = ctx.stats()
    t_begin = datetime.datetime.now()
    times, step_index = timed_bursts(ctx, dist, wl, K, step_index, 5,
                                     0.0 if args.quick else (1200.0 if primary else 800.0), max_bursts=4000)
    ctx.synchronize()
    t_end = datetime.datetime.now()
    stats1 = ctx.stats()
    clocks = sampler.stop((t_begin, t_end)) if rank == 0 else None
    ms = statistics.median(times)
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

    solve = None
    if name == "cg" and primary:
        solve = e2e_solve(ctx, dist, wl, K, rank)

    entry = None
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
            traffic, traffic_from = dram_traffic(top)
            roofline = {"bound": "hbm", "achieved": top["gbs"], "peak": peak, "unit": "GB/s",
                        "frac": top["gbs"] / peak, "traffic": traffic, "traffic_from": traffic_from,
                        "kernel": top["kernel"],
                        "peak_kind": peak_kind, "nominal_frac": top["gbs"] / 8000.0}
        # weak scaling: every GPU iterates its own slab of the (N times larger) global grid, so the
        # whole-job figure is GPUs x iterations/s; strong scaling: one fixed problem, steps/s
        agg = world if wl.scaling == "weak" else 1
        step_gbs = wl.bytes_per_step / world / (ms / K * 1e-3) / 1e9
        entry = {
            "name": name, "metric": wl.metric, "value": agg * K / (ms * 1e-3), "unit": wl.unit,
            "ms_per_step": ms / K, "scaling": wl.scaling,
            "bursts": {"count": len(times), "steps_each": K, "median_ms": ms, "min_ms": min(times),
                       "max_ms": max(times), "value_best": agg * K / (min(times) * 1e-3),
                       "value_worst": agg * K / (max(times) * 1e-3)},
            "config": dict(config_for(name, world, args.scale, halo), **({"res_every": extra["res_every"]} if extra else {})),
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
        if solve is not None:
            entry["e2e_solve"] = {
                "value": agg * K / solve["seconds"], "unit": wl.unit, "iterations": K,
                "seconds": solve["seconds"], "h2d_bytes_per_gpu": solve["h2d_bytes"],
                "d2h_bytes_per_gpu": solve["d2h_bytes"], "pinned_host_memory": solve["pinned"],
                "solution_finite": solve["solution_finite"],
                "what": "cn_put_local of the right-hand side + K iterations + cn_get_local of the solution"}
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            try:
                budget_steps = {"cg": 12, "jacobi2d": 200, "jacobi3d": 3, "chain": 3, "matvec": 5}
                v, sample = cpu_baseline(name, args.scale, budget_steps[name], threads)
                entry["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": threads, "kind": "port",
                                         "sample": sample}
                if threads > 4 and primary:
                    # the reference's own test set-up runs on four PEs (charmrun +p4)
                    v4, _ = cpu_baseline(name, args.scale, max(1, budget_steps[name] // 2), 4)
                    entry["cpu_baseline"]["p4"] = {"value": v4, "cores": 4}
                # the same arithmetic laid out as the reference runs it (tiles, messages, copies)
                tiled = cpu_baseline_tiled(name, args.scale, max(1, budget_steps[name] // 2), threads)
                if tiled:
                    entry["cpu_baseline"]["tiled"] = tiled
                    if threads > 4 and primary:
                        entry["cpu_baseline"]["tiled_p4"] = cpu_baseline_tiled(
                            name, args.scale, max(1, budget_steps[name] // 3), 4)
            except Exception as exc:  # the baseline is a report, never a gate
                entry["cpu_baseline"] = {"error": repr(exc)}
    wl.release()
    ctx.synchronize()
    barrier(dist)
    return entry


def run_gpu(args, rank, world, local_rank):
    import charmnumeric_b200 as cnp

    dist = dist_setup(world)
    uid = share_unique_id(dist, rank) if world > 1 else None
    itf = cnp.CharmNumericInterface(device=local_rank, rank=rank, nranks=world, unique_id=uid)
    ctx = itf.context
    K, W = max(1, args.steps), max(3, args.warmup)

    # ---- untimed check leg: small seeded problems against the CPU oracle, on all N ranks ----
    check = None
    if not args.no_check:
        import __graft_entry__ as entry_points
        check = entry_points.check_cases(itf, world, gather_bytes_fn(dist, world))
        everyone_ok = min_over_ranks(dist, 1.0 if check["ok"] else 0.0) > 0.5
        check["ok_on_all_ranks"] = everyone_ok
        if not check["ok"]:
            print(f"[bench] rank {rank}: check failed: "
                  f"{[c for c in check['cases'] if not c['ok']]}", file=sys.stderr, flush=True)

    names = [args.workload] + ([] if args.only else [w for w in ALL_WORKLOADS if w != args.workload])
    entries = []
    for i, name in enumerate(names):
        entries.append(measure(name, args, itf, dist, rank, world, local_rank, primary=(i == 0)))

    if rank == 0:
        first = entries[0]
        line = {
            "metric": first["metric"], "value": first["value"], "unit": first["unit"], "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": first["ms_per_step"], "higher_is_better": True,
            "scaling": first["scaling"], "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": first["config"], "bursts": first["bursts"], "roofline": first["roofline"],
            "step_hbm": first["step_hbm"], "kernels": first["kernels"], "e2e": first["e2e"],
            "gpu_launches": first["gpu_launches"], "clocks": first["clocks"],
        }
        for key in ("e2e_solve", "cpu_baseline"):
            if key in first:
                line[key] = first[key]
        if check is not None:
            line["check"] = check
        line["workloads"] = [{k: v for k, v in e.items() if k != "kernels"} for e in entries[1:]]
        print(json.dumps(line), flush=True)
    barrier(dist)
    itf.close()
    if dist is not None:
        dist.destroy_process_group()
    if check is not None and not check["ok_on_all_ranks"]:
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cg", choices=ALL_WORKLOADS,
                    help="the workload of the top-level figures; the others follow under 'workloads'")
    ap.add_argument("--only", action="store_true", help="measure the named workload only")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scale", type=float, default=1.0, help="linear problem-size factor (1 = the configured size)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true",
                    help="five timed bursts only (profiling runs); the clock sampler may then see too little load")
    ap.add_argument("--no-check", action="store_true", help="skip the untimed parity check against the oracle")
    ap.add_argument("--halo", type=int, default=0, help="halo rows per side for N > 1 (0: per-workload default)")
    ap.add_argument("--res-every", type=int, default=-1,
                    help="Jacobi workloads: residual every n-th sweep (0: never; default: the configured 10)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
