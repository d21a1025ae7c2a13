"""Benchmark of the harmonics hot path.

    python bench.py --gpus 1 --steps 200 --warmup 10
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --steps K --warmup W      # the reference's CPU path

Workload: the case the headline metric is quoted on - SphericalHarmonics (normalised), l_max = 8,
float32, values + gradients, 4,194,304 points per GPU drawn iid N(0,1) per coordinate (seed 1000 +
rank). One step = one pass of the kernel over the rank's points. Points are independent, so ranks
share nothing: no collective is on the data path (NCCL is used only for the barrier around the
timed region and to take the maximum time over ranks). Scaling is weak by default (every rank has the
workload's full point count); ``--scaling strong`` fixes the total (8 x 4,194,304 points for the
headline case, the configuration's own size otherwise) and gives rank r the contiguous shard
``workloads.shard_bounds(total, world, r)``.

Prints ONE JSON line on rank 0.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from sphericart_b200 import workloads  # noqa: E402

METRIC = "points/sec, fp32 l_max=8 Y+dY (SphericalHarmonics)"
FALLBACK_HBM_GBS = 6650.0


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one step's kernel(s), from ncu captures of
# a launch of `points` points of the same kernel(s); the commands and counters are in the summaries
# under profiles/. A capture of the full workload would break the profiler's size rule, so the figure
# for n points is the captured bytes plus the algorithmic bytes of the n - `points` further points:
# what separates captured from algorithmic bytes is written data still resident in the 126 MB L2 when
# the kernel ends, a constant that does not grow with the launch.
NCU_TRAFFIC = {
    "spherical_l8_f32_grad": {"points": 524288, "dram_bytes": 627.0e6},
    "solid_l6_f32_grad_n1e6": {"points": 1000000, "dram_bytes": 737.5e6},
    "spherical_l4_f32_fwd_vjp_n5e7": {"points": 4194304, "dram_bytes": 412.3e6 + 514.0e6},
    "spherical_l16_f32_hess_n2e6": {"points": 65536, "dram_bytes": 926.5e6},
    "spherical_l32_f64_grad_n1e6": {"points": 32768, "dram_bytes": 1087.5e6},
}


def _recorded_traffic(wl, n_points, bytes_per_point):
    entry = NCU_TRAFFIC.get(wl.name)
    if entry is None or n_points < entry["points"]:
        return None
    return {"dram_bytes_per_launch": entry["dram_bytes"] + bytes_per_point * (n_points - entry["points"]),
            "note": f"ncu capture of a {entry['points']}-point launch ({entry['dram_bytes'] / 1e6:.1f} MB) plus the "
                    f"algorithmic bytes of the other {n_points - entry['points']} points; the shortfall against the "
                    "algorithmic bytes is written data still in L2 at kernel end"}


class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons of one GPU through NVML (read-only)."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, uuid, period=0.01):
        super().__init__(daemon=True)
        self.period = period
        self.samples = []  # (t, sm_mhz, reasons bitmask)
        self.max_mhz = None
        self._stop = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID("GPU-" + uuid)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((time.perf_counter(), mhz, int(reasons)))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop.set()

    def summary(self, t0, t1):
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        note = "sampled during the timed region"
        if not inside:
            inside = self.samples
            note = "timed region shorter than the sampling period: samples span warm-up and timed region"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "NVML unavailable"}
        mask = 0
        for s in inside:
            mask |= s[2]
        reasons = sorted(name for bit, name in self.REASONS.items() if mask & bit)
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(inside), "note": note}


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return rank, local, world


def reduce_max(value, world, device=None):
    """Maximum of a Python float over ranks (device-timed durations are reduced this way)."""
    if world == 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def reduce_sum(value, world, device=None):
    if world == 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def _cpu_build_flags():
    """How the reference CPU library under oracle/_ref was compiled (recorded by oracle/Makefile). It
    travels between machines, so it targets a portable instruction set rather than the host's own."""
    try:
        with open(os.path.join(ROOT, "oracle", "_ref", "build_flags.txt")) as f:
            return f.read().strip()
    except OSError:
        return "unknown flags"


def cpu_reference_rate(wl, sample_points, seconds_budget=12.0, min_reps=3, max_reps=40):
    """Times the reference's CPU path (or the restatement when the reference library is not
    there) on ``sample_points`` points of the workload with all host threads.
    Returns (points_per_second_median, kind, cores, reps, seconds_per_pass)."""
    from oracle import oracle

    oracle.use_all_host_threads()
    xyz = workloads.make_points("metric", n_points=sample_points)
    ny = wl.ny
    sph = np.empty((sample_points, ny), dtype=wl.np_dtype)
    dsph = np.empty((sample_points, 3, ny), dtype=wl.np_dtype)
    if oracle.have_ref():
        calc = oracle.RefCalculator(wl.l_max, wl.normalized, wl.np_dtype)
        kind, cores = "reference", calc.omp_num_threads()

        def one_pass():
            calc.compute(xyz, wl.level, out=(sph, dsph, None))
    else:
        kind, cores = "port", os.cpu_count() or 1

        def one_pass():
            oracle.port_compute(xyz, wl.l_max, wl.normalized, wl.level, nthreads=0, out=(sph, dsph, None))

    one_pass()  # first touch of the outputs + warm-up
    one_pass()
    times = []
    t_start = time.perf_counter()
    while len(times) < max_reps and (len(times) < min_reps or time.perf_counter() - t_start < seconds_budget):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return sample_points / med, kind, cores, len(times), med


def run_reference_arm(args):
    rank, _, world = _dist_env()
    if rank != 0:
        return
    wl, _ = workloads.CONFIGS["metric"]
    from oracle import oracle

    host_threads = oracle.use_all_host_threads()
    sample = 1 << 20
    xyz = workloads.make_points("metric", n_points=sample)
    sph = np.empty((sample, wl.ny), dtype=wl.np_dtype)
    dsph = np.empty((sample, 3, wl.ny), dtype=wl.np_dtype)
    if oracle.have_ref():
        calc = oracle.RefCalculator(wl.l_max, wl.normalized, wl.np_dtype)
        kind, cores = "reference", calc.omp_num_threads()

        def step():
            calc.compute(xyz, wl.level, out=(sph, dsph, None))
    else:
        kind, cores = "port", host_threads

        def step():
            oracle.port_compute(xyz, wl.l_max, wl.normalized, wl.level, nthreads=0, out=(sph, dsph, None))

    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - t0
    value = sample * args.steps / elapsed
    sample_text = (f"{sample} points of the workload per step (seed 1000), reference CPU library via its C API, "
                   f"built with `{_cpu_build_flags()}`, OpenMP threads = {cores}" if kind == "reference" else
                   f"{sample} points per step, CPU restatement (reference library not built on this machine)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "points/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl.name, "l_max": wl.l_max, "level": "values+gradients",
                   "points_per_step": sample, "device": "host CPU"},
        "cpu_baseline": {"value": value, "unit": "points/s", "cores": cores, "kind": kind, "sample": sample_text},
        "e2e": {"value": value, "unit": "points/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--points", type=int, default=None, help="points per GPU (default: the workload's 4,194,304)")
    ap.add_argument("--e2e-steps", type=int, default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every GPU gets the workload's full point count; strong: the total is fixed "
                         "(8 x 4,194,304 points for the headline case, the configuration's size otherwise) and sharded")
    ap.add_argument("--config", default="metric", choices=sorted(workloads.CONFIGS),
                    help="metric = the headline case; cfg1..cfg5 = the other benchmark configurations; "
                         "aux_* = backward-kernel cases captured by the profiles")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch

    import sphericart_b200
    from sphericart_b200.host_pipeline import HostPipeline

    rank, local, world = _dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU code path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    wl, _ = workloads.CONFIGS[args.config]
    warmup = max(args.warmup, 3)
    tdtype = torch.float64 if wl.dtype == "f64" else torch.float32
    strong = args.scaling == "strong"
    if strong:
        # one point set of fixed size for any number of GPUs, cut into contiguous shards
        total = args.points or (8 * wl.n_points if args.config == "metric" else wl.n_points)
        lo, hi = workloads.shard_bounds(total, world, rank)
        n = hi - lo
        if n == 0:
            raise SystemExit("strong scaling: the point set is too small for this many GPUs")
        xyz_host = torch.from_numpy(workloads.make_points(args.config, n_points=total)[lo:hi].copy())
    else:
        n = args.points or wl.n_points
        xyz_host = torch.from_numpy(workloads.make_points(args.config, n_points=n, seed_offset=rank))
    xyz = xyz_host.to(device)
    calc = (sphericart_b200.SphericalHarmonics if wl.normalized else sphericart_b200.SolidHarmonics)(wl.l_max)
    ny = wl.ny
    sph = torch.empty((n, ny), dtype=tdtype, device=device)
    dsph = torch.empty((n, 3, ny), dtype=tdtype, device=device) if wl.level >= 1 else None
    ddsph = torch.empty((n, 3, 3, ny), dtype=tdtype, device=device) if wl.level >= 2 else None
    sph_grad = dsph_grad = xyz_grad = None
    if wl.vjp2:
        sph_grad = torch.from_numpy(workloads.make_upstream_grad(args.config, n_points=n, seed_offset=rank)).to(device)
        dsph_grad = torch.from_numpy(
            workloads.make_upstream_gradient_of_gradients(args.config, n_points=n, seed_offset=rank)).to(device)
        xyz_grad = torch.empty((n, 3), dtype=tdtype, device=device)
    if wl.vjp:
        grad_host = (workloads.make_upstream_grad(args.config, n_points=total)[lo:hi] if strong
                     else workloads.make_upstream_grad(args.config, n_points=n, seed_offset=rank))
        sph_grad = torch.from_numpy(grad_host).to(device)
        del grad_host
        xyz_grad = torch.empty((n, 3), dtype=tdtype, device=device)
    stream = torch.cuda.current_stream(device)
    ptr = lambda t: None if t is None else t.data_ptr()  # noqa: E731

    launches = 0

    def step():
        nonlocal launches
        calc.compute_raw(tdtype, wl.level, xyz.data_ptr(), n, ptr(sph), ptr(dsph), ptr(ddsph), stream.cuda_stream)
        launches += 1
        if wl.vjp:
            calc.compute_vjp_raw(tdtype, xyz.data_ptr(), n, sph_grad.data_ptr(), xyz_grad.data_ptr(), stream.cuda_stream)
            launches += 1
        if wl.vjp2:
            calc.compute_vjp_with_gradients(xyz, sph_grad, dsph_grad, out=xyz_grad)
            launches += 1

    # bytes one step moves by the algorithm's own count (forward, plus the fused backward where the
    # configuration has one)
    elem = 8 if wl.dtype == "f64" else 4
    step_bytes_per_point = (elem * (3 + ny * (1, 4, 13)[wl.level]) + (elem * (3 + ny + 3) if wl.vjp else 0) +
                            (elem * (3 + 4 * ny + 3) if wl.vjp2 else 0))
    out_bytes = step_bytes_per_point * n
    # outputs smaller than a few L2 sizes would stay cached between steps: flush L2 between timed steps
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if out_bytes < (512 << 20) else None

    sampler = ClockSampler(str(torch.cuda.get_device_properties(device).uuid))
    sampler.start()
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    launches = 0
    t_wall0 = time.perf_counter()
    if flush is None:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        torch.cuda.synchronize(device)
        my_ms = ev0.elapsed_time(ev1)
    else:
        pairs = []
        for _ in range(args.steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            step()
            e1.record(stream)
            pairs.append((e0, e1))
        torch.cuda.synchronize(device)
        my_ms = sum(a.elapsed_time(b) for a, b in pairs)
    t_wall1 = time.perf_counter()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    sampler.stop()
    timed_launches = launches
    total_ms = reduce_max(my_ms, world, device)
    total_points = reduce_sum(float(n), world, device)
    ms_per_step = total_ms / args.steps
    value = total_points * args.steps / (total_ms * 1e-3)

    # end to end through the host-buffer front end: pinned host xyz -> device -> kernel -> pinned host outputs
    e2e = None
    if not args.no_e2e and args.config == "metric":
        e2e_steps = args.e2e_steps or max(1, min(args.steps, 5))
        pipe = HostPipeline(calc, wl.level, tdtype, device)
        xyz_pin = xyz_host.pin_memory()
        sph_pin = torch.empty((n, ny), dtype=tdtype, pin_memory=True)
        dsph_pin = torch.empty((n, 3, ny), dtype=tdtype, pin_memory=True)
        pipe.run(xyz_pin, [sph_pin, dsph_pin])  # warm-up
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            pipe.run(xyz_pin, [sph_pin, dsph_pin])
        e1.record(stream)
        torch.cuda.synchronize(device)
        my_e2e_ms = e0.elapsed_time(e1)
        e2e_ms = reduce_max(my_e2e_ms, world, device)
        bi, bo = pipe.bytes_per_point()
        # the link's own rate, measured here: one large device-to-host copy into the same pinned array
        # (this rank alone is timed; with several GPUs the ranks copy at the same time, as in the pipeline)
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dsph_pin.copy_(dsph, non_blocking=True)
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        c0.record(stream)
        dsph_pin.copy_(dsph, non_blocking=True)
        c1.record(stream)
        torch.cuda.synchronize(device)
        d2h_gbs = dsph.numel() * dsph.element_size() / (c0.elapsed_time(c1) * 1e-3) / 1e9
        my_d2h_gbs = bo * n * e2e_steps / (my_e2e_ms * 1e-3) / 1e9
        e2e = {"value": total_points * e2e_steps / (e2e_ms * 1e-3), "unit": "points/s",
               "h2d_bytes_per_step": int(bi * total_points), "d2h_bytes_per_step": int(bo * total_points),
               "steps": e2e_steps,
               "d2h_link_gbs": d2h_gbs, "d2h_achieved_gbs": my_d2h_gbs, "pcie_frac": my_d2h_gbs / d2h_gbs,
               "pcie_note": "rank 0: device-to-host bytes of the pipeline / its time, over the rate of one large "
                            "pinned device-to-host copy measured in this run; 1.0 = the link is the bound",
               "path": "HostPipeline: pinned host xyz -> H2D -> kernel -> D2H of sph and dsph into pinned host "
                       "arrays, 3 streams, 262144-point chunks; bound by PCIe device-to-host bandwidth"}
        del sph_pin, dsph_pin

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = _peaks()
    bytes_per_launch = out_bytes
    achieved = bytes_per_launch / (my_ms / args.steps * 1e-3) / 1e9
    traffic = _recorded_traffic(wl, n, step_bytes_per_point)
    # the kernel names come from the library's own dispatch rule, not from a guess made here
    from sphericart_b200 import _c_lib

    ctype = "double" if wl.dtype == "f64" else "float"
    kernel = f"{_c_lib.kernel_family(wl.level, wl.l_max, elem)}<{ctype}, l_max={wl.l_max}, level={wl.level}>"
    if wl.vjp:
        kernel += f" + {_c_lib.kernel_family(3, wl.l_max, elem)}<{ctype}, l_max={wl.l_max}>"
    if wl.vjp2:
        kernel += f" + {_c_lib.kernel_family(4, wl.l_max, elem)}<{ctype}, l_max={wl.l_max}, second order>"
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": (traffic or {}).get("dram_bytes_per_launch"),
                "peak_source": f"of {peak_kind}", "kernel": kernel,
                "algorithmic_bytes_per_launch": bytes_per_launch,
                "frac_basis": "algorithmic bytes per launch / CUDA-event time per launch, over a copy (read + write) "
                              "bandwidth: a store-only kernel can read above 1.0",
                "traffic_note": (traffic or {}).get("note")}

    cpu = None
    if world == 1 and not args.no_cpu_baseline and args.config == "metric":
        sample = 1 << 21
        rate, kind, cores, reps, sec = cpu_reference_rate(wl, sample)
        cpu = {"value": rate, "unit": "points/s", "cores": cores, "kind": kind,
               "sample": f"first {sample} points of the workload (seed 1000), {kind} CPU code"
                         + (f" built with `{_cpu_build_flags()}`" if kind == "reference" else "")
                         + f", {cores} OpenMP threads, median of {reps} passes of "
                         f"{sec * 1e3:.1f} ms after 2 warm-up passes, preallocated outputs"}

    line = {
        "metric": METRIC if args.config == "metric" else f"points/sec, {wl.name}",
        "value": value, "unit": "points/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.name, "class": "SphericalHarmonics" if wl.normalized else "SolidHarmonics",
                   "l_max": wl.l_max,
                   "level": ("values", "values+gradients", "values+gradients+hessians")[wl.level] +
                            (" then fused VJP" if wl.vjp else "") + (" then fused second-order VJP" if wl.vjp2 else ""),
                   "points_per_gpu": n, "bytes_per_point": step_bytes_per_point,
                   "l2_policy": (f"{out_bytes / 1e9:.2f} GB written per step per GPU, far larger than L2: no flush"
                                 if flush is None else
                                 "small outputs: a 256 MB buffer is rewritten between timed steps to flush L2, "
                                 "each step timed with its own event pair"),
                   "total_points": int(total_points),
                   "parallelism": (f"one point set of {int(total_points)} points cut into {world} contiguous shard(s), "
                                   "no collective" if strong else
                                   f"{n} points per GPU on {world} GPU(s), no collective")},
        "roofline": roofline, "cpu_baseline": cpu, "clocks": sampler.summary(t_wall0, t_wall1), "e2e": e2e,
        "gpu_launches": timed_launches,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
