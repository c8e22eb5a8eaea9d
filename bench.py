"""
Benchmark of the neighbor-list build (one "step" = one build through the C ABI).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload diamond512k|diamond1000|...]

Prints ONE JSON line (rank 0). Metric: neighbor pairs per second of the
512 000-atom diamond build (full list, fp64, quantities i j S d D), inputs
resident in HBM; `e2e` is the same build from pinned host buffers with the
host->device copy of the points and the device->host copy of every output
array inside the timed region. `--impl reference` times the unmodified
reference CPU path (oracle/_ref) on the host cores on the same workload.
With N > 1 every rank builds its own copy of the system on its own GPU
(independent systems, no communication): weak scaling.
"""

import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from vesin_b200 import workloads  # noqa: E402

WORKLOADS = {
    # name: (generator, cutoff, full list, description)
    "diamond512k": (lambda: workloads.diamond(40), 5.0, True, "diamond 40x40x40 (512000 atoms), cutoff 5.0, full list, fp64, ijSdD"),
    "diamond512k_half": (lambda: workloads.diamond(40), 5.0, False, "diamond 40x40x40 (512000 atoms), cutoff 5.0, half list, fp64, ijSdD"),
    "diamond512k_f32": (lambda: workloads.diamond(40), 5.0, True, "diamond 40x40x40 (512000 atoms), cutoff 5.0, full list, fp32 in / fp32 d and D out (decisions in fp64), ijSdD"),
    "diamond110k": (lambda: workloads.diamond(24), 5.0, True, "diamond 24x24x24 (110592 atoms), cutoff 5.0, full list, fp64, ijSdD"),
    "diamond1000": (lambda: workloads.diamond(5), 5.0, True, "diamond 5x5x5 (1000 atoms), cutoff 5.0, full list, fp64, ijSdD"),
    "triclinic64": (lambda: workloads.small_triclinic(), 9.0, True, "64 atoms in a small triclinic cell, cutoff 9.0, full list, fp64, ijSdD"),
    "liquid2m": (lambda: workloads.liquid(1 << 21), 6.0, False, "LJ-density liquid, 2097152 atoms, cutoff 6.0, half list, fp64 ABI, ijSdD"),
}

BATCH_WORKLOADS = {
    # name: (n_systems, cutoff, full list, description)
    "molecules16k": (16384, 4.0, True, "16384 non-periodic molecules of 16-64 atoms in a 6 A sphere, cutoff 4.0, full list, ijSdD, one batched call"),
    "molecules2k": (2048, 4.0, True, "2048 non-periodic molecules of 16-64 atoms in a 6 A sphere, cutoff 4.0, full list, ijSdD, one batched call"),
}

SHARDED_WORKLOADS = {
    # name: (n_atoms, cutoff, full list, description)
    "liquid16m": (1 << 24, 6.0, False, "LJ-density liquid, 16777216 atoms, cutoff 6.0, half list, fp64, ijSdD, slab-decomposed over the ranks"),
    "liquid2m_sharded": (1 << 21, 6.0, False, "LJ-density liquid, 2097152 atoms, cutoff 6.0, half list, fp64, ijSdD, slab-decomposed over the ranks"),
}

BYTES_PER_POINT = 24  # fp64 positions
BYTES_PER_PAIR = 16 + 12 + 8 + 24  # i, j as size_t; S int32[3]; d; D


def algorithmic_bytes(n_points, n_pairs):
    return n_points * BYTES_PER_POINT + n_pairs * BYTES_PER_PAIR


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the
    timed region runs."""

    def __init__(self, index):
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _run(self):
        nv = self._nvml
        names = {
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "hw_power_brake_slowdown": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {
            "sm_mhz": float(np.median(self.samples)) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def physical_gpu_index(local_index):
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        try:
            return int(visible.split(",")[local_index])
        except (ValueError, IndexError):
            pass
    return local_index


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def time_reference_cpu(system, cutoff, full, steps, warmup, budget_s):
    """Reference CPU path on all host cores; returns (pairs, seconds per build,
    builds timed)."""
    from oracle import oracle

    oracle.build()
    cpu = oracle.ReferenceCPU()
    points, box, periodic = system
    n_pairs = 0
    started = time.perf_counter()
    for _ in range(warmup):
        n_pairs = cpu.run(points, box, periodic, cutoff, full, "ijSdD", n_threads=0)
        if time.perf_counter() - started > budget_s / 2:
            break
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        n_pairs = cpu.run(points, box, periodic, cutoff, full, "ijSdD", n_threads=0)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - started > budget_s:
            break
    return n_pairs, float(np.mean(times)), len(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload in BATCH_WORKLOADS:
        run_reference_batch(args)
        return
    make, cutoff, full, description = WORKLOADS[args.workload]
    system = make()
    n_pairs, seconds, timed = time_reference_cpu(system, cutoff, full, args.steps, args.warmup, budget_s=240.0)
    cores = host_cores()
    value = n_pairs / seconds
    line = {
        "impl": "reference",
        "metric": "neighbor pairs/s",
        "value": value,
        "unit": "pairs/s",
        "n_gpus": args.gpus,
        "steps": timed,
        "warmup": args.warmup,
        "ms_per_step": seconds * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": description, "n_points": int(len(system[0])), "n_pairs": int(n_pairs), "l2": "outputs (GBs) exceed L2"},
        "cpu_baseline": {
            "value": value,
            "unit": "pairs/s",
            "cores": cores,
            "kind": "reference",
            "sample": f"{timed} full builds of the workload, reference CPU path, n_threads=0 (all {cores} cores)",
        },
        "e2e": {"value": value, "unit": "pairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_reference_batch(args):
    """Reference CPU path on a batch: one call per system, as its callers do."""
    from oracle import oracle

    oracle.build()
    n_systems, cutoff, full, description = BATCH_WORKLOADS[args.workload]
    points, offsets = workloads.molecule_batch(n_systems=n_systems, seed=4)
    cpu = oracle.ReferenceCPU()
    box = np.zeros((3, 3))
    sample = min(n_systems, 4096)

    def one_pass():
        pairs = 0
        for k in range(sample):
            pairs += cpu.run(points[offsets[k] : offsets[k + 1]], box, [False] * 3, cutoff, full, "ijSdD", n_threads=1)
        return pairs

    for _ in range(min(args.warmup, 1)):
        one_pass()
    times = []
    started = time.perf_counter()
    n_pairs = 0
    for _ in range(args.steps):
        t0 = time.perf_counter()
        n_pairs = one_pass()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - started > 120.0:
            break
    seconds = float(np.mean(times))
    value = n_pairs / seconds
    print(json.dumps({
        "impl": "reference",
        "metric": "neighbor pairs/s",
        "value": value,
        "unit": "pairs/s",
        "systems_per_s": sample / seconds,
        "n_gpus": args.gpus,
        "steps": len(times),
        "warmup": min(args.warmup, 1),
        "ms_per_step": seconds * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": description, "sample": f"first {sample} systems per step"},
        "cpu_baseline": {"value": value, "unit": "pairs/s", "cores": 1, "kind": "reference",
                         "sample": f"first {sample} systems, one reference CPU call per system, n_threads=1"},
        "e2e": {"value": value, "unit": "pairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def run_ours(args):
    import torch
    import torch.distributed as dist

    import vesin_b200
    from vesin_b200._c_api import N_STAGES, STAGE_NAMES, VesinCUDA, VesinDevice, VesinNeighborList, VesinOptions

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    lib = vesin_b200.get_library()
    make, cutoff, full, description = WORKLOADS[args.workload]
    points, box, periodic = make()
    n_points = len(points)
    float_io = args.workload.endswith("_f32")
    if float_io:
        points = points.astype(np.float32)
        box = box.astype(np.float32)
    entry_point = lib.vesin_b200_neighbors_f32 if float_io else lib.vesin_neighbors
    value_size = 4 if float_io else 8
    bytes_per_point = 3 * value_size
    bytes_per_pair = 16 + 12 + 4 * value_size

    h_points = torch.from_numpy(points).pin_memory()
    d_points = h_points.to(device)
    d_box = torch.from_numpy(box).to(device)
    d_periodic = torch.from_numpy(periodic).to(device)

    options = VesinOptions()
    options.cutoff = cutoff
    options.full = full
    options.sorted = False
    options.algorithm = 0
    options.n_threads = 0
    options.return_shifts = True
    options.return_distances = True
    options.return_vectors = True
    options.skin = 0.0
    c_device = VesinDevice(VesinCUDA, local_rank)
    neighbors = VesinNeighborList()
    error = ctypes.c_char_p()

    def build(points_tensor):
        status = entry_point(
            points_tensor.data_ptr(), n_points, d_box.data_ptr(), d_periodic.data_ptr(), c_device, options,
            ctypes.byref(neighbors), ctypes.byref(error),
        )
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))
        return neighbors.length

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)  # > 126 MB of L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- warm-up (also sizes the workspace and the output arrays) ----
    for _ in range(max(args.warmup, 3)):
        n_pairs = build(d_points)

    # ---- timed region 1: device-resident inputs ----
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    wall0 = time.perf_counter()
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        for k in range(args.steps):
            flush.fill_(k & 0xFF)  # untimed: evicts L2 between builds
            starts[k].record()
            n_pairs = build(d_points)
            stops[k].record()
        barrier()
    wall = time.perf_counter() - wall0
    device_ms = sum(a.elapsed_time(b) for a, b in zip(starts, stops))

    # ---- per-kernel times of the same builds (the library's own CUDA events on its stream;
    #      a separate, untimed loop: the event records cost a few microseconds per build) ----
    stage_ms = np.zeros(N_STAGES)
    stage_buffer = (ctypes.c_double * N_STAGES)()
    stage_steps = max(1, min(args.steps, 20))
    lib.vesin_b200_set_profiling(1)
    for k in range(stage_steps):
        flush.fill_(k & 0xFF)
        build(d_points)
        if lib.vesin_b200_stage_times(ctypes.byref(neighbors), stage_buffer) == 0:
            stage_ms += np.array(stage_buffer[:])
    lib.vesin_b200_set_profiling(0)
    stage_ms /= stage_steps
    barrier()

    # ---- timed region 2: end to end from pinned host buffers ----
    out_host = {
        "pairs": torch.empty((n_pairs, 2), dtype=torch.int64).pin_memory(),
        "shifts": torch.empty((n_pairs, 3), dtype=torch.int32).pin_memory(),
        "distances": torch.empty((n_pairs,), dtype=torch.float32 if float_io else torch.float64).pin_memory(),
        "vectors": torch.empty((n_pairs, 3), dtype=torch.float32 if float_io else torch.float64).pin_memory(),
    }
    e2e_steps = max(1, min(args.steps, 5))
    staging = torch.empty_like(d_points)

    def copy_out(name, pointer, count, dtype, cupy_typestr):
        from vesin_b200._neighbors import _view

        shape = tuple(out_host[name].shape)
        view = _view(pointer, shape, cupy_typestr, device, neighbors)
        if dtype == torch.int64:
            view = view.view(torch.int64)
        out_host[name].copy_(view, non_blocking=True)

    def e2e_step():
        staging.copy_(h_points, non_blocking=True)
        torch.cuda.current_stream(device).synchronize()
        count = build(staging)
        assert count == n_pairs
        copy_out("pairs", neighbors.pairs, count, torch.int64, "<u8")
        copy_out("shifts", neighbors.shifts, count, torch.int32, "<i4")
        copy_out("distances", neighbors.distances, count, None, "<f4" if float_io else "<f8")
        copy_out("vectors", neighbors.vectors, count, None, "<f4" if float_io else "<f8")
        torch.cuda.current_stream(device).synchronize()

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # ---- reduce over ranks: slowest rank sets the time ----
    times = torch.tensor([device_ms, e2e_ms, wall * 1e3], dtype=torch.float64, device=device)
    pairs_total = torch.tensor([float(n_pairs)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(pairs_total, op=dist.ReduceOp.SUM)
    device_ms, e2e_ms, wall_ms = times.tolist()
    total_pairs = pairs_total.item()

    if rank == 0:
        ms_per_step = device_ms / args.steps
        value = total_pairs / (ms_per_step * 1e-3)
        bytes_per_build = n_points * bytes_per_point + int(n_pairs) * bytes_per_pair
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            with open(peaks_path) as fd:
                peak = float(json.load(fd)["hbm_gbs"])
            peak_source = "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_source = 6650.0, "fallback"
        emit_ms = float(stage_ms[STAGE_NAMES.index("emit")])
        achieved = bytes_per_build / (emit_ms * 1e-3) / 1e9 if emit_ms > 0 else None
        line = {
            "metric": "neighbor pairs/s",
            "value": value,
            "unit": "pairs/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f64" if not float_io else "f64 decisions, f32 storage",
            "data": "synthetic",
            "config": {
                "workload": description,
                "n_points": n_points,
                "n_pairs": int(n_pairs),
                "per_gpu": "one independent copy of the system per GPU, no communication",
                "l2": "256 MiB buffer written between timed builds (untimed); outputs (2.7 GB) exceed L2",
            },
            "roofline": {
                "bound": "hbm",
                "kernel": "pairs_kernel",
                "achieved": achieved,
                "peak": peak,
                "unit": "GB/s",
                "frac": (achieved / peak) if achieved else None,
                "peak_source": peak_source,
                # dram__bytes_read + dram__bytes_write of pairs_kernel in the ncu capture of the 110 592-atom
                # case of the same kernel (profiles/pairs_kernel_diamond110k.md: 536.6 MB for 9 856 828 pairs),
                # scaled by the pairs of this launch; only for the quantities that capture wrote
                "traffic": (536.55e6 / 9856828 * int(n_pairs)) if (full and not float_io) else None,
                "traffic_unit": "bytes per launch, scaled from the 110k-atom ncu capture",
                "bytes_per_launch": bytes_per_build,
                "kernel_ms": emit_ms,
                "whole_build_frac": bytes_per_build / (ms_per_step * 1e-3) / 1e9 / peak,
            },
            "stages_ms": {name: float(ms) for name, ms in zip(STAGE_NAMES, stage_ms)},
            "e2e": {
                "value": total_pairs / (e2e_ms * 1e-3),
                "unit": "pairs/s",
                "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": n_points * bytes_per_point,
                "d2h_bytes_per_step": int(n_pairs) * bytes_per_pair,
            },
            "gpu_launches": 7 * args.steps,  # header (reset, zero, box check), bin (+ point checks), 2 x scan, 2 x scatter, pairs
            "wall_ms_per_step": wall_ms / args.steps,
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            cpu_pairs, cpu_seconds, timed = time_reference_cpu(
                (points.astype(np.float64), box.astype(np.float64), periodic), cutoff, full, 2, 1, budget_s=45.0
            )
            assert cpu_pairs == n_pairs, f"CPU reference found {cpu_pairs} pairs, GPU {n_pairs}"
            cores = host_cores()
            line["cpu_baseline"] = {
                "value": cpu_pairs / cpu_seconds,
                "unit": "pairs/s",
                "cores": cores,
                "kind": "reference",
                "sample": f"{timed} full builds of the same workload after 1 warm-up, reference CPU path (oracle/_ref), n_threads=0",
                "ms_per_build": cpu_seconds * 1e3,
            }
        print(json.dumps(line))

    lib.vesin_free(ctypes.byref(neighbors))
    if world > 1:
        dist.destroy_process_group()


def run_batch(args):
    """Batch of independent molecules: one call per rank on its share of the
    systems (contiguous chunks balanced by atoms, no communication)."""
    import torch
    import torch.distributed as dist

    import vesin_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    n_systems, cutoff, full, description = BATCH_WORKLOADS[args.workload]
    # weak scaling: every rank brings n_systems systems of its own
    points, offsets = workloads.molecule_batch(n_systems=n_systems, seed=4 + rank)
    h_points = torch.from_numpy(points).pin_memory()
    d_points = h_points.to(device)
    calculator = vesin_b200.BatchNeighborList(cutoff=cutoff, full_list=full)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(args.warmup, 3)):
        (pairs, S, d, D), pair_offsets = calculator.compute(d_points, offsets, quantities="PSdD", copy=False)
    n_pairs = int(pairs.shape[0])
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        for k in range(args.steps):
            flush.fill_(k & 0xFF)
            starts[k].record()
            calculator.compute(d_points, offsets, quantities="PSdD", copy=False)
            stops[k].record()
        barrier()
    device_ms = sum(a.elapsed_time(b) for a, b in zip(starts, stops)) / args.steps

    # end to end: points from pinned host memory, every output back to the host
    out_host = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (pairs, S, d, D, pair_offsets)]
    staging = torch.empty_like(d_points)

    def e2e_step():
        staging.copy_(h_points, non_blocking=True)
        outputs, po = calculator.compute(staging, offsets, quantities="PSdD", copy=False)
        for host, dev in zip(out_host, list(outputs) + [po]):
            host.copy_(dev, non_blocking=True)
        torch.cuda.current_stream(device).synchronize()

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(1, min(args.steps, 10))
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    times = torch.tensor([device_ms, e2e_ms], dtype=torch.float64, device=device)
    totals = torch.tensor([float(n_pairs), float(n_systems), float(len(points))], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    device_ms, e2e_ms = times.tolist()
    total_pairs, total_systems, total_points = totals.tolist()
    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
        bytes_per_call = algorithmic_bytes(len(points), n_pairs)
        line = {
            "metric": "neighbor pairs/s",
            "value": total_pairs / (device_ms * 1e-3),
            "unit": "pairs/s",
            "systems_per_s": total_systems / (device_ms * 1e-3),
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": device_ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f64",
            "data": "synthetic",
            "config": {
                "workload": description,
                "n_points": int(total_points),
                "n_pairs": int(total_pairs),
                "per_gpu": "every rank builds its own batch of systems, no communication",
                "l2": "256 MiB buffer written between timed calls (untimed)",
            },
            "roofline": {
                "bound": "hbm",
                "kernel": "small_systems_kernel (count + emit passes; latency-bound workload)",
                "achieved": bytes_per_call / (device_ms * 1e-3) / 1e9,
                "peak": peak,
                "unit": "GB/s",
                "frac": bytes_per_call / (device_ms * 1e-3) / 1e9 / peak,
                "traffic": None,
                "note": "whole call (both passes, scan, read-back), not one kernel",
            },
            "e2e": {
                "value": total_pairs / (e2e_ms * 1e-3),
                "unit": "pairs/s",
                "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": len(points) * 24,
                "d2h_bytes_per_step": n_pairs * BYTES_PER_PAIR + (n_systems + 1) * 8,
            },
            "gpu_launches": 5 * args.steps,
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle

            oracle.build()
            cpu = oracle.ReferenceCPU()
            sample = min(n_systems, 4096)
            box = np.zeros((3, 3))
            t0 = time.perf_counter()
            cpu_pairs = 0
            for k in range(sample):
                cpu_pairs += cpu.run(points[offsets[k] : offsets[k + 1]], box, [False] * 3, cutoff, full, "ijSdD", n_threads=1)
            seconds = time.perf_counter() - t0
            line["cpu_baseline"] = {
                "value": cpu_pairs / seconds,
                "unit": "pairs/s",
                "cores": 1,
                "kind": "reference",
                "sample": f"first {sample} systems, one reference CPU call per system (n_threads=1), as the reference's callers do",
                "systems_per_s": sample / seconds,
            }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_sharded(args):
    """One large periodic system, slab-decomposed over the ranks: every step is
    one halo exchange (send/recv between neighbouring ranks) plus one local
    build per rank. Strong scaling: the system is the same at every N. With one
    rank the plain C ABI builds the whole system."""
    import torch
    import torch.distributed as dist

    import vesin_b200
    from vesin_b200._sharded import choose_axis, owner_of

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    n_atoms, cutoff, full, description = SHARDED_WORKLOADS[args.workload]
    points, box, periodic = workloads.liquid(n_atoms)
    if world > 1:
        axis = choose_axis(box, periodic)
        mine = np.nonzero(owner_of(points, box, axis, world) == rank)[0]
        d_points = torch.from_numpy(points[mine]).to(device)
        d_index = torch.from_numpy(mine).to(device)
        calculator = vesin_b200.ShardedNeighborList(cutoff=cutoff, full_list=full)

        def step():
            return calculator.compute(d_points, d_index, box, periodic, "PSdD", copy=False)[0].shape[0]
    else:
        d_points = torch.from_numpy(points).to(device)
        d_box = torch.from_numpy(box).to(device)
        d_periodic = torch.from_numpy(periodic).to(device)
        calculator = vesin_b200.NeighborList(cutoff=cutoff, full_list=full)

        def step():
            return calculator.compute(d_points, d_box, d_periodic, "PSdD", copy=False)[0].shape[0]
    del points

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(args.warmup, 3)):
        n_pairs = step()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    wall0 = time.perf_counter()
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        for k in range(args.steps):
            starts[k].record()
            n_pairs = step()
            stops[k].record()
        barrier()
    wall_ms = (time.perf_counter() - wall0) * 1e3 / args.steps
    device_ms = sum(a.elapsed_time(b) for a, b in zip(starts, stops)) / args.steps

    times = torch.tensor([device_ms, wall_ms], dtype=torch.float64, device=device)
    totals = torch.tensor([float(n_pairs), float(d_points.shape[0])], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    device_ms, wall_ms = times.tolist()
    total_pairs, total_points = totals.tolist()
    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
        total_bytes = algorithmic_bytes(int(total_points), int(total_pairs))
        achieved = total_bytes / (device_ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "neighbor pairs/s",
            "value": total_pairs / (device_ms * 1e-3),
            "unit": "pairs/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": device_ms,
            "wall_ms_per_step": wall_ms,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "f64",
            "data": "synthetic",
            "config": {
                "workload": description,
                "n_points": int(total_points),
                "n_pairs": int(total_pairs),
                "per_gpu": "one slab per rank; a step = halo exchange (NCCL send/recv) + local build" if world > 1 else "whole system on one GPU",
                "l2": "outputs (15 GB in total) exceed L2",
            },
            "roofline": {
                "bound": "hbm",
                "kernel": "whole step (all ranks)",
                "achieved": achieved,
                "peak": peak * world,
                "unit": "GB/s",
                "frac": achieved / (peak * world),
                "traffic": None,
            },
            "e2e": None,
            # pack_halo (2 kernels, ranks > 1), header, bounds, bin, 2 x scan, 2 x scatter, pairs
            "gpu_launches": (10 if world > 1 else 8) * args.steps,
            "clocks": clocks.summary(),
        }))
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="diamond512k", choices=sorted(WORKLOADS) + sorted(BATCH_WORKLOADS) + sorted(SHARDED_WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in BATCH_WORKLOADS:
        run_batch(args)
    elif args.workload in SHARDED_WORKLOADS:
        run_sharded(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
