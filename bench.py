"""
Benchmark of the neighbor-list build (one "step" = one build through the C ABI).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload diamond512k|diamond1000|...] [--no-extras]

Prints ONE JSON line (rank 0). Metric: neighbor pairs per second.

One GPU: the 512 000-atom diamond build (full list, fp64, quantities i j S d D),
inputs resident in HBM; `e2e` is the same build from pinned host buffers with
the host->device copy of the points and the device->host copy of every output
array inside the timed region. The line also carries a `workloads` block (the
other configurations, 10 timed builds each) and a `sharded` block (the
16.7 M-atom liquid on this one GPU: the base of the strong-scaling numbers).

N GPUs (one process per GPU, launched by torch.distributed.run): ONE periodic
diamond of N x 512 000 atoms, slab-decomposed over the ranks; a step is the halo
packing kernel, the NCCL send/recv exchange with both neighbours and the local
build on every rank (weak scaling: every rank owns 512 000 atoms at every N).
The ranks' lists are checked against the single-GPU build of the whole system
(order-independent checksum of every (i, j, S, d) row) and, up to two ranks,
against the reference CPU library; `parity: false` fails the run. The `sharded`
block times the 16.7 M-atom liquid slab-decomposed over the same ranks (strong
scaling) with the same checks.

`--impl reference` times the unmodified reference CPU path (oracle/_ref) on the
host cores on the same workload.
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
    # name: (generator, cutoff, full list, sorted, description)
    "diamond512k": (lambda: workloads.diamond(40), 5.0, True, False, "diamond 40x40x40 (512000 atoms), cutoff 5.0, full list, fp64, ijSdD"),
    "diamond512k_half": (lambda: workloads.diamond(40), 5.0, False, False, "diamond 40x40x40 (512000 atoms), cutoff 5.0, half list, fp64, ijSdD"),
    "diamond512k_f32": (lambda: workloads.diamond(40), 5.0, True, False, "diamond 40x40x40 (512000 atoms), cutoff 5.0, full list, fp32 in / fp32 d and D out (decisions in fp64), ijSdD"),
    "diamond512k_sorted": (lambda: workloads.diamond(40), 5.0, True, True, "diamond 40x40x40 (512000 atoms), cutoff 5.0, full list sorted by first index, fp64, ijSdD"),
    "diamond512k_canonical": (lambda: workloads.diamond(40), 5.0, True, "canonical", "diamond 40x40x40 (512000 atoms), cutoff 5.0, full list in canonical (i, j, S) order (sorted on the device), fp64, ijSdD"),
    "diamond110k": (lambda: workloads.diamond(24), 5.0, True, False, "diamond 24x24x24 (110592 atoms), cutoff 5.0, full list, fp64, ijSdD"),
    "diamond110k_sorted": (lambda: workloads.diamond(24), 5.0, True, True, "diamond 24x24x24 (110592 atoms), cutoff 5.0, full list sorted by first index, fp64, ijSdD"),
    "diamond110k_canonical": (lambda: workloads.diamond(24), 5.0, True, "canonical", "diamond 24x24x24 (110592 atoms), cutoff 5.0, full list in canonical (i, j, S) order, fp64, ijSdD"),
    "diamond1000": (lambda: workloads.diamond(5), 5.0, True, False, "diamond 5x5x5 (1000 atoms), cutoff 5.0, full list, fp64, ijSdD"),
    "triclinic64": (lambda: workloads.small_triclinic(), 9.0, True, False, "64 atoms in a small triclinic cell, cutoff 9.0, full list, fp64, ijSdD"),
    "liquid2m": (lambda: workloads.liquid(1 << 21), 6.0, False, False, "LJ-density liquid, 2097152 atoms, cutoff 6.0, half list, fp64 ABI, ijSdD"),
    "liquid262k": (lambda: workloads.liquid(1 << 18), 6.0, False, False, "LJ-density liquid, 262144 atoms, cutoff 6.0, half list, fp64, ijSdD"),
    "liquid2m_skin": (lambda: workloads.liquid(1 << 21), 6.0, False, False, "LJ-density liquid, 2097152 atoms, cutoff 6.0, skin 2.0 (steady state: cached candidates re-filtered, points moved by up to 0.2 A), half list, fp64, ijSdD"),
    "liquid262k_skin": (lambda: workloads.liquid(1 << 18), 6.0, False, False, "LJ-density liquid, 262144 atoms, cutoff 6.0, skin 2.0 (steady state), half list, fp64, ijSdD"),
    "liquid2m_f32": (lambda: workloads.liquid(1 << 21), 6.0, False, False, "LJ-density liquid, 2097152 atoms, cutoff 6.0, half list, fp32 in / fp32 d and D out, ijSdD"),
}

BATCH_WORKLOADS = {
    # name: (n_systems, cutoff, full list, description)
    "molecules16k": (16384, 4.0, True, "16384 non-periodic molecules of 16-64 atoms in a 6 A sphere, cutoff 4.0, full list, ijSdD, one batched call"),
    "molecules2k": (2048, 4.0, True, "2048 non-periodic molecules of 16-64 atoms in a 6 A sphere, cutoff 4.0, full list, ijSdD, one batched call"),
}

SHARDED_WORKLOADS = {
    # name: (n_atoms, cutoff, full list, float32 I/O, description)
    "liquid16m": (1 << 24, 6.0, False, True, "LJ-density liquid, 16777216 atoms, cutoff 6.0, half list, fp32 in / fp32 d and D out (decisions in fp64), ijSdD, slab-decomposed over the ranks"),
    "liquid2m_sharded": (1 << 21, 6.0, False, True, "LJ-density liquid, 2097152 atoms, cutoff 6.0, half list, fp32 in / fp32 d and D out, ijSdD, slab-decomposed over the ranks"),
}

# what the default run reports besides the headline
EXTRA_WORKLOADS = ("diamond512k_half", "diamond512k_f32", "diamond512k_sorted", "diamond512k_canonical", "diamond1000", "triclinic64", "liquid2m", "liquid2m_f32", "liquid2m_skin")
EXTRA_STEPS = 10


def bytes_per_pair(float_io):
    # i, j as size_t; S int32[3]; d; D
    return 16 + 12 + (4 if float_io else 8) * 4


def bytes_per_point(float_io):
    return 12 if float_io else 24


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


def hbm_peak():
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as fd:
            return float(json.load(fd)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback"


def measured_traffic(kernel, n_pairs):
    """DRAM traffic of one launch, scaled by pairs from the committed ncu
    capture of the same kernel (profiles/dram_traffic.json, written with the
    profile it summarises); None when no capture covers the kernel."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None, None
    with open(path) as fd:
        captures = json.load(fd)
    capture = captures.get(kernel)
    if capture is None:
        return None, None
    traffic = (capture["dram_bytes_read"] + capture["dram_bytes_write"]) / capture["pairs"] * n_pairs
    return traffic, f"bytes per launch, scaled by pairs from the ncu capture of {capture['workload']} ({capture['profile']})"


# ---------------------------------------------------------------------------
# reference arm: the reference's CPU path on the host cores
# ---------------------------------------------------------------------------


def time_reference_cpu(system, cutoff, full, steps, warmup, budget_s, sorted=False):
    sorted = bool(sorted)
    """Reference CPU path on all host cores; returns (pairs, seconds per build,
    builds timed, threads). The thread count is passed explicitly: launchers
    such as torch.distributed.run export OMP_NUM_THREADS=1, which the
    reference would otherwise obey (vesin/src/vesin.cpp:18-39)."""
    from oracle import oracle

    oracle.build()
    cpu = oracle.ReferenceCPU()
    points, box, periodic = system
    threads = host_cores()
    n_pairs = 0
    started = time.perf_counter()
    for _ in range(warmup):
        n_pairs = cpu.run(points, box, periodic, cutoff, full, "ijSdD", n_threads=threads, sorted=sorted)
        if time.perf_counter() - started > budget_s / 2:
            break
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        n_pairs = cpu.run(points, box, periodic, cutoff, full, "ijSdD", n_threads=threads, sorted=sorted)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - started > budget_s:
            break
    return n_pairs, float(np.mean(times)), len(times), threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload in BATCH_WORKLOADS:
        run_reference_batch(args)
        return
    world = max(1, args.gpus)
    if args.workload in SHARDED_WORKLOADS:
        n_atoms, cutoff, full, _, description = SHARDED_WORKLOADS[args.workload]
        # a bounded sample of the workload: the same liquid with at most 2 M atoms
        sample_atoms = min(n_atoms, 1 << 21)
        system = workloads.liquid(sample_atoms)
        sample = f"the same liquid with {sample_atoms} atoms (the CPU cost per atom does not depend on the size)"
        sorted_list = False
    else:
        make, cutoff, full, sorted_list, description = WORKLOADS[args.workload]
        system = make()
        sample = "full builds of the workload"
        if world > 1 and args.workload == "diamond512k":
            description = sharded_diamond_description(world)
            sample = f"one of the {world} identical 512000-atom blocks of the system as a periodic system of its own (same work per atom)"
    n_pairs, seconds, timed, threads = time_reference_cpu(system, cutoff, full, args.steps, args.warmup, budget_s=240.0, sorted=sorted_list)
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
            "cores": threads,
            "kind": "reference",
            "sample": f"{timed} builds, reference CPU path, n_threads={threads}: {sample}",
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


# ---------------------------------------------------------------------------
# the GPU arm
# ---------------------------------------------------------------------------


class Harness:
    """Process group, device, L2 flush buffer and the timing loop."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        import vesin_b200

        self.torch = torch
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.device)
        self.lib = vesin_b200.get_library()
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)  # > 126 MB of L2
        self.peak, self.peak_source = hbm_peak()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.device)

    def time_steps(self, step, steps):
        """Device milliseconds of `steps` calls of step(), summed; the L2 is
        flushed (untimed) before every call. CUDA events on torch's current
        stream: the library's streams are ordered after it and every call is
        complete on return."""
        torch = self.torch
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        result = None
        for k in range(steps):
            self.flush.fill_(k & 0xFF)  # untimed: evicts L2 between builds
            starts[k].record()
            result = step()
            stops[k].record()
        torch.cuda.synchronize(self.device)
        self.last_step_ms = [a.elapsed_time(b) for a, b in zip(starts, stops)]
        return sum(self.last_step_ms), result

    def max_over_ranks(self, values):
        tensor = self.torch.tensor(values, dtype=self.torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(tensor, op=self.dist.ReduceOp.MAX)
        return tensor.tolist()

    def sum_over_ranks(self, values):
        tensor = self.torch.tensor(values, dtype=self.torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(tensor, op=self.dist.ReduceOp.SUM)
        return tensor.tolist()

    def sum_checksums(self, checksum):
        """Sum (mod 2^64) of the ranks' checksum words; the row counts add up.
        The words travel as 32-bit halves so that no 64-bit sum can overflow."""
        halves = []
        for word in checksum[:3]:
            halves += [word & 0xFFFFFFFF, word >> 32]
        halves.append(checksum[3])
        tensor = self.torch.tensor(halves, dtype=self.torch.int64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(tensor, op=self.dist.ReduceOp.SUM)
        halves = [int(v) for v in tensor.tolist()]
        words = [(halves[2 * k] + (halves[2 * k + 1] << 32)) % (1 << 64) for k in range(3)]
        return tuple(words) + (halves[6],)

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


class PlainBuild:
    """One system on this rank's GPU through vesin_neighbors (or the fp32 entry point)."""

    def __init__(self, harness, system, cutoff, full, float_io=False, sorted_list=False, skin=0.0):
        from vesin_b200._c_api import VesinCUDA, VesinDevice, VesinNeighborList, VesinOptions

        torch = harness.torch
        self.harness = harness
        points, box, periodic = system
        self.float_io = float_io
        self.n_points = len(points)
        dtype = np.float32 if float_io else np.float64
        self.h_points = torch.from_numpy(np.ascontiguousarray(points, dtype=dtype)).pin_memory()
        self.d_points = self.h_points.to(harness.device)
        self.d_box = torch.from_numpy(np.ascontiguousarray(box, dtype=dtype)).to(harness.device)
        self.d_periodic = torch.from_numpy(np.ascontiguousarray(periodic, dtype=np.bool_)).to(harness.device)
        self.entry_point = harness.lib.vesin_b200_neighbors_f32 if float_io else harness.lib.vesin_neighbors
        if sorted_list == "canonical":
            self.entry_point = harness.lib.vesin_b200_neighbors_canonical
        options = VesinOptions()
        options.cutoff = cutoff
        options.full = full
        options.sorted = bool(sorted_list)
        options.algorithm = 0
        options.n_threads = 0
        options.return_shifts = True
        options.return_distances = True
        options.return_vectors = True
        options.skin = skin
        self.options = options
        # with a skin the timed builds alternate between the points the candidates were built for
        # and a copy moved by up to 0.2 A per coordinate: every step re-filters cached candidates
        self.moved = None
        self.calls = 0
        if skin > 0.0:
            shift = np.random.default_rng(11).uniform(-0.2, 0.2, np.shape(points)).astype(dtype)
            self.moved = torch.from_numpy(np.ascontiguousarray(points, dtype=dtype) + shift).to(harness.device)
        self.c_device = VesinDevice(VesinCUDA, harness.local_rank)
        self.neighbors = VesinNeighborList()
        self.error = ctypes.c_char_p()

    def build(self, points_tensor=None):
        tensor = self.d_points if points_tensor is None else points_tensor
        if points_tensor is None and self.moved is not None:
            self.calls += 1
            tensor = self.moved if self.calls % 2 == 0 else self.d_points
        status = self.entry_point(
            tensor.data_ptr(), self.n_points, self.d_box.data_ptr(), self.d_periodic.data_ptr(), self.c_device, self.options,
            ctypes.byref(self.neighbors), ctypes.byref(self.error),
        )
        if status != 0:
            raise RuntimeError(self.error.value.decode("utf8"))
        return self.neighbors.length

    def checksum(self):
        from vesin_b200._sharded import list_checksum

        return list_checksum(self.neighbors)

    def stage_times(self, steps):
        """Mean device time of every stage over `steps` builds (the library's own
        CUDA events on its stream; a separate, untimed loop)."""
        from vesin_b200._c_api import N_STAGES, STAGE_NAMES

        lib = self.harness.lib
        total = np.zeros(N_STAGES)
        buffer = (ctypes.c_double * N_STAGES)()
        lib.vesin_b200_set_profiling(1)
        for k in range(steps):
            self.harness.flush.fill_(k & 0xFF)
            self.build()
            if lib.vesin_b200_stage_times(ctypes.byref(self.neighbors), buffer) == 0:
                total += np.array(buffer[:])
        lib.vesin_b200_set_profiling(0)
        return {name: float(ms) for name, ms in zip(STAGE_NAMES, total / steps)}

    def outputs(self):
        """Zero-copy torch views of the four output arrays."""
        from vesin_b200._neighbors import _view

        n = self.neighbors.length
        device = self.harness.device
        value = "<f4" if self.float_io else "<f8"
        return [
            _view(self.neighbors.pairs, (n, 2), "<u8", device, self.neighbors).view(self.harness.torch.int64),
            _view(self.neighbors.shifts, (n, 3), "<i4", device, self.neighbors),
            _view(self.neighbors.distances, (n,), value, device, self.neighbors),
            _view(self.neighbors.vectors, (n, 3), value, device, self.neighbors),
        ]

    def free(self):
        self.harness.lib.vesin_free(ctypes.byref(self.neighbors))


def end_to_end(harness, h_inputs, d_staging, step, outputs, steps):
    """ms per step of: host->device copy of the inputs (pinned), the build, and
    the device->host copy of every output array into pinned host memory."""
    torch = harness.torch
    step_result = [None]

    def one():
        for host, staged in zip(h_inputs, d_staging):
            staged.copy_(host, non_blocking=True)
        torch.cuda.current_stream(harness.device).synchronize()
        step_result[0] = step(*d_staging)
        for host, dev in zip(host_out, outputs()):
            host.copy_(dev, non_blocking=True)
        torch.cuda.current_stream(harness.device).synchronize()

    # size the host arrays from a first build
    for host, staged in zip(h_inputs, d_staging):
        staged.copy_(host)
    step(*d_staging)
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outputs()]
    one()
    harness.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    harness.barrier()
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    h2d = sum(t.numel() * t.element_size() for t in h_inputs)
    return e0.elapsed_time(e1) / steps, h2d, d2h


def measure_extra(harness, name):
    """One entry of the `workloads` block: EXTRA_STEPS timed builds."""
    if name in BATCH_WORKLOADS:
        return measure_extra_batch(harness, name)
    make, cutoff, full, sorted_list, description = WORKLOADS[name]
    float_io = name.endswith("_f32")
    build = PlainBuild(harness, make(), cutoff, full, float_io, sorted_list, skin=2.0 if name.endswith("_skin") else 0.0)
    for _ in range(3):
        n_pairs = build.build()
    device_ms, n_pairs = harness.time_steps(build.build, EXTRA_STEPS)
    ms = device_ms / EXTRA_STEPS
    stages = build.stage_times(5)
    kernel_ms = stages["count"] + stages["emit"]
    algorithmic = build.n_points * bytes_per_point(float_io) + n_pairs * bytes_per_pair(float_io)
    entry = {
        "workload": description,
        "n_points": build.n_points,
        "n_pairs": int(n_pairs),
        "steps": EXTRA_STEPS,
        "ms_per_step": ms,
        "pairs_per_s": n_pairs / (ms * 1e-3),
        "kernel_ms": kernel_ms,
        "stages_ms": stages,
        "bytes": algorithmic,
        "frac": algorithmic / (ms * 1e-3) / 1e9 / harness.peak,
        "kernel_frac": (algorithmic / (kernel_ms * 1e-3) / 1e9 / harness.peak) if kernel_ms > 0 else None,
    }
    build.free()
    return entry


def measure_extra_batch(harness, name):
    import vesin_b200

    n_systems, cutoff, full, description = BATCH_WORKLOADS[name]
    points, offsets = workloads.molecule_batch(n_systems=n_systems, seed=4)
    d_points = harness.torch.from_numpy(points).to(harness.device)
    calculator = vesin_b200.BatchNeighborList(cutoff=cutoff, full_list=full)

    def step():
        # the C call alone, like the other workloads
        calculator.build(d_points, offsets, quantities="PSdD")
        return calculator.n_pairs

    for _ in range(3):
        n_pairs = step()
    device_ms, _ = harness.time_steps(step, EXTRA_STEPS)
    ms = device_ms / EXTRA_STEPS
    algorithmic = len(points) * 24 + n_pairs * bytes_per_pair(False)
    return {
        "workload": description,
        "n_points": int(len(points)),
        "n_pairs": n_pairs,
        "steps": EXTRA_STEPS,
        "ms_per_step": ms,
        "pairs_per_s": n_pairs / (ms * 1e-3),
        "systems_per_s": n_systems / (ms * 1e-3),
        "bytes": algorithmic,
        "frac": algorithmic / (ms * 1e-3) / 1e9 / harness.peak,
    }


def reference_checksum(system, cutoff, full, float_io):
    """Checksum of the list the reference CPU library builds (all host cores)."""
    from oracle import oracle
    from vesin_b200._sharded import checksum_of_arrays

    oracle.build()
    points, box, periodic = system
    if float_io:
        points = points.astype(np.float32).astype(np.float64)
        box = box.astype(np.float32).astype(np.float64)
    result = oracle.ReferenceCPU().compute(points, box, periodic, cutoff, full, "ijSd", n_threads=host_cores())
    distances = result["d"].astype(np.float32) if float_io else result["d"]
    return checksum_of_arrays(result["i"], result["j"], result["S"], distances)


def sharded_diamond_description(world):
    return (
        f"diamond 40x40x{40 * world} ({512000 * world} atoms: {world} blocks of 512000 along z, same generator and seed per block), "
        f"cutoff 5.0, full list, fp64, ijSdD, ONE periodic system slab-decomposed over {world} ranks"
    )


def diamond_blocks(world):
    """The N-block diamond: block b is the 512 000-atom diamond moved by b box
    lengths along z."""
    points, box, periodic = workloads.diamond(40)
    length = box[2, 2]
    blocks = [points + np.array([0.0, 0.0, b * length]) for b in range(world)]
    box = box.copy()
    box[2, 2] = length * world
    return np.concatenate(blocks), box, periodic


class ShardedBuild:
    """This rank's slab of one system through vesin_b200.ShardedNeighborList."""

    def __init__(self, harness, system, cutoff, full, float_io):
        import vesin_b200
        from vesin_b200._sharded import owner_of, slab_geometry

        torch = harness.torch
        points, box, periodic = system
        dtype = np.float32 if float_io else np.float64
        self.harness = harness
        self.float_io = float_io
        used_points = points.astype(dtype).astype(np.float64) if float_io else points
        self.box = np.ascontiguousarray(box, dtype=dtype)
        self.periodic = periodic
        axis, _, _ = slab_geometry(self.box.astype(np.float64), periodic, cutoff)
        mine = np.nonzero(owner_of(used_points, self.box.astype(np.float64), axis, harness.world) == harness.rank)[0]
        self.n_owned = len(mine)
        self.h_points = torch.from_numpy(np.ascontiguousarray(points[mine], dtype=dtype)).pin_memory()
        self.h_index = torch.from_numpy(mine.astype(np.int64)).pin_memory()
        self.d_points = self.h_points.to(harness.device)
        self.d_index = self.h_index.to(harness.device)
        self.calculator = vesin_b200.ShardedNeighborList(cutoff=cutoff, full_list=full)

    def build(self, points_tensor=None, index_tensor=None):
        """The C call (vesin_b200_sharded_neighbors), like PlainBuild.build."""
        points_tensor = self.d_points if points_tensor is None else points_tensor
        index_tensor = self.d_index if index_tensor is None else index_tensor
        return self.calculator.build(points_tensor, index_tensor, self.box, self.periodic, "PSdD")

    def outputs(self):
        torch = self.harness.torch
        return list(self.calculator.outputs(self.harness.device, "PSdD", torch.float32 if self.float_io else torch.float64))

    def checksum(self):
        return self.calculator.checksum()

    def stage_times(self, steps):
        import vesin_b200

        total = {}
        vesin_b200.set_profiling(True)
        for k in range(steps):
            self.harness.flush.fill_(k & 0xFF)
            self.build()
            for key, value in (self.calculator.stage_times() or {}).items():
                total[key] = total.get(key, 0.0) + value
        vesin_b200.set_profiling(False)
        return {key: value / steps for key, value in total.items()}

    def free(self):
        self.calculator.close()


def single_gpu_reference_build(harness, system, cutoff, full, float_io, steps=0):
    """Rank 0 builds the WHOLE system on its own GPU: the checksum every sharded
    result is compared with and, when `steps` > 0, the one-GPU time of the same
    system. The other ranks wait."""
    result = None
    if harness.rank == 0:
        build = PlainBuild(harness, system, cutoff, full, float_io)
        for _ in range(3 if steps else 1):
            n_pairs = build.build()
        result = {"n_pairs": int(n_pairs), "checksum": build.checksum()}
        if steps:
            device_ms, _ = harness.time_steps(build.build, steps)
            result["ms_per_step"] = device_ms / steps
        build.free()
        harness.torch.cuda.empty_cache()
    harness.barrier()
    return result


def run_sharded_leg(harness, name, steps, reference_parity):
    """One system slab-decomposed over all ranks (strong scaling), with parity:
    the summed checksums of the ranks against the one-GPU build of the same
    system and, when asked, against the reference CPU library's list."""
    n_atoms, cutoff, full, float_io, description = SHARDED_WORKLOADS[name]
    system = workloads.liquid(n_atoms)
    peak = harness.peak
    entry = {"workload": description, "n_points": n_atoms, "steps": steps}
    if harness.world == 1:
        build = PlainBuild(harness, system, cutoff, full, float_io)
        for _ in range(3):
            n_pairs = build.build()
        device_ms, _ = harness.time_steps(build.build, steps)
        ms = device_ms / steps
        stages = build.stage_times(3)
        checksum = build.checksum()
        build.free()
        entry.update({
            "n_pairs": int(n_pairs), "ms_per_step": ms, "pairs_per_s": n_pairs / (ms * 1e-3), "stages_ms": stages,
            "per_gpu": "the whole system on one GPU (vesin_b200_neighbors_f32): the base of speedup_vs_1gpu at N > 1",
        })
        total_pairs = n_pairs
    else:
        single = single_gpu_reference_build(harness, system, cutoff, full, float_io, steps=min(steps, 5))
        build = ShardedBuild(harness, system, cutoff, full, float_io)
        for _ in range(3):
            n_pairs = build.build()
        harness.barrier()
        device_ms, _ = harness.time_steps(build.build, steps)
        harness.barrier()
        stages = build.stage_times(3)
        checksum = harness.sum_checksums(build.checksum())
        (ms,) = harness.max_over_ranks([device_ms / steps])
        (total_pairs,) = harness.sum_over_ranks([float(n_pairs)])
        stage_names = sorted(stages)
        stage_max = dict(zip(stage_names, harness.max_over_ranks([stages[key] for key in stage_names])))
        build.free()
        entry.update({
            "n_pairs": int(total_pairs), "ms_per_step": ms, "pairs_per_s": total_pairs / (ms * 1e-3),
            "pack_ms": stage_max.get("pack"), "exchange_ms": stage_max.get("exchange"),
            "build_ms": sum(value for key, value in stage_max.items() if key not in ("pack", "exchange")),
            "stages_ms": stage_max,
            "per_gpu": "one slab per rank; a step = halo packing kernel + NCCL send/recv with both neighbours + local build, max over ranks",
        })
        if harness.rank == 0:
            entry["one_gpu_ms_per_step"] = single["ms_per_step"]
            entry["speedup_vs_1gpu"] = single["ms_per_step"] / ms
            entry["parity_single_gpu"] = bool(tuple(single["checksum"]) == tuple(checksum))
    algorithmic = n_atoms * bytes_per_point(float_io) + total_pairs * bytes_per_pair(float_io)
    entry["bytes"] = algorithmic
    entry["frac"] = algorithmic / (entry["ms_per_step"] * 1e-3) / 1e9 / (peak * harness.world)
    if reference_parity and harness.rank == 0:
        entry["parity_reference_cpu"] = bool(tuple(reference_checksum(system, cutoff, full, float_io)) == tuple(checksum))
    harness.barrier()
    return entry


def run_ours(args):
    harness = Harness()
    world, rank = harness.world, harness.rank
    name = args.workload
    make, cutoff, full, sorted_list, description = WORKLOADS[name]
    float_io = name.endswith("_f32")
    sharded = world > 1 and name == "diamond512k"

    if sharded:
        system = diamond_blocks(world)
        description = sharded_diamond_description(world)
        build = ShardedBuild(harness, system, cutoff, full, float_io)
        n_points_rank = build.n_owned
        per_gpu = ("one slab of the system per rank (about 512000 owned atoms); a step = halo packing kernel + NCCL send/recv "
                   "exchange with both neighbours + local build of the owned atoms' pairs")
        launches_per_step = 9  # pack, header, bin (owned), bin (halo), 2 x scan, 2 x scatter, pairs (+ the NCCL send/recv kernel)
    else:
        system = make()
        build = PlainBuild(harness, system, cutoff, full, float_io, sorted_list, skin=2.0 if name.endswith("_skin") else 0.0)
        n_points_rank = build.n_points
        per_gpu = "one independent copy of the system per GPU, no communication" if world > 1 else "the whole system on one GPU"
        launches_per_step = 7  # header (reset, zero, box check), bin (+ point checks), 2 x scan, 2 x scatter, pairs

    # ---- warm-up (also sizes the workspace and the output arrays) ----
    for _ in range(max(args.warmup, 3)):
        n_pairs = build.build()

    # ---- timed region 1: device-resident inputs ----
    clocks = ClockSampler(physical_gpu_index(harness.local_rank))
    harness.barrier()
    wall0 = time.perf_counter()
    with clocks:
        device_ms, n_pairs = harness.time_steps(build.build, args.steps)
        step_ms = sorted(harness.last_step_ms)
        harness.barrier()
    wall = time.perf_counter() - wall0

    # ---- per-kernel times of the same builds ----
    stages = build.stage_times(max(1, min(args.steps, 20)))
    harness.barrier()

    # ---- parity of the sharded result ----
    parity = None
    if sharded:
        checksum = harness.sum_checksums(build.checksum())
        single = single_gpu_reference_build(harness, system, cutoff, full, float_io)
        if rank == 0:
            parity = {"single_gpu": bool(tuple(single["checksum"]) == tuple(checksum)), "rows": checksum[3], "single_gpu_rows": single["n_pairs"]}
            if world <= 2:
                parity["reference_cpu"] = bool(tuple(reference_checksum(system, cutoff, full, float_io)) == tuple(checksum))
        harness.barrier()

    # ---- timed region 2: end to end from pinned host buffers ----
    e2e_steps = max(1, min(args.steps, 5))
    if sharded:
        staging = [harness.torch.empty_like(build.d_points), harness.torch.empty_like(build.d_index)]
        e2e_ms, h2d, d2h = end_to_end(harness, [build.h_points, build.h_index], staging, build.build, build.outputs, e2e_steps)
    else:
        staging = [harness.torch.empty_like(build.d_points)]
        e2e_ms, h2d, d2h = end_to_end(harness, [build.h_points], staging, build.build, build.outputs, e2e_steps)

    # ---- reduce over ranks: the slowest rank sets the time ----
    device_ms, e2e_ms, wall_ms = harness.max_over_ranks([device_ms, e2e_ms, wall * 1e3])
    total_pairs, total_points, h2d_total, d2h_total = harness.sum_over_ranks([float(n_pairs), float(n_points_rank), float(h2d), float(d2h)])
    stage_names = sorted(stages)
    stages = dict(zip(stage_names, harness.max_over_ranks([stages[key] for key in stage_names])))
    build.free()
    harness.torch.cuda.empty_cache()

    line = None
    if rank == 0:
        ms_per_step = device_ms / args.steps
        value = total_pairs / (ms_per_step * 1e-3)
        # roofline of the pair kernel on one GPU (rank 0's launch)
        bytes_per_launch = n_points_rank * bytes_per_point(float_io) + int(n_pairs) * bytes_per_pair(float_io)
        kernel_ms = stages["count"] + stages["emit"]
        achieved = bytes_per_launch / (kernel_ms * 1e-3) / 1e9 if kernel_ms > 0 else None
        total_bytes = total_points * bytes_per_point(float_io) + total_pairs * bytes_per_pair(float_io)
        traffic, traffic_unit = (None, None)
        if full and not float_io and not sorted_list:
            traffic, traffic_unit = measured_traffic("pairs_kernel", int(n_pairs))
        line = {
            "metric": "neighbor pairs/s",
            "value": value,
            "unit": "pairs/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "step_ms": {"min": step_ms[0], "median": step_ms[len(step_ms) // 2], "max": step_ms[-1], "of": "rank 0's timed steps"},
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f64" if not float_io else "f64 decisions, f32 storage",
            "data": "synthetic",
            "config": {
                "workload": description,
                "n_points": int(total_points),
                "n_pairs": int(total_pairs),
                "per_gpu": per_gpu,
                "l2": "256 MiB buffer written between timed builds (untimed); outputs (2.7 GB per GPU) exceed L2",
            },
            "roofline": {
                "bound": "hbm",
                "kernel": "pairs_kernel" if not sorted_list else "count_kernel + emit_kernel",
                "achieved": achieved,
                "peak": harness.peak,
                "unit": "GB/s",
                "frac": (achieved / harness.peak) if achieved else None,
                "peak_source": harness.peak_source,
                "traffic": traffic,
                "traffic_unit": traffic_unit,
                "bytes_per_launch": bytes_per_launch,
                "kernel_ms": kernel_ms,
                "whole_build_frac": total_bytes / (ms_per_step * 1e-3) / 1e9 / (harness.peak * world),
            },
            "stages_ms": stages,
            "e2e": {
                "value": total_pairs / (e2e_ms * 1e-3),
                "unit": "pairs/s",
                "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(h2d_total),
                "d2h_bytes_per_step": int(d2h_total),
            },
            "gpu_launches": launches_per_step * args.steps * world,
            "wall_ms_per_step": wall_ms / args.steps,
            "clocks": clocks.summary(),
        }
        if parity is not None:
            line["parity"] = bool(all(value for key, value in parity.items() if key in ("single_gpu", "reference_cpu")))
            line["parity_checks"] = parity

    # ---- the other configurations ----
    if not args.no_extras and name == "diamond512k":
        if world == 1:
            extras = {}
            for extra in EXTRA_WORKLOADS + ("molecules16k",):
                extras[extra] = measure_extra(harness, extra)
                harness.torch.cuda.empty_cache()
            line["workloads"] = extras
        leg = run_sharded_leg(harness, "liquid16m", EXTRA_STEPS, reference_parity=False)
        check = run_sharded_leg(harness, "liquid2m_sharded", 3, reference_parity=True)
        if rank == 0:
            leg["liquid2m_check"] = {key: check[key] for key in check if key.startswith("parity") or key in ("n_pairs", "ms_per_step", "workload")}
            line["sharded"] = leg
            if world > 1:
                flags = [leg.get("parity_single_gpu"), check.get("parity_single_gpu"), check.get("parity_reference_cpu")]
                line["parity"] = bool(line.get("parity", True) and all(flag is not False for flag in flags) and None not in flags)

    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            points, box, periodic = system
            used = points.astype(np.float32).astype(np.float64) if float_io else points
            used_box = box.astype(np.float32).astype(np.float64) if float_io else box
            cpu_pairs, cpu_seconds, timed, threads = time_reference_cpu((used, used_box, periodic), cutoff, full, 2, 1, budget_s=45.0, sorted=sorted_list)
            assert cpu_pairs == n_pairs, f"CPU reference found {cpu_pairs} pairs, GPU {n_pairs}"
            line["cpu_baseline"] = {
                "value": cpu_pairs / cpu_seconds,
                "unit": "pairs/s",
                "cores": threads,
                "kind": "reference",
                "sample": f"{timed} full builds of the same workload after 1 warm-up, reference CPU path (oracle/_ref), n_threads={threads}",
                "ms_per_build": cpu_seconds * 1e3,
            }
        print(json.dumps(line))
    harness.close()
    if rank == 0 and line.get("parity") is False:
        sys.exit("parity check failed: the sharded lists differ from the single-GPU / reference lists")


def run_batch(args):
    """Batch of independent molecules: one call per rank on its share of the
    systems (contiguous chunks balanced by atoms, no communication)."""
    import vesin_b200

    harness = Harness()
    torch = harness.torch
    world, rank, device = harness.world, harness.rank, harness.device
    n_systems, cutoff, full, description = BATCH_WORKLOADS[args.workload]
    # weak scaling: every rank brings n_systems systems of its own
    points, offsets = workloads.molecule_batch(n_systems=n_systems, seed=4 + rank)
    h_points = torch.from_numpy(points).pin_memory()
    d_points = h_points.to(device)
    calculator = vesin_b200.BatchNeighborList(cutoff=cutoff, full_list=full)

    for _ in range(max(args.warmup, 3)):
        calculator.build(d_points, offsets, quantities="PSdD")
    n_pairs = calculator.n_pairs
    clocks = ClockSampler(physical_gpu_index(harness.local_rank))
    harness.barrier()
    with clocks:
        device_ms, _ = harness.time_steps(lambda: calculator.build(d_points, offsets, quantities="PSdD"), args.steps)
        harness.barrier()
    device_ms /= args.steps

    last = [None]

    def step(staged):
        last[0] = calculator.compute(staged, offsets, quantities="PSdD", copy=False)

    def outputs():
        results, pair_offsets = last[0]
        return list(results) + [pair_offsets]

    e2e_ms, h2d, d2h = end_to_end(harness, [h_points], [torch.empty_like(d_points)], step, outputs, max(1, min(args.steps, 10)))
    device_ms, e2e_ms = harness.max_over_ranks([device_ms, e2e_ms])
    total_pairs, total_systems, total_points = harness.sum_over_ranks([float(n_pairs), float(n_systems), float(len(points))])
    if rank == 0:
        bytes_per_call = len(points) * 24 + n_pairs * bytes_per_pair(False)
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
                "peak": harness.peak,
                "unit": "GB/s",
                "frac": bytes_per_call / (device_ms * 1e-3) / 1e9 / harness.peak,
                "traffic": None,
                "note": "whole call (both passes, scan, read-back), not one kernel",
            },
            "e2e": {
                "value": total_pairs / (e2e_ms * 1e-3),
                "unit": "pairs/s",
                "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h,
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
    harness.close()


def run_sharded(args):
    """One of the strong-scaling workloads alone (`--workload liquid16m`)."""
    harness = Harness()
    entry = run_sharded_leg(harness, args.workload, args.steps, reference_parity=args.workload != "liquid16m")
    if harness.rank == 0:
        line = {
            "metric": "neighbor pairs/s",
            "value": entry["pairs_per_s"],
            "unit": "pairs/s",
            "n_gpus": harness.world,
            "steps": args.steps,
            "warmup": 3,
            "ms_per_step": entry["ms_per_step"],
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "f64 decisions, f32 storage",
            "data": "synthetic",
            "config": {"workload": entry["workload"], "n_points": entry["n_points"], "n_pairs": entry["n_pairs"], "per_gpu": entry["per_gpu"],
                       "l2": "256 MiB buffer written between timed builds (untimed)"},
            "roofline": {"bound": "hbm", "kernel": "whole step (all ranks)", "achieved": entry["bytes"] / (entry["ms_per_step"] * 1e-3) / 1e9,
                         "peak": harness.peak * harness.world, "unit": "GB/s", "frac": entry["frac"], "traffic": None},
            "sharded": entry,
            "e2e": None,
            "gpu_launches": (9 if harness.world > 1 else 7) * args.steps * harness.world,
        }
        flags = [value for key, value in entry.items() if key.startswith("parity")]
        if flags:
            line["parity"] = bool(all(flags))
        print(json.dumps(line))
    harness.close()
    if harness.rank == 0 and line.get("parity") is False:
        sys.exit("parity check failed")


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="diamond512k", choices=sorted(WORKLOADS) + sorted(BATCH_WORKLOADS) + sorted(SHARDED_WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-extras", action="store_true", help="only the headline: no `workloads` and no `sharded` block")
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
