"""GPU test of the list build that allocates nothing
(vesin_b200_neighbors_no_alloc, include/vesin_b200.h).

That entry point exists for callers that may not call cudaMalloc when they
need a neighbor list (an application that owns all device memory through its
own pool, a loop with a hard latency bound, a plugin inside a framework that
forbids allocations outside its allocator): the caller brings the output
arrays and the kernels work in a fixed scratch array inside the library. The
test calls it through the C ABI and checks the result against vesin_neighbors
on the same inputs and against the CPU oracle: indices and shifts bit for bit
after canonical sorting, distances and vectors within the 1e-12 relative
tolerance of the other fp64 tests. Two calls are made in a
row on different systems, the second smaller than the first, so that data left
in the shared scratch by the first call would show up as wrong pairs.

This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""

import ctypes

import numpy as np
import pytest

from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu

RTOL_FP64 = 1e-12


def _existing_entry_point(torch, points, box, periodic, cutoff, full):
    from gpu_utils import gpu_compute

    return gpu_compute(points, box, periodic, cutoff, full, "ijSdD")


def _no_alloc(torch, lib, points, box, periodic, cutoff, full, capacity, offset_bytes=(0, 0, 0, 0)):
    """`offset_bytes`: start the four output arrays that many bytes into their
    allocation (pairs, shifts, distances, vectors), to test alignment handling."""
    from vesin_b200._c_api import get_library

    lib = get_library()
    device = torch.device("cuda", 0)
    d_points = torch.tensor(np.asarray(points, dtype=np.float64).reshape(-1, 3), device=device)
    d_box = torch.tensor(np.asarray(box, dtype=np.float64), device=device)
    d_periodic = torch.tensor(np.asarray(periodic, dtype=bool), device=device)
    # the caller owns the outputs
    def shifted(count, dtype, fill, offset):
        item = torch.empty((), dtype=dtype).element_size()
        assert offset % item == 0
        return torch.full((count + offset // item,), fill, dtype=dtype, device=device)[offset // item :]

    pairs = shifted(2 * capacity, torch.int64, -1, offset_bytes[0]).view(capacity, 2)
    shifts = shifted(3 * capacity, torch.int32, 99, offset_bytes[1]).view(capacity, 3)
    distances = shifted(capacity, torch.float64, -1.0, offset_bytes[2])
    vectors = shifted(3 * capacity, torch.float64, -1.0, offset_bytes[3]).view(capacity, 3)
    torch.cuda.synchronize()
    length = ctypes.c_size_t(0)
    error = ctypes.c_char_p()
    status = lib.vesin_b200_neighbors_no_alloc(
        d_points.data_ptr(), d_points.shape[0], d_box.data_ptr(), d_periodic.data_ptr(), 0, float(cutoff), bool(full), capacity,
        pairs.data_ptr(), shifts.data_ptr(), distances.data_ptr(), vectors.data_ptr(), ctypes.byref(length), ctypes.byref(error),
    )
    message = error.value.decode() if error.value else None
    n = min(length.value, capacity)
    result = {
        "i": pairs[:n, 0].cpu().numpy(),
        "j": pairs[:n, 1].cpu().numpy(),
        "S": shifts[:n].cpu().numpy(),
        "d": distances[:n].cpu().numpy(),
        "D": vectors[:n].cpu().numpy(),
    }
    return status, message, length.value, result


def test_two_calls_in_a_row_match_vesin_neighbors():
    import torch

    assert torch.cuda.is_available()
    calls = [
        (W.diamond(6, seed=17), 5.0, True),      # 1728 points, full list
        (W.small_triclinic(48, seed=9), 7.5, False),  # smaller system, many images, half list
    ]
    for (points, box, periodic), cutoff, full in calls:
        expected = _existing_entry_point(torch, points, box, periodic, cutoff, full)
        capacity = len(expected["i"]) + 100
        status, message, length, got = _no_alloc(torch, None, points, box, periodic, cutoff, full, capacity)
        assert status == 0, message
        assert length == len(expected["i"])
        O.assert_same(got, expected, RTOL_FP64, "no-alloc build against vesin_neighbors")
        # both entry points share kernels: the CPU oracle is the independent check
        oracle = O.restated_neighbors(points, box, periodic, cutoff, full, "ijSdD")
        O.assert_same(got, oracle, RTOL_FP64, "no-alloc build against the CPU oracle")


def test_limits_are_reported():
    import torch

    points, box, periodic = W.diamond(3, seed=1)
    status, message, length, _ = _no_alloc(torch, None, points, box, periodic, 5.0, True, 10)
    assert status == 1 and "output arrays hold 10" in message
    expected = _existing_entry_point(torch, points, box, periodic, 5.0, True)
    assert length == len(expected["i"])  # the number of pairs needed is still reported

    from vesin_b200._c_api import NO_ALLOC_MAX_POINTS

    too_many = np.zeros((NO_ALLOC_MAX_POINTS + 1, 3))
    status, message, _, _ = _no_alloc(torch, None, too_many, np.eye(3) * 10, [True] * 3, 1.0, True, 10)
    assert status == 1 and f"at most {NO_ALLOC_MAX_POINTS} points" in message


def test_output_alignment():
    """Full lists use paired stores when the arrays allow it (pairs on 32 bytes,
    distances / vectors on 16, shifts on 8) and single stores otherwise: both
    give the same list. A `pairs` array off its 16-byte boundary is refused."""
    import torch

    points, box, periodic = W.diamond(6, seed=23)
    expected = _existing_entry_point(torch, points, box, periodic, 5.0, True)
    oracle = O.restated_neighbors(points, box, periodic, 5.0, True, "ijSdD")
    capacity = len(expected["i"]) + 64
    for offsets in [(16, 4, 8, 8), (0, 4, 0, 0), (16, 0, 0, 8)]:
        status, message, length, got = _no_alloc(torch, None, points, box, periodic, 5.0, True, capacity, offsets)
        assert status == 0, message
        assert length == len(expected["i"])
        O.assert_same(got, expected, RTOL_FP64, f"no-alloc build with output offsets {offsets}")
        O.assert_same(got, oracle, RTOL_FP64, f"no-alloc build with output offsets {offsets} against the CPU oracle")
    status, message, _, _ = _no_alloc(torch, None, points, box, periodic, 5.0, True, capacity, (8, 0, 0, 0))
    assert status == 1 and "aligned to 16 bytes" in message
