"""The Verlet-skin cache on the device (`skin > 0`, through the C ABI and the
calculator): candidates found at cutoff + skin are re-filtered on later calls
while no point has moved more than skin / 2. Whatever the cache does, every
call must return the exact list at the cutoff: (i, j, S) identical to the CPU
oracle's, d and D bit-identical. The reference has the same contract
(vesin/src/verlet_cuda.cpp:307-322; tests: python/vesin/tests/test_numpy.py:405-551,
vesin/tests/cuda.cpp:161-227)."""

import numpy as np
import pytest

from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _step(calculator, points, box, periodic, dtype=np.float64):
    import torch

    device = torch.device("cuda", 0)
    i, j, S, d, D = calculator.compute(
        torch.tensor(points.astype(dtype), device=device), torch.tensor(box.astype(dtype), device=device),
        torch.tensor(np.asarray(periodic, dtype=bool), device=device), "ijSdD", copy=False,
    )
    return {"i": i.cpu().numpy().astype(np.int64), "j": j.cpu().numpy().astype(np.int64), "S": S.cpu().numpy(), "d": d.cpu().numpy(), "D": D.cpu().numpy()}


def _same_as_oracle(got, points, box, periodic, cutoff, full, dtype=np.float64, label=""):
    used_points = points.astype(dtype).astype(np.float64)
    used_box = box.astype(dtype).astype(np.float64)
    expected = O.canonical(O.restated_neighbors(used_points, used_box, periodic, cutoff, full, "ijSdD"))
    got = O.canonical(got)
    assert len(got["i"]) == len(expected["i"]), label
    for key in "ijS":
        assert np.array_equal(got[key], expected[key]), f"{label}: {key}"
    assert np.array_equal(got["d"], expected["d"].astype(dtype)), f"{label}: d"
    assert np.array_equal(got["D"], expected["D"].astype(dtype)), f"{label}: D"


def _served_from_cache(calculator):
    """Stage times of the last call: a call served from cached candidates runs
    the displacement check and the filter ("emit") and bins nothing; the stages
    of a candidate build are added to the call that needed it."""
    times = calculator.stage_times()
    return times is not None and times["bin"] == 0.0 and times["emit"] > 0.0


@pytest.mark.parametrize("full", [True, False])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_trajectory(full, dtype):
    import vesin_b200

    points, box, periodic = W.liquid(20000, seed=41)
    rng = np.random.default_rng(7)
    calculator = vesin_b200.NeighborList(cutoff=6.0, full_list=full, skin=2.0)
    vesin_b200.set_profiling(True)
    try:
        cached_steps = 0
        for step in range(12):
            if step == 8:
                points = points.copy()
                points[123] += np.array([0.0, 1.2, 0.0])  # further than skin / 2: new candidates
            elif step > 0:
                points = points + rng.normal(0.0, 0.03, points.shape)
            got = _step(calculator, points, box, periodic, dtype)
            _same_as_oracle(got, points, box, periodic, 6.0, full, dtype, f"step {step}")
            served = _served_from_cache(calculator)
            if step in (0, 8):
                assert not served, f"step {step} has to build new candidates"
            cached_steps += int(served)
        assert cached_steps >= 8, "small moves are served from the cached candidates"
    finally:
        vesin_b200.set_profiling(False)


def test_box_changes_and_periodicity():
    """The box breathes (every corner moves less than the skin): the candidates
    stay, the threshold on the points shrinks. A change of periodicity, or a
    box that moved too far, brings new candidates."""
    import vesin_b200

    points, box, periodic = W.liquid(8000, seed=3)
    calculator = vesin_b200.NeighborList(cutoff=5.0, full_list=True, skin=1.5)
    vesin_b200.set_profiling(True)
    try:
        _same_as_oracle(_step(calculator, points, box, periodic), points, box, periodic, 5.0, True, label="first")
        scale = 1.0 + 1e-4
        for step in range(3):
            points, box = points * scale, box * scale
            got = _step(calculator, points, box, periodic)
            _same_as_oracle(got, points, box, periodic, 5.0, True, label=f"scaled {step}")
        assert _served_from_cache(calculator)
        open_z = np.array([True, True, False])
        _same_as_oracle(_step(calculator, points, box, open_z), points, box, open_z, 5.0, True, label="periodicity")
        assert not _served_from_cache(calculator)
        points, box = points * 1.05, box * 1.05  # corners move by more than the skin
        _same_as_oracle(_step(calculator, points, box, open_z), points, box, open_z, 5.0, True, label="large box change")
        assert not _served_from_cache(calculator)
    finally:
        vesin_b200.set_profiling(False)


def test_more_pairs_than_the_arrays_hold():
    """The points contract between two calls: the cached candidates give more
    pairs than the output arrays of the previous call hold."""
    import vesin_b200

    points, box, periodic = W.diamond(6, seed=2)
    calculator = vesin_b200.NeighborList(cutoff=3.0, full_list=True, skin=2.5)
    _same_as_oracle(_step(calculator, points, box, periodic), points, box, periodic, 3.0, True, label="first")
    squeezed, small_box = points * 0.97, box * 0.97
    _same_as_oracle(_step(calculator, squeezed, small_box, periodic), squeezed, small_box, periodic, 3.0, True, label="squeezed")


def test_points_far_outside_the_box():
    """Shifts beyond what a candidate record stores: the list is rebuilt on every
    call, the results are the same."""
    import vesin_b200

    points, box, periodic = W.diamond(3, seed=9)
    points = points + 700.0 * box[0] - 900.0 * box[2]
    points[::2] -= 1300.0 * box[1]
    calculator = vesin_b200.NeighborList(cutoff=4.0, full_list=False, skin=1.0)
    for step in range(3):
        moved = points + 0.01 * step
        _same_as_oracle(_step(calculator, moved, box, periodic), moved, box, periodic, 4.0, False, label=f"step {step}")


def test_dense_system_keeps_exact_lists():
    """A dense crystal with a large skin: filtering its many candidates may take
    longer than building the list, in which case the engine stops caching for
    this list. Whichever way it goes, every call returns the exact list."""
    import vesin_b200

    points, box, periodic = W.diamond(24)
    rng = np.random.default_rng(3)
    calculator = vesin_b200.NeighborList(cutoff=5.0, full_list=True, skin=2.0)
    for step in range(5):
        moved = points + rng.normal(0.0, 0.02, points.shape)
        _same_as_oracle(_step(calculator, moved, box, periodic), moved, box, periodic, 5.0, True, label=f"step {step}")


def test_large_system_through_the_timed_trial():
    """A system large enough for the engine to time its filter pass against
    plain builds (the calls after the first filter pass are served by plain
    builds, then by whichever was faster): every call returns the list a
    calculator without skin builds from the same points, compared on the device
    by the checksums of (i, j, S) and (i, j, S, bits of d)."""
    import torch

    import vesin_b200
    from vesin_b200._sharded import list_checksum

    device = torch.device("cuda", 0)
    points, box, periodic = W.liquid(1 << 18, seed=12)
    rng = np.random.default_rng(3)
    with_skin = vesin_b200.NeighborList(cutoff=6.0, full_list=False, skin=2.0)
    plain = vesin_b200.NeighborList(cutoff=6.0, full_list=False)
    box_d = torch.tensor(box, device=device)
    periodic_d = torch.tensor(np.asarray(periodic, dtype=bool), device=device)
    for step in range(8):
        if step == 6:
            points = points.copy()
            points[77] += np.array([1.3, 0.0, 0.0])  # further than skin / 2
        elif step > 0:
            points = points + rng.uniform(-0.05, 0.05, points.shape)
        points_d = torch.tensor(points, device=device)
        got = with_skin.compute(points_d, box_d, periodic_d, "ijSdD", copy=False)
        expected = plain.compute(points_d, box_d, periodic_d, "ijSdD", copy=False)
        assert len(got[0]) == len(expected[0]), f"step {step}"
        assert list_checksum(with_skin._neighbors) == list_checksum(plain._neighbors), f"step {step}"
