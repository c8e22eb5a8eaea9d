"""GPU parity of the batch entry point (vesin_b200_neighbors_batch, through
the C ABI): every system of a batch must get the list that the CPU oracle
gives for that system alone."""

import numpy as np
import pytest

from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _check_batch(points, offsets, boxes, periodic, cutoff, full, global_indices=False, calculator=None):
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    if calculator is None:
        calculator = vesin_b200.BatchNeighborList(cutoff=cutoff, full_list=full)
    (i, j, S, d, D), pair_offsets = calculator.compute(
        torch.tensor(points, device=device),
        offsets,
        None if boxes is None else torch.tensor(boxes, device=device),
        None if periodic is None else torch.tensor(periodic, device=device),
        "ijSdD",
        global_indices=global_indices,
    )
    i, j, S, d, D = (t.cpu().numpy() for t in (i, j, S, d, D))
    pair_offsets = pair_offsets.cpu().numpy()
    assert pair_offsets[0] == 0 and pair_offsets[-1] == len(i)
    for k in range(len(offsets) - 1):
        lo, hi = pair_offsets[k], pair_offsets[k + 1]
        shift = offsets[k] if global_indices else 0
        got = {"i": i[lo:hi] - shift, "j": j[lo:hi] - shift, "S": S[lo:hi], "d": d[lo:hi], "D": D[lo:hi]}
        system = points[offsets[k] : offsets[k + 1]]
        box = np.zeros((3, 3)) if boxes is None else boxes[k]
        pbc = [False] * 3 if periodic is None else periodic[k]
        expected = O.restated_neighbors(system, box, pbc, cutoff, full, "ijSdD")
        O.assert_same(got, expected, 1e-12, f"system {k}")
        expected = O.canonical(expected)
        got = O.canonical(got)
        assert np.array_equal(got["d"], expected["d"]) and np.array_equal(got["D"], expected["D"])


@pytest.mark.parametrize("full", [True, False])
def test_molecules(full):
    points, offsets = W.molecule_batch(n_systems=400, seed=4)
    _check_batch(points, offsets, None, None, 4.0, full)
    _check_batch(points, offsets, None, None, 4.0, full, global_indices=True)


@pytest.mark.parametrize("full", [True, False])
def test_periodic_systems_with_many_images(full, monkeypatch):
    monkeypatch.setenv("VESIN_CUDA_MAX_PAIRS_PER_POINT", "100000")
    rng = np.random.default_rng(12)
    systems, boxes, periodic = [], [], []
    for k in range(24):
        n_atoms = int(rng.integers(1, 40))
        p, b, _ = W.small_triclinic(n_atoms, seed=100 + k)
        flags = [bool(x) for x in rng.integers(0, 2, 3)] if k % 3 else [True, True, True]
        # some points far outside the box
        p = p + rng.integers(-3, 4, (n_atoms, 3)) @ b * (k % 2)
        systems.append(p)
        boxes.append(b)
        periodic.append(flags)
    offsets = np.concatenate([[0], np.cumsum([len(s) for s in systems])])
    _check_batch(np.concatenate(systems), offsets, np.array(boxes), np.array(periodic), 7.0, full)


def test_empty_systems_and_errors():
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    points, offsets = W.molecule_batch(n_systems=6, seed=9)
    # an empty system in the middle
    offsets = np.concatenate([offsets[:3], offsets[2:]])
    _check_batch(points, offsets, None, None, 4.0, True)

    calculator = vesin_b200.BatchNeighborList(cutoff=4.0, full_list=True)
    big = torch.zeros((3000, 3), dtype=torch.float64, device=device)
    with pytest.raises(RuntimeError, match="at most 2048 points per system"):
        calculator.compute(big, [0, 3000])
    boxes = torch.zeros((1, 3, 3), dtype=torch.float64, device=device)
    periodic = torch.ones((1, 3), dtype=torch.bool, device=device)
    with pytest.raises(RuntimeError, match="the box matrix is not invertible \\(system 0"):
        calculator.compute(big[:10], [0, 10], boxes, periodic)
    bad = torch.zeros((10, 3), dtype=torch.float64, device=device)
    bad[4, 0] = float("inf")
    with pytest.raises(RuntimeError, match="point 4 of the batch has a non-finite coordinate"):
        calculator.compute(bad, [0, 10])


def test_molecules_float32_and_mixed_sizes():
    """The fp32 batch entry point (float points in, float d and D out, decisions
    in fp64 on the upcast values), on a batch that mixes molecules small enough
    for the warp-per-system kernel with larger ones."""
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    rng = np.random.default_rng(77)
    sizes = [1, 2, 0, 96, 97, 130, 33, 64, 5]
    systems = [rng.uniform(-4.0, 4.0, (n, 3)).astype(np.float32) for n in sizes]
    points = np.concatenate(systems)
    offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    for full in (True, False):
        calculator = vesin_b200.BatchNeighborList(cutoff=3.0, full_list=full)
        (i, j, S, d, D), pair_offsets = calculator.compute(torch.tensor(points, device=device), offsets, None, None, "ijSdD")
        assert d.dtype == torch.float32 and D.dtype == torch.float32
        i, j, S, d, D = (t.cpu().numpy() for t in (i, j, S, d, D))
        pair_offsets = pair_offsets.cpu().numpy()
        for k, system in enumerate(systems):
            lo, hi = pair_offsets[k], pair_offsets[k + 1]
            expected = O.canonical(O.restated_neighbors(system.astype(np.float64), np.zeros((3, 3)), [False] * 3, 3.0, full, "ijSdD"))
            got = O.canonical({"i": i[lo:hi], "j": j[lo:hi], "S": S[lo:hi], "d": d[lo:hi], "D": D[lo:hi]})
            assert np.array_equal(got["i"], expected["i"]) and np.array_equal(got["j"], expected["j"]), f"system {k}"
            assert np.array_equal(got["S"], expected["S"])
            assert np.array_equal(got["d"], expected["d"].astype(np.float32)), "d is the fp64 value rounded once"
            assert np.array_equal(got["D"], expected["D"].astype(np.float32))


def test_molecules_on_the_edge_of_the_cutoff():
    """Pairs within rounding distance of the cutoff: the fp32 screen must hand
    them to the exact predicate."""
    rng = np.random.default_rng(5)
    systems = []
    for _ in range(50):
        n = int(rng.integers(2, 40))
        base = rng.uniform(-5.0, 5.0, 3) + 1000.0 * rng.standard_normal(3)
        directions = rng.standard_normal((n, 3))
        directions /= np.linalg.norm(directions, axis=1)[:, None]
        radii = 2.0 * (1.0 + rng.integers(-3, 4, n) * 2.0 ** -52)
        systems.append(base + directions * radii[:, None] * 0.5 + np.where(rng.random((n, 1)) < 0.5, 0.0, 1e-16))
    points = np.concatenate(systems)
    offsets = np.concatenate([[0], np.cumsum([len(s) for s in systems])]).astype(np.int64)
    _check_batch(points, offsets, None, None, 2.0, True)


def test_cutoff_far_beyond_the_box_of_a_system_is_refused():
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    points = np.random.default_rng(1).random((6, 3))
    offsets = np.array([0, 3, 6])
    boxes = np.stack([np.eye(3) * 5.0, np.eye(3) * 1e-3])
    periodic = np.ones((2, 3), dtype=bool)
    calculator = vesin_b200.BatchNeighborList(cutoff=2.0, full_list=True)
    with pytest.raises(RuntimeError, match="too large for the box of system 1"):
        calculator.compute(torch.tensor(points, device=device), offsets, torch.tensor(boxes, device=device), torch.tensor(periodic, device=device), "ij")


def test_one_calculator_over_changing_batches():
    """The same list serves batches of the same layout (the writing pass runs
    before the host knows the total; the offsets stay on the device), then a
    batch of the same size with other offsets, a batch with more pairs than the
    arrays hold (molecules squeezed together), and the first batch again."""
    import vesin_b200

    calculator = vesin_b200.BatchNeighborList(cutoff=4.0, full_list=True)
    points, offsets = W.molecule_batch(n_systems=300, seed=21)
    rng = np.random.default_rng(5)
    _check_batch(points, offsets, None, None, 4.0, True, calculator=calculator)
    moved = points + rng.normal(0.0, 0.05, points.shape)
    _check_batch(moved, offsets, None, None, 4.0, True, calculator=calculator)
    other_points, other_offsets = W.molecule_batch(n_systems=300, seed=22)
    assert len(other_offsets) == len(offsets) and not np.array_equal(other_offsets, offsets)
    _check_batch(other_points, other_offsets, None, None, 4.0, True, calculator=calculator)
    # every molecule shrunk towards its first atom: many more pairs within the cutoff
    squeezed = points.copy()
    for k in range(len(offsets) - 1):
        lo, hi = offsets[k], offsets[k + 1]
        squeezed[lo:hi] = points[lo] + 0.6 * (points[lo:hi] - points[lo])
    _check_batch(squeezed, offsets, None, None, 4.0, True, calculator=calculator)
    _check_batch(points, offsets, None, None, 4.0, True, calculator=calculator)
