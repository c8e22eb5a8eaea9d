"""GPU parity tests: the CUDA engine, called through the C ABI, against the
reference's known answers, the golden fixtures made by the unmodified
reference CPU path, and the CPU restatement on the same seeded inputs.
Integers (i, j, S) must match bit for bit after canonical sorting; d and D
within 1e-12 relative (fp64)."""

import hashlib

import numpy as np
import pytest

import known_answers as KA
from gpu_utils import gpu_compute
from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu

RTOL_FP64 = 1e-12


def _gpu(points, box, periodic, cutoff, full, quantities):
    return gpu_compute(points, box, periodic, cutoff, full, quantities)


@pytest.mark.parametrize("name", sorted(KA.EXACT_CASES))
def test_known_answers(name):
    KA.check_known_answer(KA.EXACT_CASES[name], _gpu)


def test_slanted_box():
    KA.check_known_answer(KA.SLANTED, _gpu)


def test_golden_fixtures(golden):
    """Every fixture produced by the reference CPU library."""
    for name in [str(n) for n in golden["names"]]:
        _, cutoff, full = name.split("|")
        points, box, periodic = golden[name + "/points"], golden[name + "/box"], golden[name + "/periodic"]
        res = O.canonical(_gpu(points, box, periodic, float(cutoff), bool(int(full)), "ijSdD"))
        assert len(res["i"]) == int(golden[name + "/n_pairs"]), name
        table = np.concatenate([res["i"][:, None], res["j"][:, None], res["S"].astype(np.int64)], axis=1)
        sha = hashlib.sha256(np.ascontiguousarray(table).tobytes()).hexdigest()
        assert sha == str(golden[name + "/sha256"]), name
        scale = max(float(golden[name + "/sum_d"]), 1.0)
        assert abs(res["d"].sum() - float(golden[name + "/sum_d"])) <= 1e-12 * scale, name
        if name + "/d" in golden.files and len(res["i"]):
            assert np.max(np.abs(res["d"] - golden[name + "/d"])) <= RTOL_FP64 * float(cutoff), name
            assert np.max(np.abs(res["D"] - golden[name + "/D"])) <= RTOL_FP64 * float(cutoff), name


@pytest.mark.parametrize("sorted", [False, True])
@pytest.mark.parametrize("full", [True, False])
@pytest.mark.parametrize(
    "system,cutoff",
    [("diamond5", 5.0), ("triclinic64", 9.0), ("diamond12", 5.0), ("diamond3_big_cutoff", 12.0), ("liquid", 6.0), ("dense_cell", 3.0)],
)
def test_against_restatement(system, cutoff, full, sorted, monkeypatch):
    monkeypatch.setenv("VESIN_CUDA_MAX_PAIRS_PER_POINT", "100000")
    points, box, periodic = {
        "diamond5": lambda: W.diamond(5),
        "triclinic64": lambda: W.small_triclinic(),
        "diamond12": lambda: W.diamond(12, seed=11),
        "diamond3_big_cutoff": lambda: W.diamond(3, seed=5),
        # few points per cell: pencils of several cells
        "liquid": lambda: W.liquid(20000, seed=8),
        # 700 points in one small cell: many tiles of home points per unit
        "dense_cell": lambda: (np.random.default_rng(2).random((700, 3)) * 4.0, np.eye(3) * 4.0, np.array([True, True, False])),
    }[system]()
    got = gpu_compute(points, box, periodic, cutoff, full, "ijSdD", sorted=sorted)
    if sorted:
        assert np.all(np.diff(got["i"]) >= 0), "sorted lists are ordered by the first index"
    expected = O.restated_neighbors(points, box, periodic, cutoff, full, "ijSdD")
    O.assert_same(got, expected, RTOL_FP64, f"{system} full={full}")
    # the arithmetic is the reference's, operation for operation
    got, expected = O.canonical(got), O.canonical(expected)
    assert np.array_equal(got["d"], expected["d"])
    assert np.array_equal(got["D"], expected["D"])


@pytest.mark.parametrize("bits", range(8))
def test_mixed_periodicity(bits, monkeypatch):
    # dense unit box: more pairs per point than the default limit of 128
    monkeypatch.setenv("VESIN_CUDA_MAX_PAIRS_PER_POINT", "100000")
    periodic = [bool((bits >> 2) & 1), bool((bits >> 1) & 1), bool(bits & 1)]
    points, box, periodic = W.skewed_random(periodic, seed=40 + bits, n=300)
    for cutoff in (0.2, 0.35, 0.8):
        got = _gpu(points, box, periodic, cutoff, True, "ijSdD")
        expected = O.restated_neighbors(points, box, periodic, cutoff, True, "ijSdD")
        O.assert_same(got, expected, RTOL_FP64, f"periodic={periodic} cutoff={cutoff}")


def test_quantities_subsets_and_reuse():
    """Re-use of one list across option changes (vesin/tests/memory.cpp)."""
    import vesin_b200

    points, box, periodic = KA.FCC["points"], KA.FCC["box"], KA.FCC["periodic"]
    for (cutoff, full), length in KA.REUSE_LENGTHS:
        res = _gpu(points, box, periodic, cutoff, full, "ij")
        assert len(res["i"]) == length
    calculator = vesin_b200.NeighborList(cutoff=3.4, full_list=False)
    res = gpu_compute(points, box, periodic, 3.4, False, "ijd", calculator=calculator)
    assert len(res["i"]) == 9
    lst = calculator._neighbors
    assert lst.pairs and lst.distances and not lst.shifts and not lst.vectors
    calculator.cutoff = 6.0
    calculator.full_list = True
    res = gpu_compute(points, box, periodic, 6.0, True, "ijd", calculator=calculator)
    assert len(res["i"]) == 134
    assert lst.pairs and lst.distances and not lst.shifts and not lst.vectors
    calculator.cutoff = 4.5
    calculator.full_list = False
    res = gpu_compute(points, box, periodic, 4.5, False, "ijS", calculator=calculator)
    assert len(res["i"]) == 27
    assert lst.pairs and lst.shifts and not lst.distances and not lst.vectors


def test_sorted_rows_and_empty():
    points, box, periodic = W.diamond(4, seed=9)
    res = gpu_compute(points, box, periodic, 4.0, True, "ij", sorted=True)
    assert np.all(np.diff(res["i"]) >= 0), "sorted lists are ordered by the first index"
    res = _gpu(points, box, periodic, 0.3, True, "ijSdD")
    assert len(res["i"]) == 0


def test_errors():
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    points = torch.zeros((2, 3), dtype=torch.float64, device=device)
    box = torch.eye(3, dtype=torch.float64, device=device)
    with pytest.raises(RuntimeError, match="cutoff must be a finite, positive number"):
        vesin_b200.NeighborList(cutoff=-1.0, full_list=True).compute(points, box, True, "ij")
    with pytest.raises(RuntimeError, match="cutoff is too small"):
        vesin_b200.NeighborList(cutoff=1e-7, full_list=True).compute(points, box, True, "ij")
    with pytest.raises(RuntimeError, match="the box matrix is not invertible"):
        vesin_b200.NeighborList(cutoff=1.0, full_list=True).compute(points, torch.zeros_like(box), True, "ij")
    bad = points.clone()
    bad[1, 2] = float("inf")
    with pytest.raises(RuntimeError, match="point 1 has non-finite coordinate along axis 2: inf"):
        vesin_b200.NeighborList(cutoff=1.0, full_list=True).compute(bad, box, True, "ij")
    with pytest.raises(RuntimeError, match="Invalid cutoff: too large for box dimensions"):
        vesin_b200.NeighborList(cutoff=0.6, full_list=True, algorithm="brute_force").compute(points, box, True, "ij")
    # a zero box is fine when nothing is periodic
    res = vesin_b200.NeighborList(cutoff=1.0, full_list=True).compute(points, torch.zeros_like(box), False, "ij")
    assert len(res[0]) == 2


def test_reused_list_follows_changing_inputs():
    """A re-used list starts every build from the plan of the previous one; a
    kernel checks box, periodicity and extent, and the build is redone when
    they changed. Every step must give the oracle's list."""
    import torch

    import vesin_b200

    rng = np.random.default_rng(77)
    points, box, periodic = W.diamond(4, seed=31)
    calculator = vesin_b200.NeighborList(cutoff=4.0, full_list=True)
    steps = [
        (points, box, periodic),                                    # first build: plans from a read-back
        (points + rng.normal(0, 0.02, points.shape), box, periodic),  # same box: speculative plan accepted
        (points, box * 1.07, periodic),                             # box changed
        (points, box * 1.07, np.array([True, False, True])),        # periodicity changed
        (points * 1.6, box * 1.07, np.array([True, False, True])),  # points left the non-periodic window
        (points * 1.6, box * 1.07, np.array([True, False, True])),  # accepted again
        (points @ W.random_rotation(5).T, box @ W.random_rotation(5).T, periodic),
    ]
    for step, (p, b, per) in enumerate(steps):
        for _ in range(2):
            got = gpu_compute(p, b, per, 4.0, True, "ijSdD", calculator=calculator)
            expected = O.restated_neighbors(p, b, per, 4.0, True, "ijSdD")
            O.assert_same(got, expected, RTOL_FP64, f"step {step}")

    # errors are still raised when the plan is speculative
    device = torch.device("cuda", 0)
    bad = torch.tensor(points, device=device)
    bad[7, 1] = float("nan")
    with pytest.raises(RuntimeError, match="point 7 has non-finite coordinate along axis 1: nan"):
        calculator.compute(bad, torch.tensor(box * 1.07, device=device), torch.tensor(periodic, device=device), "ij")
    with pytest.raises(RuntimeError, match="the box matrix is not invertible"):
        calculator.compute(torch.tensor(points, device=device), torch.zeros((3, 3), dtype=torch.float64, device=device), True, "ij")
    got = gpu_compute(points, box, periodic, 4.0, True, "ijSdD", calculator=calculator)
    O.assert_same(got, O.restated_neighbors(points, box, periodic, 4.0, True, "ijSdD"), RTOL_FP64, "after errors")

    # the sorted path speculates too
    calculator = vesin_b200.NeighborList(cutoff=4.0, full_list=False, sorted=True)
    for p, b, per in steps[:4]:
        got = gpu_compute(p, b, per, 4.0, False, "ijSdD", calculator=calculator)
        O.assert_same(got, O.restated_neighbors(p, b, per, 4.0, False, "ijSdD"), RTOL_FP64, "sorted")


@pytest.mark.parametrize("full", [True, False])
def test_skin_gives_the_list_at_the_cutoff(full):
    """`skin > 0`: the reference re-filters cached candidates while the atoms
    have moved less than skin / 2 (vesin/src/verlet.cpp:82-191; tests:
    python/vesin/tests/test_numpy.py:405-551), this engine rebuilds; both give
    the exact list at `cutoff` on every step of a trajectory with small moves, a
    jump, a box change and a change of the number of points."""
    import vesin_b200

    rng = np.random.default_rng(2024)
    points, box, periodic = W.diamond(4, seed=41)
    calculator = vesin_b200.NeighborList(cutoff=4.0, full_list=full, skin=1.0)
    reference = O.ReferenceCPU() if O.reference_available() else None
    trajectory = [(points, box)]
    for _ in range(4):  # small moves: the reference keeps its candidates
        trajectory.append((trajectory[-1][0] + rng.normal(0, 0.03, points.shape), box))
    jumped = trajectory[-1][0].copy()
    jumped[5] += 0.9  # more than skin / 2: the reference rebuilds
    trajectory.append((jumped, box))
    trajectory.append((jumped, box * 1.01))  # the box breathes
    trajectory.append((jumped[:-3], box * 1.01))  # three points fewer
    for step, (p, b) in enumerate(trajectory):
        got = gpu_compute(p, b, periodic, 4.0, full, "ijSdD", calculator=calculator)
        if reference is not None:
            expected = reference.compute(p, b, periodic, 4.0, full, "ijSdD", n_threads=1, skin=1.0)
        else:
            expected = O.restated_neighbors(p, b, periodic, 4.0, full, "ijSdD")
        O.assert_same(got, expected, RTOL_FP64, f"skin, step {step}")


@pytest.mark.parametrize("sorted", [False, True])
@pytest.mark.parametrize("full", [True, False])
def test_float32_entry_point(full, sorted):
    """float32 in, float32 out through vesin_b200_neighbors_f32: pairs and shifts
    are the oracle's on the exactly upcast inputs; d and D are its fp64 values
    rounded once (well inside the 1e-5 relative tolerance for fp32)."""
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    for (points, box, periodic), cutoff in ((W.diamond(6, seed=2), 5.0), (W.small_triclinic(40, seed=8), 6.5), (W.cluster(), 4.0)):
        p32 = points.astype(np.float32)
        b32 = box.astype(np.float32)
        calculator = vesin_b200.NeighborList(cutoff=cutoff, full_list=full, sorted=sorted)
        i, j, S, d, D = calculator.compute(
            torch.tensor(p32, device=device), torch.tensor(b32, device=device), torch.tensor(periodic, device=device), "ijSdD"
        )
        assert d.dtype == torch.float32 and D.dtype == torch.float32
        got = {"i": i.cpu().numpy().astype(np.int64), "j": j.cpu().numpy().astype(np.int64), "S": S.cpu().numpy(),
               "d": d.cpu().numpy(), "D": D.cpu().numpy()}
        expected = O.restated_neighbors(p32.astype(np.float64), b32.astype(np.float64), periodic, cutoff, full, "ijSdD")
        O.assert_same(got, expected, 1e-5, "float32")
        got, expected = O.canonical(got), O.canonical(expected)
        assert np.array_equal(got["d"], expected["d"].astype(np.float32))
        assert np.array_equal(got["D"], expected["D"].astype(np.float32))
    # numpy float32 in -> numpy float32 out
    i, j, d = vesin_b200.NeighborList(cutoff=5.0, full_list=True).compute(p32, b32, periodic, "ijd")
    assert d.dtype == np.float32
