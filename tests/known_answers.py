"""
Known-answer vectors held by the reference's own tests for the neighbor-list
path, written out as data. Each entry: inputs, options and the expected
canonical content. Sources (paths relative to the reference project root):

* vesin/tests/neighbors.cpp:86-135   non-periodic, 5 points, half list
* vesin/tests/neighbors.cpp:137-182  one-atom FCC cell, 6 self-image pairs
* vesin/tests/neighbors.cpp:184-223  54-wide box, atoms outside the box
* vesin/tests/neighbors.cpp:225-262  cutoff larger than the box
* vesin/tests/neighbors.cpp:264-328  slanted box: 90 pairs, shifts (-2, 0..2, 0)
* vesin/tests/memory.cpp:5-87        list lengths 9 / 67 / 134 / 27
* vesin/tests/cuda.cpp:19-126        triclinic FCC-like box, 3 points, 5 pairs
* fortran/tests/tests.f90:20-122     2 points, 3.2 box, cutoff 3.3, 10 pairs
* python/vesin/tests/test_numpy.py:341-370  three points, all pairs, any origin
"""

import math

import numpy as np

T3 = [True, True, True]
F3 = [False, False, False]

NON_PERIODIC = dict(
    points=[
        [0.134, 1.282, 1.701],
        [-0.273, 1.026, -1.471],
        [1.922, -0.124, 1.900],
        [1.400, -0.464, 0.480],
        [0.149, 1.865, 0.635],
    ],
    box=np.zeros((3, 3)),
    periodic=F3,
    cutoff=3.42,
    full=False,
    pairs=[[0, 1], [0, 2], [0, 3], [0, 4], [1, 3], [1, 4], [2, 3], [2, 4], [3, 4]],
    distances=[
        3.2082345612501593,
        2.283282943482914,
        2.4783286706972505,
        1.215100818862369,
        2.9707625283755013,
        2.3059143522689647,
        1.550639867925496,
        2.9495550511899244,
        2.6482573515427084,
    ],
)

FCC = dict(
    points=[[0.0, 0.0, 0.0]],
    box=[[0.0, 1.5, 1.5], [1.5, 0.0, 1.5], [1.5, 1.5, 0.0]],
    periodic=T3,
    cutoff=3.0,
    full=False,
    pairs=[[0, 0]] * 6,
    shifts=[[-1, 0, 1], [-1, 1, 0], [0, -1, 1], [0, 0, 1], [0, 1, 0], [1, 0, 0]],
    distances=[2.1213203435596424] * 6,
    vectors=[
        [1.5, 0.0, -1.5],
        [1.5, -1.5, 0.0],
        [0.0, 1.5, -1.5],
        [1.5, 1.5, 0.0],
        [1.5, 0.0, 1.5],
        [0.0, 1.5, 1.5],
    ],
)

LARGE_BOX = dict(
    points=[
        [0.0, 0.0, 0.0],
        [0.0, 2.0, 0.0],
        [0.0, 0.0, 2.0],
        [-6.0, 0.0, 0.0],
        [-6.0, -2.0, 0.0],
        [-6.0, 0.0, -2.0],
    ],
    box=np.eye(3) * 54.0,
    periodic=T3,
    cutoff=2.1,
    full=False,
    pairs=[[0, 1], [0, 2], [3, 4], [3, 5]],
    shifts=[[0, 0, 0]] * 4,
    distances=[2.0] * 4,
)

CUTOFF_OVER_BOX = dict(
    points=[[0.0, 0.0, 0.0]],
    box=np.eye(3) * 0.5,
    periodic=T3,
    cutoff=0.6,
    full=False,
    pairs=[[0, 0]] * 3,
    shifts=[[0, 0, 1], [0, 1, 0], [1, 0, 0]],
    distances=[0.5] * 3,
    vectors=[[0.0, 0.0, 0.5], [0.0, 0.5, 0.0], [0.5, 0.0, 0.0]],
)

SLANTED = dict(
    points=[
        [1.42, 0.0, 0.0],
        [2.84, 0.0, 0.0],
        [3.55, -1.22975607, 0.0],
        [4.97, -1.22975607, 0.0],
    ],
    box=[[4.26, -2.45951215, 0.0], [2.13, 1.22975607, 0.0], [0.0, 0.0, 50.0]],
    periodic=T3,
    cutoff=6.4,
    full=False,
    n_pairs=90,
    must_contain=[(0, 3, (-2, 0, 0)), (0, 3, (-2, 1, 0)), (0, 3, (-2, 2, 0))],
)

# vesin/tests/memory.cpp: (cutoff, full) -> length, same one-atom FCC cell
REUSE_LENGTHS = [((3.4, False), 9), ((6.0, False), 67), ((6.0, True), 134), ((4.5, False), 27)]

CUDA_TRICLINIC = dict(
    points=[[0.0, 0.0, 0.0], [1.0, 1.0, 1.0], [2.0, 2.0, 2.0]],
    box=[[0.0, 3.0, 3.0], [3.0, 0.0, 3.0], [3.0, 3.0, 0.0]],
    periodic=T3,
    cutoff=3.0,
    full=False,
    pairs=[[0, 1], [0, 2], [0, 2], [0, 2], [1, 2]],
    shifts=[[0, 0, 0], [-1, 0, 0], [0, -1, 0], [0, 0, -1], [0, 0, 0]],
    distances=[math.sqrt(3.0), math.sqrt(6.0), math.sqrt(6.0), math.sqrt(6.0), math.sqrt(3.0)],
    vectors=[[1.0, 1.0, 1.0], [2.0, -1.0, -1.0], [-1.0, 2.0, -1.0], [-1.0, -1.0, 2.0], [1.0, 1.0, 1.0]],
    exact=True,  # the reference test compares d and D with ==
)

_f = np.float32
FORTRAN = dict(
    # the Fortran test holds single-precision data, promoted to double
    points=[[0.0, 0.0, 0.0], [0.0, float(_f(1.3)), float(_f(1.3))]],
    box=np.eye(3) * float(_f(3.2)),
    periodic=T3,
    cutoff=float(_f(3.3)),
    full=False,
    pairs=[[0, 0], [0, 0], [0, 0], [0, 1], [0, 1], [0, 1], [0, 1], [1, 1], [1, 1], [1, 1]],
    shifts=[
        [0, 0, 1],
        [0, 1, 0],
        [1, 0, 0],
        [0, -1, -1],
        [0, -1, 0],
        [0, 0, -1],
        [0, 0, 0],
        [0, 0, 1],
        [0, 1, 0],
        [1, 0, 0],
    ],
    distances=[3.2, 3.2, 3.2, 2.6870059, 2.3021729, 2.3021729, 1.8384775, 3.2, 3.2, 3.2],
    vectors=[
        [0.0, 0.0, 3.2],
        [0.0, 3.2, 0.0],
        [3.2, 0.0, 0.0],
        [0.0, -1.9, -1.9],
        [0.0, -1.9, 1.3],
        [0.0, 1.3, -1.9],
        [0.0, 1.3, 1.3],
        [0.0, 0.0, 3.2],
        [0.0, 3.2, 0.0],
        [3.2, 0.0, 0.0],
    ],
    atol=1e-6,
)

THREE_POINTS = dict(
    points=[
        [3.87166034, 1.63896135, 22.14371739],
        [3.19075223, 1.6182371, 22.87858863],
        [5.01141342, 1.73904134, 20.79729257],
    ],
    box=np.zeros((3, 3)),
    periodic=F3,
    cutoff=8.0,
    full=True,
    pairs=[[0, 1], [0, 2], [1, 0], [1, 2], [2, 0], [2, 1]],
)

EXACT_CASES = {
    "non_periodic": NON_PERIODIC,
    "fcc": FCC,
    "large_box": LARGE_BOX,
    "cutoff_over_box": CUTOFF_OVER_BOX,
    "cuda_triclinic": CUDA_TRICLINIC,
    "fortran": FORTRAN,
    "three_points": THREE_POINTS,
}


def ulp_close(a, b, ulps=4):
    """The reference's WithinULP(b, 4) check (vesin/tests/neighbors.cpp:11)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.all(np.abs(a - b) <= ulps * np.spacing(np.maximum(np.abs(a), np.abs(b))))


def check_known_answer(case, compute):
    """`compute(points, box, periodic, cutoff, full, quantities)` must return a
    dict with canonical-sortable i, j, S, d, D numpy arrays."""
    from oracle.oracle import canonical

    got = canonical(compute(case["points"], case["box"], case["periodic"], case["cutoff"], case["full"], "ijSdD"))
    pairs = np.stack([got["i"], got["j"]], axis=1)
    if "n_pairs" in case:
        assert len(pairs) == case["n_pairs"]
        have = {(int(i), int(j), tuple(int(x) for x in s)) for i, j, s in zip(got["i"], got["j"], got["S"])}
        for item in case["must_contain"]:
            assert item in have
        return
    assert np.array_equal(pairs, np.array(case["pairs"], dtype=np.int64).reshape(-1, 2))
    if "shifts" in case:
        assert np.array_equal(got["S"], np.array(case["shifts"], dtype=np.int32))
    atol = case.get("atol")
    for key, name in (("d", "distances"), ("D", "vectors")):
        if name not in case:
            continue
        expected = np.array(case[name], dtype=np.float64)
        if "shifts" not in case and key == "D":
            continue
        if case.get("exact"):
            assert np.array_equal(got[key], expected)
        elif atol is not None:
            assert np.all(np.abs(got[key] - expected) <= atol)
        else:
            assert ulp_close(got[key], expected)
