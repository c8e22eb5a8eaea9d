"""CPU tests that pin the checker itself: the plain-C restatement against the
reference's known answers and against fixtures produced by the unmodified
reference CPU path (tests/golden/make_golden.py)."""

import hashlib

import numpy as np
import pytest

import known_answers as KA
from oracle import oracle as O
from vesin_b200 import workloads as W


def _restated(points, box, periodic, cutoff, full, quantities):
    return O.restated_neighbors(points, box, periodic, cutoff, full, quantities)


@pytest.mark.parametrize("name", sorted(KA.EXACT_CASES))
def test_known_answers(name):
    KA.check_known_answer(KA.EXACT_CASES[name], _restated)


def test_slanted_box():
    KA.check_known_answer(KA.SLANTED, _restated)


def test_reuse_lengths():
    for (cutoff, full), length in KA.REUSE_LENGTHS:
        res = _restated(KA.FCC["points"], KA.FCC["box"], KA.FCC["periodic"], cutoff, full, "ij")
        assert len(res["i"]) == length


def test_golden_fixtures(golden):
    names = [str(n) for n in golden["names"]]
    assert len(names) > 250
    for name in names:
        _, cutoff, full = name.split("|")
        res = O.canonical(
            _restated(golden[name + "/points"], golden[name + "/box"], golden[name + "/periodic"], float(cutoff), bool(int(full)), "ijSdD")
        )
        assert len(res["i"]) == int(golden[name + "/n_pairs"]), name
        table = np.concatenate([res["i"][:, None], res["j"][:, None], res["S"].astype(np.int64)], axis=1)
        sha = hashlib.sha256(np.ascontiguousarray(table).tobytes()).hexdigest()
        assert sha == str(golden[name + "/sha256"]), name
        assert res["d"].sum() == pytest.approx(float(golden[name + "/sum_d"]), rel=1e-12, abs=1e-12), name
        if name + "/d" in golden.files:
            assert np.array_equal(res["d"], golden[name + "/d"]), name
            assert np.array_equal(res["D"], golden[name + "/D"]), name


def test_errors():
    points = np.zeros((2, 3))
    with pytest.raises(RuntimeError, match="the box matrix is not invertible"):
        _restated(points, np.zeros((3, 3)), [True, True, True], 1.0, True, "ij")
    points[1, 2] = np.inf
    with pytest.raises(RuntimeError, match="point 1 has non-finite coordinate along axis 2: inf"):
        _restated(points, np.eye(3), [True, True, True], 1.0, True, "ij")


@pytest.mark.skipif(not O.reference_available(), reason="reference CPU library not built")
@pytest.mark.parametrize("full", [True, False])
def test_restatement_matches_reference_library(full):
    """Same values AND same (single-thread) order as the reference."""
    for system, cutoff in ((W.diamond(5), 5.0), (W.small_triclinic(), 9.0), (W.diamond(3, seed=2), 3.0)):
        a = _restated(*system, cutoff, full, "ijSdD")
        b = O.reference_neighbors(*system, cutoff, full, "ijSdD", n_threads=1)
        for key in a:
            assert np.array_equal(a[key], b[key]), key


def test_config_pair_counts():
    """Pair counts of the two CPU-sized benchmark configurations."""
    assert len(_restated(*W.diamond(5), 5.0, True, "ij")["i"]) == 89072
    assert len(_restated(*W.diamond(5), 5.0, False, "ij")["i"]) == 44536
    assert len(_restated(*W.small_triclinic(), 9.0, True, "ij")["i"]) == 45676


def test_reference_with_skin_gives_the_plain_list():
    """The reference's Verlet cache (vesin/src/verlet.cpp:82-191) is an
    optimisation: with `skin > 0` every call still returns the exact list at
    `cutoff`. Pinned here because the engine serves `skin > 0` by rebuilding."""
    if not O.reference_available():
        pytest.skip("reference CPU library not built")
    from vesin_b200 import workloads as W

    rng = np.random.default_rng(99)
    points, box, periodic = W.diamond(3, seed=2)
    reference = O.ReferenceCPU()
    for step in range(6):
        cached = reference.compute(points, box, periodic, 4.0, step % 2 == 0, "ijSdD", n_threads=1, skin=1.5)
        plain = O.restated_neighbors(points, box, periodic, 4.0, step % 2 == 0, "ijSdD")
        O.assert_same(cached, plain, 1e-12, f"skin, step {step}")
        points = points + rng.normal(0, 0.05 if step != 3 else 0.6, points.shape)
