"""Randomised differential test: seeded random systems (triclinic boxes, any
mix of periodic directions, cutoffs from a fraction of the box to several box
lengths, 1 to 1500 points, points inside and outside the box) through the C
ABI on the GPU against the CPU restatement. (i, j, S) identical after
canonical sorting, d and D bit-identical. The small boxes with large cutoffs
reach the units whose candidate batches several CTAs share; the large sparse
ones reach pencils of several cells."""

import numpy as np
import pytest

from gpu_utils import gpu_compute
from oracle import oracle as O

pytestmark = pytest.mark.gpu

N_CASES = 48


def _random_case(seed):
    rng = np.random.default_rng(1000 + seed)
    n = int(rng.choice([1, 2, 3, 7, 33, 64, 200, 700, 1500]))
    lengths = rng.uniform(2.0, 14.0, 3)
    box = np.diag(lengths)
    # a triclinic box two times out of three: tilt the cell vectors, keep the box well conditioned
    if seed % 3 != 0:
        box[1, 0] = rng.uniform(-0.4, 0.4) * lengths[0]
        box[2, 0] = rng.uniform(-0.4, 0.4) * lengths[0]
        box[2, 1] = rng.uniform(-0.4, 0.4) * lengths[1]
        # and rotate it, so that no direction is aligned with an axis
        q, _ = np.linalg.qr(rng.normal(size=(3, 3)))
        box = box @ q
    periodic = rng.random(3) < 0.6
    fractional = rng.random((n, 3))
    if seed % 4 == 1:
        fractional = fractional * 3.0 - 1.0  # points up to a box length outside
    points = fractional @ box
    # expected pairs per point stay below a few hundred: cutoff from the density
    volume = abs(np.linalg.det(box))
    density = n / volume
    c_max = (200.0 / (density * 4.19)) ** (1.0 / 3.0)
    cutoff = float(min(rng.uniform(0.4, 2.5) * lengths.min(), c_max, 3.0 * lengths.max()))
    cutoff = max(cutoff, 0.3)
    return points, box, periodic, cutoff


@pytest.mark.parametrize("seed", range(N_CASES))
def test_random_system(seed, monkeypatch):
    monkeypatch.setenv("VESIN_CUDA_MAX_PAIRS_PER_POINT", "100000")
    points, box, periodic, cutoff = _random_case(seed)
    full = seed % 2 == 0
    sorted_list = seed % 5 == 0
    expected = O.restated_neighbors(points, box, periodic, cutoff, full, "ijSdD")
    got = gpu_compute(points, box, periodic, cutoff, full, "ijSdD", sorted=sorted_list)
    label = f"seed {seed}: n={len(points)} cutoff={cutoff:.3f} periodic={periodic.tolist()} full={full} sorted={sorted_list}"
    O.assert_same(got, expected, 1e-12, label)
    got, expected = O.canonical(got), O.canonical(expected)
    assert np.array_equal(got["d"], expected["d"]), label
    assert np.array_equal(got["D"], expected["D"]), label
