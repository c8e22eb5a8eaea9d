"""The canonical list on the device (vesin_b200_neighbors_canonical, through the
C ABI): rows in index order, every row sorted by (second index, shift). The
GPU output is compared ELEMENT BY ELEMENT, with no sorting on the host side of
the GPU result, against the CPU oracle's list in canonical order (the
comparison recipe of the reference's CPU / GPU consistency test,
python/vesin/tests/test_gpu_consistency.py:17-26, applied to the oracle only).
(i, j, S) must be identical, d and D bit-identical."""

import ctypes

import numpy as np
import pytest

from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _canonical_on_gpu(points, box, periodic, cutoff, full, quantities="ijSdD"):
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    calculator = vesin_b200.NeighborList(cutoff=cutoff, full_list=full, canonical=True)
    outputs = calculator.compute(
        torch.tensor(np.asarray(points, dtype=np.float64), device=device), torch.tensor(np.asarray(box, dtype=np.float64), device=device),
        torch.tensor(np.asarray(periodic, dtype=bool), device=device), quantities, copy=False,
    )
    return calculator, outputs


def _check(points, box, periodic, cutoff, full):
    _, (i, j, S, d, D) = _canonical_on_gpu(points, box, periodic, cutoff, full)
    expected = O.canonical(O.restated_neighbors(points, box, periodic, cutoff, full, "ijSdD"))
    assert len(i) == len(expected["i"])
    assert np.array_equal(i.cpu().numpy().astype(np.int64), expected["i"])
    assert np.array_equal(j.cpu().numpy().astype(np.int64), expected["j"])
    assert np.array_equal(S.cpu().numpy(), expected["S"])
    assert np.array_equal(d.cpu().numpy(), expected["d"])
    assert np.array_equal(D.cpu().numpy(), expected["D"])


@pytest.mark.parametrize("full", [True, False])
def test_diamond_1000(full):
    _check(*W.diamond(5), 5.0, full)


@pytest.mark.parametrize("full", [True, False])
def test_small_triclinic_many_images(full):
    """64 atoms, cutoff 9: the same second index comes with many shifts in a row."""
    _check(*W.small_triclinic(), 9.0, full)


def test_small_systems_and_mixed_periodicity():
    for name, make in W.SMALL_SYSTEMS.items():
        points, box, periodic = make()
        for full in (True, False):
            _check(points, box, periodic, 3.5, full)
    for periodic in ([True, False, True], [False, False, False], [True, True, False]):
        points, box, _ = W.skewed_random(periodic, seed=4)
        _check(points, box, np.array(periodic), 0.35, True)


def test_canonical_without_shifts():
    """Only the indices are requested: rows are ordered by the second index (equal
    ones keep the order of the build)."""
    points, box, periodic = W.diamond(5)
    _, (i, j) = _canonical_on_gpu(points, box, periodic, 5.0, True, "ij")
    expected = O.canonical(O.restated_neighbors(points, box, periodic, 5.0, True, "ijS"))
    assert np.array_equal(i.cpu().numpy().astype(np.int64), expected["i"])
    assert np.array_equal(j.cpu().numpy().astype(np.int64), expected["j"])


def test_diamond_512k_canonical():
    """The benchmark system: 45.6 M pairs compared on the GPU, element by element."""
    import torch

    device = torch.device("cuda", 0)
    points, box, periodic = W.diamond(40)
    calculator, (i, j, S, d, D) = _canonical_on_gpu(points, box, periodic, 5.0, True)
    if O.reference_available():
        cpu = O.ReferenceCPU().compute(points, box, periodic, 5.0, True, "ijSdD", n_threads=0)
    else:
        cpu = O.restated_neighbors(points, box, periodic, 5.0, True, "ijSdD")
    assert len(i) == len(cpu["i"]) == 45629706
    # canonical order of the CPU list: one sort key per pair, sorted with torch on the device
    ci = torch.from_numpy(cpu["i"]).to(device)
    cj = torch.from_numpy(cpu["j"]).to(device)
    cS = torch.from_numpy(cpu["S"]).to(device)
    s_range = int(cS.abs().max())
    width = 2 * s_range + 1
    code = ((cS[:, 0].long() + s_range) * width + (cS[:, 1].long() + s_range)) * width + (cS[:, 2].long() + s_range)
    order = torch.argsort((ci * len(points) + cj) * width**3 + code)
    assert torch.equal(i.view(torch.int64), ci[order])
    assert torch.equal(j.view(torch.int64), cj[order])
    assert torch.equal(S, cS[order])
    assert torch.equal(d, torch.from_numpy(cpu["d"]).to(device)[order])
    assert torch.equal(D, torch.from_numpy(cpu["D"]).to(device)[order])
