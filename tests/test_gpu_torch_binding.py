"""The reference's own TorchScript binding, unmodified, on top of this engine.

tests/torch_binding/Makefile compiles vesin-torch/src/vesin_torch.cpp (the
source of the reference's `libvesin_torch.so`; the custom class
`torch.classes.vesin._NeighborList` and its autograd node,
vesin-torch/src/vesin_torch.cpp:45-479) against include/vesin.h and links it to
vesin_b200/lib/libvesin.so. The tests drive the engine through that binding
with CUDA tensors and compare with the CPU oracle: the same checks as the
other parity tests, one layer further out. Skipped when the binding was not
built (its source is not part of this repository).
"""

import os

import numpy as np
import pytest

from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu

BINDING = os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch_binding", "_ref", "libvesin_torch.so")
RTOL_FP64 = 1e-12


@pytest.fixture(scope="module")
def binding():
    import torch

    if not os.path.exists(BINDING):
        pytest.skip("the reference's torch binding was not compiled (tests/torch_binding/Makefile)")
    assert torch.cuda.is_available()
    torch.ops.load_library(BINDING)
    return torch


def _through_binding(torch, points, box, periodic, cutoff, full, sorted_, quantities="ijSdD"):
    device = torch.device("cuda", 0)
    calculator = torch.classes.vesin._NeighborList(float(cutoff), bool(full), bool(sorted_), "auto", 0)
    outputs = calculator.compute(
        torch.tensor(np.asarray(points, dtype=np.float64), device=device),
        torch.tensor(np.asarray(box, dtype=np.float64), device=device),
        torch.tensor(np.asarray(periodic, dtype=bool), device=device),
        quantities,
        True,
    )
    return {name: value.cpu().numpy() for name, value in zip(quantities, outputs)}


@pytest.mark.parametrize("full", [True, False])
@pytest.mark.parametrize("sorted_", [False, True])
def test_binding_matches_oracle(binding, full, sorted_):
    systems = [
        (W.diamond(4, seed=3), 5.0),
        (W.small_triclinic(48, seed=5), 7.0),
        (W.cluster(), 3.5),
        (W.sheet_2d(), 3.0),
    ]
    for (points, box, periodic), cutoff in systems:
        got = _through_binding(binding, points, box, periodic, cutoff, full, sorted_)
        expected = O.restated_neighbors(points, box, periodic, cutoff, full)
        O.assert_same(got, expected, RTOL_FP64, f"torch binding, full={full}, sorted={sorted_}")
        if sorted_:
            assert np.all(np.diff(got["i"]) >= 0)  # rows ordered by the first index


def test_binding_autograd(binding):
    """Gradients come from the binding's autograd node (vesin_torch.cpp:340-440),
    fed with the pairs, shifts, distances and vectors of this engine."""
    torch = binding
    points, box, periodic = W.diamond(3, seed=11)
    device = torch.device("cuda", 0)
    positions = torch.tensor(points, device=device, requires_grad=True)
    cell = torch.tensor(box, device=device, requires_grad=True)
    calculator = torch.classes.vesin._NeighborList(4.5, True, False, "auto", 0)
    i, j, shifts, distances = calculator.compute(positions, cell, torch.tensor(periodic, device=device), "ijSd", True)
    distances.pow(2).sum().backward()

    # the same sum written with torch operations on the list the oracle gives
    expected = O.restated_neighbors(points, box, periodic, 4.5, True)
    check_positions = torch.tensor(points, device=device, requires_grad=True)
    check_cell = torch.tensor(box, device=device, requires_grad=True)
    index_i = torch.tensor(expected["i"].astype(np.int64), device=device)
    index_j = torch.tensor(expected["j"].astype(np.int64), device=device)
    image = torch.tensor(expected["S"].astype(np.float64), device=device)
    vectors = check_positions[index_j] - check_positions[index_i] + image @ check_cell
    vectors.pow(2).sum().backward()
    assert len(i) == len(index_i)
    torch.testing.assert_close(positions.grad, check_positions.grad, rtol=1e-10, atol=1e-10)
    torch.testing.assert_close(cell.grad, check_cell.grad, rtol=1e-10, atol=1e-9)


def test_binding_reports_engine_errors(binding):
    torch = binding
    device = torch.device("cuda", 0)
    calculator = torch.classes.vesin._NeighborList(3.0, True, False, "auto", 0)
    points = torch.zeros((4, 3), dtype=torch.float64, device=device)
    singular = torch.zeros((3, 3), dtype=torch.float64, device=device)
    with pytest.raises(RuntimeError, match="the box matrix is not invertible"):
        calculator.compute(points, singular, torch.tensor([True, True, True], device=device), "ij", True)
