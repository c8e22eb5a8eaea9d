"""GPU parity at the benchmark sizes: the 512 000-atom diamond build (full and
half lists) and a 2 097 152-atom liquid (the slab-decomposed configuration at
one eighth of its size), against the unmodified reference CPU library where it
is available (oracle/_ref travels with the repository as a built file) and the
C restatement otherwise, plus size-independent properties of the lists.
Canonical sorting and comparison run on the GPU with torch (45 M rows)."""

import numpy as np
import pytest

from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _cpu_reference(points, box, periodic, cutoff, full):
    if O.reference_available():
        return O.ReferenceCPU().compute(points, box, periodic, cutoff, full, "ijSdD", n_threads=0)
    return O.restated_neighbors(points, box, periodic, cutoff, full, "ijSdD")


def _keys(torch, i, j, S, n_points, s_range):
    """One int64 per pair, ordered like the lexicographic (i, j, Sx, Sy, Sz)."""
    width = 2 * s_range + 1
    code = ((S[:, 0].long() + s_range) * width + (S[:, 1].long() + s_range)) * width + (S[:, 2].long() + s_range)
    return (i.long() * n_points + j.long()) * (width**3) + code


def _gpu_build(torch, points, box, periodic, cutoff, full, sorted=False):
    import vesin_b200

    device = torch.device("cuda", 0)
    calculator = vesin_b200.NeighborList(cutoff=cutoff, full_list=full, sorted=sorted)
    i, j, S, d, D = calculator.compute(
        torch.tensor(points, device=device), torch.tensor(box, device=device), torch.tensor(periodic, device=device), "ijSdD", copy=False
    )
    return calculator, (i.view(torch.int64) if i.dtype != torch.int64 else i, j.view(torch.int64) if j.dtype != torch.int64 else j, S, d, D)


def _compare(torch, gpu, cpu, n_points, cutoff):
    device = torch.device("cuda", 0)
    i, j, S, d, D = gpu
    s_range = int(max(int(S.abs().max().item()) if len(S) else 0, int(np.abs(cpu["S"]).max()) if len(cpu["S"]) else 0))
    assert len(i) == len(cpu["i"]), f"{len(i)} pairs on the GPU, {len(cpu['i'])} on the CPU"
    keys = _keys(torch, i, j, S, n_points, s_range)
    order = torch.argsort(keys)
    ci = torch.from_numpy(cpu["i"]).to(device)
    cj = torch.from_numpy(cpu["j"]).to(device)
    cS = torch.from_numpy(cpu["S"]).to(device)
    cpu_keys = _keys(torch, ci, cj, cS, n_points, s_range)
    cpu_order = torch.argsort(cpu_keys)
    assert torch.equal(keys[order], cpu_keys[cpu_order]), "(i, j, S) differ"
    assert torch.unique_consecutive(keys[order]).numel() == keys.numel(), "duplicate pairs"
    cd = torch.from_numpy(cpu["d"]).to(device)[cpu_order]
    cD = torch.from_numpy(cpu["D"]).to(device)[cpu_order]
    assert float((d[order] - cd).abs().max()) <= 1e-12 * cutoff
    assert float((D[order] - cD).abs().max()) <= 1e-12 * cutoff
    # in fact the arithmetic is the reference's, operation for operation
    assert torch.equal(d[order], cd)
    assert torch.equal(D[order], cD)


def _properties(torch, gpu, n_points, cutoff, full):
    i, j, S, d, D = gpu
    assert float(d.max()) < cutoff
    assert torch.equal(d, torch.sqrt((D[:, 0] * D[:, 0] + D[:, 1] * D[:, 1]) + D[:, 2] * D[:, 2]))
    assert int(i.min()) >= 0 and int(i.max()) < n_points and int(j.min()) >= 0 and int(j.max()) < n_points
    if full:
        s_range = int(S.abs().max().item())
        forward = torch.sort(_keys(torch, i, j, S, n_points, s_range)).values
        backward = torch.sort(_keys(torch, j, i, -S, n_points, s_range)).values
        assert torch.equal(forward, backward), "a full list holds (j, i, -S) for every (i, j, S)"
    else:
        assert bool((i <= j).all())


@pytest.mark.parametrize("full", [True, False])
def test_diamond_512k(full):
    import torch

    points, box, periodic = W.diamond(40)
    calculator, gpu = _gpu_build(torch, points, box, periodic, 5.0, full)
    assert len(gpu[0]) == (45629706 if full else 22814853)
    _properties(torch, gpu, len(points), 5.0, full)
    cpu = _cpu_reference(points, box, periodic, 5.0, full)
    _compare(torch, gpu, cpu, len(points), 5.0)


def test_diamond_512k_float32():
    """The fp32 entry point at the size it is benchmarked on: float points and
    box in, float d and D out. Pairs and shifts are the CPU reference's on the
    upcast inputs; d and D are its fp64 values rounded once."""
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    points, box, periodic = W.diamond(40)
    points32, box32 = points.astype(np.float32), box.astype(np.float32)
    calculator = vesin_b200.NeighborList(cutoff=5.0, full_list=True)
    i, j, S, d, D = calculator.compute(
        torch.tensor(points32, device=device), torch.tensor(box32, device=device), torch.tensor(periodic, device=device), "ijSdD", copy=False
    )
    assert d.dtype == torch.float32 and D.dtype == torch.float32
    assert vesin_b200.get_library().vesin_b200_list_value_bytes(calculator._neighbors) == 4
    cpu = _cpu_reference(points32.astype(np.float64), box32.astype(np.float64), periodic, 5.0, True)
    n_points = len(points)
    s_range = int(max(int(S.abs().max().item()), int(np.abs(cpu["S"]).max())))
    assert len(i) == len(cpu["i"])
    keys = _keys(torch, i.view(torch.int64), j.view(torch.int64), S, n_points, s_range)
    order = torch.argsort(keys)
    cpu_keys = _keys(
        torch, torch.from_numpy(cpu["i"]).to(device), torch.from_numpy(cpu["j"]).to(device), torch.from_numpy(cpu["S"]).to(device), n_points, s_range
    )
    cpu_order = torch.argsort(cpu_keys)
    assert torch.equal(keys[order], cpu_keys[cpu_order]), "(i, j, S) differ"
    assert torch.equal(d[order], torch.from_numpy(cpu["d"].astype(np.float32)).to(device)[cpu_order])
    assert torch.equal(D[order], torch.from_numpy(cpu["D"].astype(np.float32)).to(device)[cpu_order])


def test_diamond_512k_sorted_half():
    import torch

    points, box, periodic = W.diamond(40)
    calculator, gpu = _gpu_build(torch, points, box, periodic, 5.0, False, sorted=True)
    assert len(gpu[0]) == 22814853
    assert bool((gpu[0][1:] >= gpu[0][:-1]).all()), "sorted lists are ordered by the first index"
    cpu = _cpu_reference(points, box, periodic, 5.0, False)
    _compare(torch, gpu, cpu, len(points), 5.0)


def test_liquid_2m_half():
    import torch

    points, box, periodic = W.liquid(1 << 21)
    calculator, gpu = _gpu_build(torch, points, box, periodic, 6.0, False)
    _properties(torch, gpu, len(points), 6.0, False)
    cpu = _cpu_reference(points, box, periodic, 6.0, False)
    _compare(torch, gpu, cpu, len(points), 6.0)
