"""GPU parity of the slab-decomposed build (vesin_b200_neighbors_slab, through
the C ABI). The ranks are emulated one after the other on one GPU: every rank
gets its owned points plus the halo a real exchange would bring, builds its
share, and the union over ranks must be the CPU oracle's list of the whole
system: (i, j, S) bit for bit, d and D bit-identical."""

import numpy as np
import pytest

from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _sharded_union(points, box, periodic, cutoff, full, world):
    import torch

    import vesin_b200
    from vesin_b200._sharded import choose_axis, local_set

    device = torch.device("cuda", 0)
    axis = choose_axis(box, periodic)
    parts = []
    for rank in range(world):
        owned, halo = local_set(points, box, periodic, cutoff, rank, world)
        local = np.concatenate([owned, halo])
        calculator = vesin_b200.ShardedNeighborList(cutoff=cutoff, full_list=full)
        i, j, S, d, D = calculator.build_local(
            torch.tensor(points[local], device=device),
            torch.tensor(local, device=device),
            len(owned),
            box,
            periodic,
            axis,
            rank,
            world,
            "ijSdD",
        )
        part = {"i": i.cpu().numpy(), "j": j.cpu().numpy(), "S": S.cpu().numpy(), "d": d.cpu().numpy(), "D": D.cpu().numpy()}
        if full:
            assert np.all(np.isin(part["i"], owned)), "a rank writes the pairs of its own points"
        parts.append(part)
    return {key: np.concatenate([p[key] for p in parts]) for key in parts[0]}


@pytest.mark.parametrize("full", [True, False])
@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_liquid_slabs(full, world):
    points, box, periodic = W.liquid(40000, seed=15)  # 106 A box: slabs of 13 A at 8 ranks, cutoff 6
    got = _sharded_union(points, box, periodic, 6.0, full, world)
    expected = O.restated_neighbors(points, box, periodic, 6.0, full, "ijSdD")
    O.assert_same(got, expected, 1e-12, f"world={world} full={full}")
    got, expected = O.canonical(got), O.canonical(expected)
    assert np.array_equal(got["d"], expected["d"]) and np.array_equal(got["D"], expected["D"])


@pytest.mark.parametrize("full", [True, False])
def test_triclinic_crystal_slabs(full):
    """Skewed box, points outside the box, dense cells (several tiles per unit)."""
    points, box, periodic = W.diamond(8, seed=3)
    shear = np.array([[1.0, 0.0, 0.0], [0.15, 1.0, 0.0], [0.1, -0.2, 1.0]])
    box = box @ shear
    points = points @ shear + np.array([40.0, -33.0, 71.0])
    for world in (2, 4):
        got = _sharded_union(points, box, periodic, 5.0, full, world)
        expected = O.restated_neighbors(points, box, periodic, 5.0, full, "ijSdD")
        O.assert_same(got, expected, 1e-12, f"world={world} full={full}")


def test_slab_limits():
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    points, box, periodic = W.diamond(4, seed=3)  # 14.3 A box
    calculator = vesin_b200.ShardedNeighborList(cutoff=5.0, full_list=True)
    args = (torch.tensor(points, device=device), torch.arange(len(points), device=device), len(points), box, periodic, 2)
    with pytest.raises(RuntimeError, match="thinner than the cutoff"):
        calculator.build_local(*args, 0, 4)
    with pytest.raises(RuntimeError, match="longer than the box"):
        calculator.build_local(*args, 0, 2)
    with pytest.raises(RuntimeError, match="must be a periodic direction"):
        calculator.build_local(args[0], args[1], args[2], box, [True, True, False], 2, 0, 2)
