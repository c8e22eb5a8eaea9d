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


def test_pack_halo_kernel():
    """vesin_b200_pack_halo against the numpy selection, for every rank of a
    4-rank decomposition, and the capacity overflow report."""
    import ctypes

    import torch

    import vesin_b200
    from vesin_b200._sharded import choose_axis, halo_masks, halo_reach, owner_of, wrapped_fraction

    lib = vesin_b200.get_library()
    device = torch.device("cuda", 0)
    points, box, periodic = W.liquid(30000, seed=4)
    points = points + np.array([300.0, -170.0, 55.0])  # far outside the box
    world, cutoff = 4, 6.0
    axis = choose_axis(box, periodic)
    reach = halo_reach(box, axis, cutoff)
    column = (ctypes.c_double * 3)(*np.linalg.inv(box)[:, axis])
    owner = owner_of(points, box, axis, world)
    for rank in range(world):
        mine = np.nonzero(owner == rank)[0]
        g = wrapped_fraction(points[mine], box, axis)
        down, up = halo_masks(g, rank, world, reach)
        for capacity in (len(mine), 10):
            d_points = torch.tensor(points[mine], device=device)
            d_index = torch.tensor(mine, device=device)
            to_lower = torch.zeros((capacity + 1, 4), dtype=torch.float64, device=device)
            to_upper = torch.zeros((capacity + 1, 4), dtype=torch.float64, device=device)
            counts = torch.zeros(2, dtype=torch.int64, device=device)
            error = ctypes.c_char_p()
            status = lib.vesin_b200_pack_halo(
                d_points.data_ptr(), d_index.data_ptr(), len(mine), column, rank / world, (rank + 1) / world, reach,
                to_lower.data_ptr(), to_upper.data_ptr(), capacity, counts.data_ptr(), ctypes.byref(error),
            )
            assert status == 0, error.value
            torch.cuda.synchronize()
            for message, mask in ((to_lower, down), (to_upper, up)):
                message = message.cpu().numpy()
                expected = mine[mask]
                assert int(message[0, 0]) == len(expected)  # the count is reported even when it does not fit
                if len(expected) <= capacity:
                    got_index = message[1 : 1 + len(expected), 3].copy().view(np.int64)
                    order = np.argsort(got_index)
                    assert np.array_equal(got_index[order], np.sort(expected))
                    assert np.array_equal(message[1 : 1 + len(expected), :3][order], points[np.sort(expected)])
