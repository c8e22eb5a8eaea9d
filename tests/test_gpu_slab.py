"""GPU parity of the slab-decomposed build through the C ABI, with the ranks
emulated one after the other on one GPU. Two routes: vesin_b200_neighbors_slab
(every rank gets its owned points plus the halo a real exchange would bring,
selected by numpy) and the library's own sharded build split into its two
halves (vesin_b200_sharded_pack / _build: packing kernel, messages moved by the
test, build from owned points + received messages). The union over ranks must
be the CPU oracle's list of the whole system: (i, j, S) bit for bit, d and D
bit-identical. The same build over real NCCL is tests/test_gpu_sharded_nccl.py."""

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


@pytest.mark.parametrize("full", [True, False])
@pytest.mark.parametrize("world", [2, 3, 8])
def test_library_sharded_build_emulated(full, world):
    from gpu_utils import emulate_sharded
    from vesin_b200._sharded import checksum_of_arrays

    points, box, periodic = W.liquid(40000, seed=16)
    points = points + np.array([500.0, -210.0, 1234.5])  # most points far outside the box
    got, checksums = emulate_sharded(points, box, periodic, 6.0, full, world)
    expected = O.restated_neighbors(points, box, periodic, 6.0, full, "ijSdD")
    O.assert_same(got, expected, 1e-12, f"world={world} full={full}")
    got, expected = O.canonical(got), O.canonical(expected)
    assert np.array_equal(got["d"], expected["d"]) and np.array_equal(got["D"], expected["D"])
    # the device checksums of the ranks add up to the checksum of the oracle's list
    total = [sum(c[k] for c in checksums) % (1 << 64) for k in range(3)] + [sum(c[3] for c in checksums)]
    assert tuple(total) == checksum_of_arrays(expected["i"], expected["j"], expected["S"], expected["d"])


def test_library_sharded_build_mixed_periodicity():
    """A slab system with a non-periodic direction: the extent of the points is
    taken from the first build and checked by the later ones."""
    from gpu_utils import emulate_sharded

    points, box, periodic = W.liquid(20000, seed=5)
    periodic = np.array([True, False, True])
    for full in (True, False):
        got, _ = emulate_sharded(points, box, periodic, 6.0, full, 4)
        expected = O.restated_neighbors(points, box, periodic, 6.0, full, "ijSdD")
        O.assert_same(got, expected, 1e-12, f"mixed periodicity full={full}")


def test_slab_float32_entry_point():
    """vesin_b200_neighbors_slab_f32: float points and box in, float d and D
    out; pairs and shifts are those of the upcast inputs."""
    import torch

    import vesin_b200
    from vesin_b200._sharded import choose_axis, local_set

    device = torch.device("cuda", 0)
    points, box, periodic = W.liquid(30000, seed=8)
    points32, box32 = points.astype(np.float32), box.astype(np.float32)
    upcast, box_up = points32.astype(np.float64), box32.astype(np.float64)
    world = 3
    axis = choose_axis(box_up, periodic)
    parts = []
    for rank in range(world):
        owned, halo = local_set(upcast, box_up, periodic, 6.0, rank, world)
        local = np.concatenate([owned, halo])
        calculator = vesin_b200.ShardedNeighborList(cutoff=6.0, full_list=False)
        i, j, S, d, D = calculator.build_local(
            torch.tensor(points32[local], device=device), torch.tensor(local, device=device), len(owned), box_up, periodic, axis, rank,
            world, "ijSdD",
        )
        assert d.dtype == torch.float32 and D.dtype == torch.float32
        assert vesin_b200.get_library().vesin_b200_list_value_bytes(calculator._neighbors) == 4
        parts.append({"i": i.cpu().numpy(), "j": j.cpu().numpy(), "S": S.cpu().numpy(), "d": d.cpu().numpy(), "D": D.cpu().numpy()})
    got = {key: np.concatenate([p[key] for p in parts]) for key in parts[0]}
    expected = O.restated_neighbors(upcast, box_up, periodic, 6.0, False, "ijSdD")
    got, expected = O.canonical(got), O.canonical(expected)
    assert np.array_equal(got["i"], expected["i"]) and np.array_equal(got["j"], expected["j"]) and np.array_equal(got["S"], expected["S"])
    assert np.array_equal(got["d"], expected["d"].astype(np.float32)), "d is the fp64 result rounded once"
    assert np.array_equal(got["D"], expected["D"].astype(np.float32))


def test_global_index_range_is_checked():
    import torch

    import vesin_b200
    from vesin_b200._sharded import choose_axis, local_set

    device = torch.device("cuda", 0)
    points, box, periodic = W.liquid(5000, seed=2)
    axis = choose_axis(box, periodic)
    owned, halo = local_set(points, box, periodic, 6.0, 0, 2)
    local = np.concatenate([owned, halo]).astype(np.int64)
    local[7] = 1 << 31
    calculator = vesin_b200.ShardedNeighborList(cutoff=6.0, full_list=True)
    with pytest.raises(RuntimeError, match="does not fit 31 bits"):
        calculator.build_local(torch.tensor(points[np.concatenate([owned, halo])], device=device), torch.tensor(local, device=device),
                               len(owned), box, periodic, axis, 0, 2)


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
            counts = torch.zeros(3, dtype=torch.int64, device=device)
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


def test_pack_halo_refuses_host_memory():
    """Arrays that are not device memory are refused before anything is launched."""
    import ctypes

    import torch

    import vesin_b200

    lib = vesin_b200.get_library()
    device = torch.device("cuda", 0)
    host_points = np.zeros((10, 3))
    d_index = torch.arange(10, device=device)
    message = torch.zeros((11, 4), dtype=torch.float64, device=device)
    counts = torch.zeros(3, dtype=torch.int64, device=device)
    column = (ctypes.c_double * 3)(0.0, 0.0, 0.1)
    error = ctypes.c_char_p()
    status = lib.vesin_b200_pack_halo(
        host_points.ctypes.data, d_index.data_ptr(), 10, column, 0.0, 0.5, 0.1, message.data_ptr(), message.data_ptr(), 10,
        counts.data_ptr(), ctypes.byref(error),
    )
    assert status == 1 and b"must be device memory" in error.value
    torch.cuda.synchronize()
    assert float(message.abs().sum()) == 0.0
