"""Helpers shared by the GPU tests: run the CUDA engine through the C ABI
(ctypes, via the package's calculator) and bring the result to numpy."""

import numpy as np


def gpu_compute(points, box, periodic, cutoff, full, quantities="ijSdD", algorithm="auto", sorted=False, calculator=None):
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    if calculator is None:
        calculator = vesin_b200.NeighborList(cutoff=cutoff, full_list=full, algorithm=algorithm, sorted=sorted)
    outputs = calculator.compute(
        torch.tensor(np.asarray(points, dtype=np.float64).reshape(-1, 3), device=device),
        torch.tensor(np.asarray(box, dtype=np.float64), device=device),
        torch.tensor(np.asarray(periodic, dtype=bool), device=device),
        quantities,
        copy=False,
    )
    result = {}
    for key, value in zip(quantities, outputs):
        value = value.cpu().numpy()
        if key in "ij":
            value = value.astype(np.int64)
        result[key] = value
    return result


def emulate_sharded(points, box, periodic, cutoff, full, world, quantities="ijSdD", float_io=False):
    """The library's sharded build with every rank on ONE GPU and the test as
    the transport: each rank packs its halo messages
    (vesin_b200_sharded_pack), the messages are copied to the neighbours'
    receive buffers, each rank builds (vesin_b200_sharded_build). Everything a
    real run does except the four NCCL calls. Returns the concatenated lists
    and the per-rank checksums."""
    import ctypes

    import torch

    import vesin_b200
    from vesin_b200._c_api import VesinNeighborList, VesinOptions
    from vesin_b200._neighbors import _view
    from vesin_b200._sharded import list_checksum, owner_of, slab_geometry

    lib = vesin_b200.get_library()
    device = torch.device("cuda", 0)
    points = np.asarray(points, dtype=np.float64)
    box = np.ascontiguousarray(box, dtype=np.float64)
    periodic = np.ascontiguousarray(periodic, dtype=np.bool_)
    axis, _, reach = slab_geometry(box, periodic, cutoff)
    owner = owner_of(points, box, axis, world)
    error = ctypes.c_char_p()

    def check(status):
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))

    handles, inputs, messages = [], [], []
    capacity = int(1.5 * len(points) / world * min(1.0, reach * world)) + 64
    for rank in range(world):
        handle = ctypes.c_void_p()
        check(lib.vesin_b200_sharded_create(None, rank, world, 0, ctypes.byref(handle), ctypes.byref(error)))
        check(lib.vesin_b200_sharded_set_halo_capacity(handle, capacity, ctypes.byref(error)))
        handles.append(handle)
        mine = np.nonzero(owner == rank)[0]
        inputs.append((torch.tensor(points[mine], device=device), torch.tensor(mine, device=device), mine))
    torch.cuda.synchronize()
    try:
        for rank in range(world):
            d_points, d_index, mine = inputs[rank]
            pointers = (ctypes.c_void_p * 4)()
            rows = ctypes.c_size_t()
            check(lib.vesin_b200_sharded_pack(
                handles[rank], d_points.data_ptr(), d_index.data_ptr(), len(mine), box.ctypes.data, periodic.ctypes.data, float(cutoff),
                pointers, ctypes.byref(rows), ctypes.byref(error),
            ))
            messages.append([_view(pointers[k], (rows.value, 4), "<f8", device, None) for k in range(4)])
        for rank in range(world):
            lower, upper = (rank - 1) % world, (rank + 1) % world
            messages[lower][2].copy_(messages[rank][0])  # to lower -> its "from upper"
            messages[upper][3].copy_(messages[rank][1])  # to upper -> its "from lower"
        torch.cuda.synchronize()
        options = VesinOptions()
        options.cutoff = cutoff
        options.full = full
        options.return_shifts = "S" in quantities
        options.return_distances = "d" in quantities
        options.return_vectors = "D" in quantities
        parts, checksums = [], []
        for rank in range(world):
            d_points, d_index, mine = inputs[rank]
            neighbors = VesinNeighborList()
            check(lib.vesin_b200_sharded_build(
                handles[rank], d_points.data_ptr(), d_index.data_ptr(), len(mine), box.ctypes.data, periodic.ctypes.data, options,
                ctypes.byref(neighbors), ctypes.byref(error),
            ))
            n = neighbors.length
            part = {}
            if n:
                pairs = _view(neighbors.pairs, (n, 2), "<u8", device, None).view(torch.int64).cpu().numpy()
            else:
                pairs = np.zeros((0, 2), dtype=np.int64)
            part["i"], part["j"] = pairs[:, 0].copy(), pairs[:, 1].copy()
            if "S" in quantities:
                part["S"] = _view(neighbors.shifts, (n, 3), "<i4", device, None).cpu().numpy() if n else np.zeros((0, 3), np.int32)
            if "d" in quantities:
                part["d"] = _view(neighbors.distances, (n,), "<f8", device, None).cpu().numpy() if n else np.zeros(0)
            if "D" in quantities:
                part["D"] = _view(neighbors.vectors, (n, 3), "<f8", device, None).cpu().numpy() if n else np.zeros((0, 3))
            if full:
                assert np.all(np.isin(part["i"], mine)), "a rank writes the pairs of its own points"
            checksums.append(list_checksum(neighbors))
            parts.append(part)
            lib.vesin_free(ctypes.byref(neighbors))
    finally:
        for handle in handles:
            lib.vesin_b200_sharded_free(handle)
    return {key: np.concatenate([p[key] for p in parts]) for key in parts[0]}, checksums
