"""Slab decomposition of one large periodic system over the GPUs of a node.

Every rank owns the points of one slab of the box (a range of the wrapped
fractional coordinate along the cut direction). One exchange per build: each
rank sends the points within the cutoff of its two faces to its two
neighbours, then builds the pairs of its own points. For CUDA tensors all of
it happens inside the library (``vesin_b200_sharded_neighbors``: packing
kernel, ncclSend / ncclRecv over NVLink, local build); ``torch.distributed`` is
only used once, to hand the communicator's id to every rank. Indices in the
result are indices into the whole system; shifts refer to the whole box.
``exchange_halo`` is the same exchange on ``torch.distributed`` send/recv, used
with gloo to test the host logic without GPUs.

The reference has no multi-GPU notion (one system, one device per call,
vesin/include/vesin.h:103-108); this layer is additive.
"""

import ctypes

import numpy as np
import torch

from ._c_api import (
    N_STAGES,
    STAGE_NAMES,
    UNIQUE_ID_BYTES,
    VesinB200Slab,
    VesinCUDA,
    VesinDevice,
    VesinNeighborList,
    VesinOptions,
    get_library,
)
from ._neighbors import _view


def slab_geometry(box, periodic, cutoff):
    """(axis, inverse column, reach) of the slab decomposition of `box`, as the
    library computes them (``vesin_b200_slab_geometry``)."""
    lib = get_library()
    box = np.ascontiguousarray(box, dtype=np.float64)
    periodic = np.ascontiguousarray(periodic, dtype=np.bool_)
    axis = ctypes.c_int()
    column = (ctypes.c_double * 3)()
    reach = ctypes.c_double()
    error = ctypes.c_char_p()
    status = lib.vesin_b200_slab_geometry(
        box.ctypes.data, periodic.ctypes.data, float(cutoff), ctypes.byref(axis), column, ctypes.byref(reach), ctypes.byref(error)
    )
    if status != 0:
        raise RuntimeError(error.value.decode("utf8"))
    return axis.value, np.array(column[:]), reach.value


def list_checksum(neighbors):
    """Checksum of a list on its device (``vesin_b200_list_checksum``): four
    Python ints."""
    lib = get_library()
    words = (ctypes.c_uint64 * 4)()
    error = ctypes.c_char_p()
    if lib.vesin_b200_list_checksum(ctypes.byref(neighbors), words, ctypes.byref(error)) != 0:
        raise RuntimeError(error.value.decode("utf8"))
    return tuple(int(w) for w in words)


def checksum_of_arrays(i, j, S=None, d=None):
    """The same checksum from host arrays (numpy), e.g. of a list the CPU
    reference built. `d` float64 or float32; its raw bits enter the third word."""
    mask = np.uint64(0xFFFFFFFFFFFFFFFF)

    def mix(x):
        x = x ^ (x >> np.uint64(33))
        x = x * np.uint64(0xFF51AFD7ED558CCD)
        x = x ^ (x >> np.uint64(33))
        x = x * np.uint64(0xC4CEB9FE1A85EC53)
        return x ^ (x >> np.uint64(33))

    with np.errstate(over="ignore"):
        i = np.asarray(i).astype(np.uint64)
        j = np.asarray(j).astype(np.uint64)
        key = i * np.uint64(0x9E3779B97F4A7C15) + j * np.uint64(0xC2B2AE3D27D4EB4F)
        if S is not None:
            S = np.asarray(S).astype(np.int32).view(np.uint32).astype(np.uint64).reshape(-1, 3)
            key = key + S[:, 0] * np.uint64(0x165667B19E3779F9)
            key = key + S[:, 1] * np.uint64(0x27D4EB2F165667C5)
            key = key + S[:, 2] * np.uint64(0x85EBCA77C2B2AE63)
        if d is None:
            bits = np.zeros(len(key), dtype=np.uint64)
        else:
            d = np.ascontiguousarray(d)
            bits = d.view(np.uint32).astype(np.uint64) if d.dtype == np.float32 else d.astype(np.float64).view(np.uint64)
        words = (
            mix(key).sum(dtype=np.uint64),
            mix(key ^ np.uint64(0x5555555555555555)).sum(dtype=np.uint64),
            mix(key + bits * np.uint64(0xD6E8FEB86659FD93)).sum(dtype=np.uint64),
        )
    return tuple(int(w & mask) for w in words) + (len(key),)


def face_distances(box):
    """Distance between opposite faces of the cell along each of its vectors."""
    box = np.asarray(box, dtype=np.float64)
    inverse = np.linalg.inv(box)
    return 1.0 / np.linalg.norm(inverse, axis=0)


def choose_axis(box, periodic):
    """Cut along the periodic direction with the largest face distance; on ties
    the later direction wins (pencils of cells run along the first one)."""
    distances = face_distances(box)
    best = -1
    for axis in (2, 1, 0):
        if periodic[axis] and (best < 0 or distances[axis] > distances[best]):
            best = axis
    if best < 0:
        raise ValueError("slab decomposition needs at least one periodic direction")
    return best


def wrapped_fraction(points, box, axis):
    """Fractional coordinate along `axis`, wrapped into [0, 1). Works on torch
    tensors (any device) and numpy arrays."""
    inverse = np.linalg.inv(np.asarray(box, dtype=np.float64))[:, axis]
    if isinstance(points, torch.Tensor):
        column = torch.as_tensor(inverse, dtype=points.dtype, device=points.device)
        f = points @ column
        g = f - torch.floor(f)
        return torch.where(g >= 1.0, torch.zeros_like(g), g)
    f = np.asarray(points) @ inverse
    g = f - np.floor(f)
    g[g >= 1.0] = 0.0
    return g


def owner_of(points, box, axis, world_size):
    """Rank that owns every point."""
    g = wrapped_fraction(points, box, axis)
    if isinstance(g, torch.Tensor):
        return torch.clamp((g * world_size).to(torch.int64), 0, world_size - 1)
    return np.clip((g * world_size).astype(np.int64), 0, world_size - 1)


def halo_reach(box, axis, cutoff):
    """Fractional thickness of the layer a rank has to send to a neighbour."""
    return cutoff * (1.0 + 1e-9) / face_distances(box)[axis]


def halo_masks(g, rank, world_size, reach):
    """Which of a rank's own points go to its lower / upper neighbour."""
    lower = rank / world_size
    upper = (rank + 1) / world_size
    return (g - lower) <= reach, (upper - g) <= reach


def local_set(points, box, periodic, cutoff, rank, world_size):
    """numpy reference of what a rank ends up holding: (owned indices, halo
    indices). Used by the single-process tests and to check the exchange."""
    axis = choose_axis(box, periodic)
    g = wrapped_fraction(points, box, axis)
    owner = np.clip((g * world_size).astype(np.int64), 0, world_size - 1)
    reach = halo_reach(box, axis, cutoff)
    owned = np.nonzero(owner == rank)[0]
    left, right = (rank - 1) % world_size, (rank + 1) % world_size
    # the upper layer of the lower neighbour, the lower layer of the upper neighbour
    from_left = np.nonzero((owner == left) & (((left + 1) / world_size - g) <= reach))[0]
    from_right = np.nonzero((owner == right) & ((g - right / world_size) <= reach))[0]
    return owned, np.concatenate([from_right, from_left])


def exchange_halo(points, global_index, box, axis, cutoff, group=None):
    """One halo exchange. `points` (n, 3) float64 and `global_index` (n,) int64
    are this rank's owned points; returns the received halo as a pair of
    tensors on the same device. Collective over `group`."""
    import torch.distributed as dist

    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    left, right = (rank - 1) % world, (rank + 1) % world
    g = wrapped_fraction(points, box, axis)
    to_left, to_right = halo_masks(g, rank, world, halo_reach(box, axis, cutoff))

    def pack(mask):
        selected = torch.nonzero(mask).flatten()
        record = torch.empty((selected.numel(), 4), dtype=torch.float64, device=points.device)
        record[:, :3] = points.index_select(0, selected)
        record[:, 3] = global_index.index_select(0, selected).view(torch.float64)
        return record

    send_left, send_right = pack(to_left), pack(to_right)
    counts = torch.tensor([send_left.shape[0], send_right.shape[0]], dtype=torch.int64, device=points.device)
    gathered = [torch.zeros_like(counts) for _ in range(world)]
    dist.all_gather(gathered, counts, group=group)
    all_counts = torch.stack(gathered).cpu()
    # the upper neighbour's lower layer and the lower neighbour's upper layer
    recv_right = torch.empty((int(all_counts[right, 0]), 4), dtype=torch.float64, device=points.device)
    recv_left = torch.empty((int(all_counts[left, 1]), 4), dtype=torch.float64, device=points.device)

    def peer(r):
        return r if group is None else dist.get_global_rank(group, r)

    # With two ranks both neighbours are the same peer: messages between two
    # ranks keep their order, so sends (lower, upper) pair with the peer's
    # receives (from upper, from lower).
    operations = []
    if send_left.shape[0]:
        operations.append(dist.P2POp(dist.isend, send_left, peer(left), group))
    if send_right.shape[0]:
        operations.append(dist.P2POp(dist.isend, send_right, peer(right), group))
    if recv_right.shape[0]:
        operations.append(dist.P2POp(dist.irecv, recv_right, peer(right), group))
    if recv_left.shape[0]:
        operations.append(dist.P2POp(dist.irecv, recv_left, peer(left), group))
    if operations:
        for request in dist.batch_isend_irecv(operations):
            request.wait()
    halo = torch.cat([recv_right, recv_left])
    return halo[:, :3].contiguous(), halo[:, 3].contiguous().view(torch.int64)


class ShardedNeighborList:
    """Neighbor list of one periodic system spread over the ranks of a process
    group, one slab per rank (CUDA tensors; one process per GPU)."""

    def __init__(self, cutoff, full_list, group=None):
        self._lib = get_library()
        self.cutoff = float(cutoff)
        self.full_list = bool(full_list)
        self.group = group
        self._neighbors = VesinNeighborList()
        self._handle = None
        self._box_key = None

    def __del__(self):
        try:
            if hasattr(self, "_lib") and hasattr(self, "_neighbors"):
                self._lib.vesin_free(ctypes.byref(self._neighbors))
                if getattr(self, "_handle", None):
                    self._lib.vesin_b200_sharded_free(self._handle)
                    self._handle = None
        except (AttributeError, TypeError):
            pass

    def close(self):
        """Release the list and the communicator (collective: every rank calls it)."""
        self._lib.vesin_free(ctypes.byref(self._neighbors))
        ctypes.memset(ctypes.byref(self._neighbors), 0, ctypes.sizeof(self._neighbors))
        if self._handle:
            self._lib.vesin_b200_sharded_free(self._handle)
            self._handle = None

    def _options(self, quantities):
        options = VesinOptions()
        options.cutoff = self.cutoff
        options.full = self.full_list
        options.return_shifts = "S" in quantities
        options.return_distances = "d" in quantities
        options.return_vectors = "D" in quantities
        return options

    def _outputs(self, device, quantities, copy, value_dtype=torch.float64):
        n_pairs = self._neighbors.length
        owner = self._neighbors
        finish = (lambda t: t.clone()) if copy else (lambda t: t)
        typestr = "<f4" if value_dtype == torch.float32 else "<f8"
        if n_pairs == 0:
            pairs = torch.empty((0, 2), dtype=torch.int64, device=device)
            shifts = torch.empty((0, 3), dtype=torch.int32, device=device)
            distances = torch.empty((0,), dtype=value_dtype, device=device)
            vectors = torch.empty((0, 3), dtype=value_dtype, device=device)
        else:
            pairs = _view(self._neighbors.pairs, (n_pairs, 2), "<u8", device, owner).view(torch.int64)
            shifts = _view(self._neighbors.shifts, (n_pairs, 3), "<i4", device, owner) if "S" in quantities else None
            distances = _view(self._neighbors.distances, (n_pairs,), typestr, device, owner) if "d" in quantities else None
            vectors = _view(self._neighbors.vectors, (n_pairs, 3), typestr, device, owner) if "D" in quantities else None
        data = []
        for quantity in quantities:
            if quantity == "P":
                data.append(finish(pairs))
            elif quantity == "i":
                data.append(finish(pairs[:, 0]))
            elif quantity == "j":
                data.append(finish(pairs[:, 1]))
            elif quantity == "S":
                data.append(finish(shifts))
            elif quantity == "d":
                data.append(finish(distances))
            elif quantity == "D":
                data.append(finish(vectors))
        return tuple(data)

    def build_local(self, points, global_index, n_owned, box, periodic, axis, rank, world_size, quantities="ij", copy=True):
        """The local build alone, with the halo brought by the caller: `points`
        holds the owned points first, then the halo
        (``vesin_b200_neighbors_slab``)."""
        device = points.device
        float_io = points.dtype == torch.float32
        points = points.to(torch.float32 if float_io else torch.float64).contiguous()
        global_index = global_index.to(torch.int64).contiguous()
        d_box, d_periodic = self._device_box(box, periodic, device, torch.float32 if float_io else torch.float64)
        slab = VesinB200Slab(int(axis), rank / world_size, (rank + 1) / world_size)
        torch.cuda.current_stream(device).synchronize()
        error = ctypes.c_char_p()
        entry_point = self._lib.vesin_b200_neighbors_slab_f32 if float_io else self._lib.vesin_b200_neighbors_slab
        status = entry_point(
            points.data_ptr(),
            points.shape[0],
            int(n_owned),
            global_index.data_ptr(),
            d_box.data_ptr(),
            d_periodic.data_ptr(),
            slab,
            VesinDevice(VesinCUDA, device.index or 0),
            self._options(quantities),
            ctypes.byref(self._neighbors),
            ctypes.byref(error),
        )
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))
        return self._outputs(device, quantities, copy, points.dtype)

    def _device_box(self, box, periodic, device, dtype=torch.float64):
        """Device copies of box and periodicity, re-used while they do not change."""
        box = np.ascontiguousarray(box, dtype=np.float64)
        periodic = np.ascontiguousarray(periodic, dtype=bool)
        key = (box.tobytes(), periodic.tobytes(), str(device), str(dtype))
        if self._box_key != key:
            self._box_key = key
            self._d_box = torch.as_tensor(box, device=device).to(dtype).contiguous()
            self._d_periodic = torch.as_tensor(periodic, device=device).contiguous()
        return self._d_box, self._d_periodic

    def _ensure_handle(self, device):
        """First build: rank 0 of the group draws the communicator's id, every
        rank gets it through ``torch.distributed`` and joins (collective)."""
        if self._handle:
            return
        import torch.distributed as dist

        rank = dist.get_rank(self.group)
        world = dist.get_world_size(self.group)
        error = ctypes.c_char_p()
        unique = (ctypes.c_ubyte * UNIQUE_ID_BYTES)()
        if rank == 0 and self._lib.vesin_b200_sharded_unique_id(unique, ctypes.byref(error)) != 0:
            raise RuntimeError(error.value.decode("utf8"))
        payload = [bytes(unique)]
        source = 0 if self.group is None else dist.get_global_rank(self.group, 0)
        dist.broadcast_object_list(payload, src=source, group=self.group)
        unique = (ctypes.c_ubyte * UNIQUE_ID_BYTES).from_buffer_copy(payload[0])
        handle = ctypes.c_void_p()
        status = self._lib.vesin_b200_sharded_create(unique, rank, world, device.index or 0, ctypes.byref(handle), ctypes.byref(error))
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))
        self._handle = handle

    def set_halo_capacity(self, records):
        """Records a halo message can hold; the same value on every rank."""
        error = ctypes.c_char_p()
        if self._lib.vesin_b200_sharded_set_halo_capacity(self._handle, int(records), ctypes.byref(error)) != 0:
            raise RuntimeError(error.value.decode("utf8"))

    def compute(self, points, global_index, box, periodic, quantities="ij", copy=True):
        """`points` (n, 3) and `global_index` (n,): the points this rank owns
        (see ``owner_of``), CUDA tensors, float64 or float32. `box` (3, 3) and
        `periodic` (3,): host values, the same on every rank. Returns this
        rank's pairs. Collective over the group."""
        if points.device.type != "cuda":
            raise RuntimeError("sharded lists are built on CUDA devices: there is no CPU engine in this package")
        device = points.device
        float_io = points.dtype == torch.float32
        points = points.to(torch.float32 if float_io else torch.float64).contiguous()
        global_index = global_index.to(torch.int64).contiguous()
        # inputs produced on another stream of the caller must be complete: the library works on its own streams
        torch.cuda.current_stream(device).synchronize()
        self.build(points, global_index, box, periodic, quantities)
        return self._outputs(device, quantities, copy, points.dtype)

    def build(self, points, global_index, box, periodic, quantities="ij"):
        """The C call alone (``vesin_b200_sharded_neighbors`` or its float32
        twin): `points` float64 or float32 and `global_index` int64, contiguous
        CUDA tensors whose contents are complete. The result stays in the
        list; returns the number of pairs of this rank."""
        float_io = points.dtype == torch.float32
        self._ensure_handle(points.device)
        h_box = np.ascontiguousarray(box, dtype=np.float32 if float_io else np.float64)
        h_periodic = np.ascontiguousarray(periodic, dtype=np.bool_)
        error = ctypes.c_char_p()
        entry_point = self._lib.vesin_b200_sharded_neighbors_f32 if float_io else self._lib.vesin_b200_sharded_neighbors
        status = entry_point(
            self._handle,
            points.data_ptr(),
            global_index.data_ptr(),
            points.shape[0],
            h_box.ctypes.data,
            h_periodic.ctypes.data,
            self._options(quantities),
            ctypes.byref(self._neighbors),
            ctypes.byref(error),
        )
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))
        return self._neighbors.length

    def outputs(self, device, quantities, value_dtype=torch.float64):
        """Zero-copy views of the arrays the last build left in the list."""
        return self._outputs(device, quantities, False, value_dtype)

    def checksum(self):
        """Checksum of this rank's part of the list (add the ranks' words mod 2^64)."""
        return list_checksum(self._neighbors)

    def stage_times(self):
        """Device milliseconds of the last build: packing, exchange and the
        stages of the local build (needs ``vesin_b200.set_profiling(True)``)."""
        pack_ms, exchange_ms = ctypes.c_double(), ctypes.c_double()
        if self._lib.vesin_b200_sharded_stage_times(self._handle, ctypes.byref(pack_ms), ctypes.byref(exchange_ms)) != 0:
            return None
        values = (ctypes.c_double * N_STAGES)()
        if self._lib.vesin_b200_stage_times(ctypes.byref(self._neighbors), values) != 0:
            return None
        times = {"pack": pack_ms.value, "exchange": exchange_ms.value}
        times.update(dict(zip(STAGE_NAMES, values)))
        return times
