"""Slab decomposition of one large periodic system over the GPUs of a node.

Every rank owns the points of one slab of the box (a range of the wrapped
fractional coordinate along the cut direction). One exchange per build: each
rank sends the points within the cutoff of its two faces to its two
neighbours (``torch.distributed`` send/recv: NCCL over NVLink for CUDA
tensors, gloo in the CPU tests), then builds the pairs of its own points with
``vesin_b200_neighbors_slab``. Indices in the result are indices into the
whole system; shifts refer to the whole box.

The reference has no multi-GPU notion (one system, one device per call,
vesin/include/vesin.h:103-108); this layer is additive.
"""

import ctypes

import numpy as np
import torch

from ._c_api import VesinB200Slab, VesinCUDA, VesinDevice, VesinNeighborList, VesinOptions, get_library
from ._neighbors import _view


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
    group, one slab per rank."""

    def __init__(self, cutoff, full_list, group=None):
        self._lib = get_library()
        self.cutoff = float(cutoff)
        self.full_list = bool(full_list)
        self.group = group
        self._neighbors = VesinNeighborList()
        # records per halo message, the same on every rank; None: agreed on at the
        # first build (twice the uniform-density estimate of the fullest rank)
        self.halo_capacity = None
        self._box_key = None
        self._messages = None

    def __del__(self):
        try:
            if hasattr(self, "_lib") and hasattr(self, "_neighbors"):
                self._lib.vesin_free(ctypes.byref(self._neighbors))
        except (AttributeError, TypeError):
            pass

    def build_local(self, points, global_index, n_owned, box, periodic, axis, rank, world_size, quantities="ij", copy=True):
        """The local build alone: `points` holds the owned points first, then
        the halo. This is the C ABI call; `compute` adds the exchange."""
        device = points.device
        points = points.to(torch.float64).contiguous()
        global_index = global_index.to(torch.int64).contiguous()
        d_box, d_periodic = self._device_box(box, periodic, device)
        options = VesinOptions()
        options.cutoff = self.cutoff
        options.full = self.full_list
        options.return_shifts = "S" in quantities
        options.return_distances = "d" in quantities
        options.return_vectors = "D" in quantities
        slab = VesinB200Slab(int(axis), rank / world_size, (rank + 1) / world_size)
        torch.cuda.current_stream(device).synchronize()
        error = ctypes.c_char_p()
        status = self._lib.vesin_b200_neighbors_slab(
            points.data_ptr(),
            points.shape[0],
            int(n_owned),
            global_index.data_ptr(),
            d_box.data_ptr(),
            d_periodic.data_ptr(),
            slab,
            VesinDevice(VesinCUDA, device.index or 0),
            options,
            ctypes.byref(self._neighbors),
            ctypes.byref(error),
        )
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))
        n_pairs = self._neighbors.length
        owner = self._neighbors
        finish = (lambda t: t.clone()) if copy else (lambda t: t)
        if n_pairs == 0:
            pairs = torch.empty((0, 2), dtype=torch.int64, device=device)
            shifts = torch.empty((0, 3), dtype=torch.int32, device=device)
            distances = torch.empty((0,), dtype=torch.float64, device=device)
            vectors = torch.empty((0, 3), dtype=torch.float64, device=device)
        else:
            pairs = _view(self._neighbors.pairs, (n_pairs, 2), "<u8", device, owner).view(torch.int64)
            shifts = _view(self._neighbors.shifts, (n_pairs, 3), "<i4", device, owner) if "S" in quantities else None
            distances = _view(self._neighbors.distances, (n_pairs,), "<f8", device, owner) if "d" in quantities else None
            vectors = _view(self._neighbors.vectors, (n_pairs, 3), "<f8", device, owner) if "D" in quantities else None
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

    def _device_box(self, box, periodic, device):
        """Device copies of box and periodicity, re-used while they do not change."""
        box = np.ascontiguousarray(box, dtype=np.float64)
        periodic = np.ascontiguousarray(periodic, dtype=bool)
        key = (box.tobytes(), periodic.tobytes(), str(device))
        if self._box_key != key:
            self._box_key = key
            self._d_box = torch.as_tensor(box, device=device).contiguous()
            self._d_periodic = torch.as_tensor(periodic, device=device).contiguous()
            inverse = np.linalg.inv(box)
            self._inverse_columns = [(ctypes.c_double * 3)(*inverse[:, axis]) for axis in range(3)]
        return self._d_box, self._d_periodic

    def _exchange_on_device(self, points, global_index, box, axis, rank, world):
        """Halo exchange for CUDA tensors: one kernel selects and packs both
        messages (vesin_b200_pack_halo), the messages have a fixed capacity so no
        sizes are exchanged, and the host waits once, for the four record counts."""
        import torch.distributed as dist

        device = points.device
        n = points.shape[0]
        reach = halo_reach(box, axis, self.cutoff)
        # every rank must use the same message size: agree on it once (the
        # largest of the ranks' estimates, twice the uniform-density halo)
        if self.halo_capacity is None:
            wanted = torch.tensor([max(4096, int(2.0 * n * reach * world) + 1024)], dtype=torch.int64, device=device)
            dist.all_reduce(wanted, op=dist.ReduceOp.MAX, group=self.group)
            self.halo_capacity = int(wanted.item())
        capacity = self.halo_capacity
        if self._messages is None or self._messages[0].shape[0] != capacity + 1 or self._messages[0].device != device:
            self._messages = [torch.empty((capacity + 1, 4), dtype=torch.float64, device=device) for _ in range(4)]
            self._counts = torch.zeros(2, dtype=torch.int64, device=device)
        to_lower, to_upper, from_upper, from_lower = self._messages
        if torch.cuda.current_stream(device) != torch.cuda.default_stream(device):
            torch.cuda.current_stream(device).synchronize()  # the pack kernel runs on the default stream
        error = ctypes.c_char_p()
        status = self._lib.vesin_b200_pack_halo(
            points.data_ptr(), global_index.data_ptr(), n, self._inverse_columns[axis], rank / world, (rank + 1) / world, reach,
            to_lower.data_ptr(), to_upper.data_ptr(), capacity, self._counts.data_ptr(), ctypes.byref(error),
        )
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))
        left, right = (rank - 1) % world, (rank + 1) % world

        def peer(r):
            return r if self.group is None else dist.get_global_rank(self.group, r)

        # two ranks: both neighbours are the same peer; sends (lower, upper)
        # pair with the peer's receives (from upper, from lower)
        operations = [
            dist.P2POp(dist.isend, to_lower, peer(left), self.group),
            dist.P2POp(dist.isend, to_upper, peer(right), self.group),
            dist.P2POp(dist.irecv, from_upper, peer(right), self.group),
            dist.P2POp(dist.irecv, from_lower, peer(left), self.group),
        ]
        for request in dist.batch_isend_irecv(operations):
            request.wait()
        counts = torch.stack([from_upper[0, 0], from_lower[0, 0], to_lower[0, 0], to_upper[0, 0]]).cpu()
        if float(counts.max()) > capacity:
            raise RuntimeError(
                f"a halo message needs {int(counts.max())} records but holds {capacity}: "
                "set `halo_capacity` (same value on every rank) on the calculator"
            )
        n_upper, n_lower = int(counts[0]), int(counts[1])
        halo_points = torch.cat([from_upper[1 : 1 + n_upper, :3], from_lower[1 : 1 + n_lower, :3]])
        halo_index = torch.cat([from_upper[1 : 1 + n_upper, 3], from_lower[1 : 1 + n_lower, 3]]).view(torch.int64)
        return halo_points, halo_index

    def compute(self, points, global_index, box, periodic, quantities="ij", copy=True):
        """`points` (n, 3) and `global_index` (n,): the points this rank owns
        (see ``owner_of``), CUDA tensors. `box` (3, 3) and `periodic` (3,):
        host values, the same on every rank. Returns this rank's pairs."""
        import torch.distributed as dist

        box = np.asarray(box, dtype=np.float64)
        periodic = np.asarray(periodic, dtype=bool)
        rank = dist.get_rank(self.group)
        world = dist.get_world_size(self.group)
        if world == 1:
            raise RuntimeError("a single rank has no slab to exchange with: use vesin_b200.NeighborList")
        axis = choose_axis(box, periodic)
        if points.device.type == "cuda":
            points = points.to(torch.float64).contiguous()
            global_index = global_index.to(torch.int64).contiguous()
            self._device_box(box, periodic, points.device)
            halo_points, halo_index = self._exchange_on_device(points, global_index, box, axis, rank, world)
        else:
            halo_points, halo_index = exchange_halo(points, global_index, box, axis, self.cutoff, self.group)
        local_points = torch.cat([points, halo_points])
        local_index = torch.cat([global_index, halo_index])
        return self.build_local(local_points, local_index, points.shape[0], box, periodic, axis, rank, world, quantities, copy)
