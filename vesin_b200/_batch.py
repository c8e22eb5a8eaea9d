"""Batches of independent small systems: one call for all of them
(``vesin_b200_neighbors_batch``), and the split of a batch over the GPUs of a
node (no communication: every rank builds the lists of its own systems).

The reference has no batch notion; its callers loop over systems
(python/vesin/vesin/metatomic/_neighbors.py:197-199).
"""

import ctypes

import numpy as np
import torch

from ._c_api import VesinCUDA, VesinDevice, VesinNeighborList, VesinOptions, get_library
from ._neighbors import _view


def split_batch(system_offsets, world_size):
    """Contiguous chunks of systems, balanced by number of points.

    Returns a list of ``world_size`` pairs ``(first_system, last_system)``
    (half-open). Every system belongs to exactly one chunk; chunks are in rank
    order; a chunk may be empty when there are fewer systems than ranks.
    """
    offsets = np.asarray(system_offsets, dtype=np.int64)
    n_systems = len(offsets) - 1
    total = offsets[-1] - offsets[0]
    bounds = [0]
    for rank in range(1, world_size):
        target = offsets[0] + (total * rank) // world_size
        # first system that starts at or after the target
        cut = int(np.searchsorted(offsets[:-1], target, side="left"))
        bounds.append(min(max(cut, bounds[-1]), n_systems))
    bounds.append(n_systems)
    return [(bounds[r], bounds[r + 1]) for r in range(world_size)]


class BatchNeighborList:
    """Neighbor lists of many small systems at once (CUDA engine)."""

    def __init__(self, cutoff, full_list):
        self._lib = get_library()
        self.cutoff = float(cutoff)
        self.full_list = bool(full_list)
        self._neighbors = VesinNeighborList()

    def __del__(self):
        try:
            if hasattr(self, "_lib") and hasattr(self, "_neighbors"):
                self._lib.vesin_free(ctypes.byref(self._neighbors))
        except (AttributeError, TypeError):
            pass

    def compute(self, points, system_offsets, boxes=None, periodic=None, quantities="ij", global_indices=False, copy=True):
        """``points``: (N, 3) float64 or float32 CUDA tensor, all systems back to back;
        ``system_offsets``: n_systems + 1 integers (host); ``boxes``
        (n_systems, 3, 3) and ``periodic`` (n_systems, 3) CUDA tensors or both
        None for non-periodic systems. Returns ``(outputs, pair_offsets)``:
        the requested quantities as for ``NeighborList.compute`` and a CUDA
        int64 tensor of n_systems + 1 offsets into them."""
        if not isinstance(points, torch.Tensor) or points.device.type != "cuda":
            raise RuntimeError("`points` must be a torch tensor on a CUDA device")
        device = points.device
        # float32 data goes through the fp32 entry point (float d and D come out, decisions stay fp64)
        float_io = points.dtype == torch.float32
        work_dtype = torch.float32 if float_io else torch.float64
        points = points.to(work_dtype).contiguous()
        n_systems = len(system_offsets) - 1
        if (boxes is None) != (periodic is None):
            raise ValueError("`boxes` and `periodic` must be given together")
        if boxes is not None:
            boxes = torch.as_tensor(boxes, device=device).to(work_dtype).contiguous()
            periodic = torch.as_tensor(periodic, device=device).to(torch.bool).contiguous()
            if tuple(boxes.shape) != (n_systems, 3, 3) or tuple(periodic.shape) != (n_systems, 3):
                raise ValueError("`boxes` must be (n_systems, 3, 3) and `periodic` (n_systems, 3)")
        torch.cuda.current_stream(device).synchronize()
        pair_offsets = self.build(points, system_offsets, boxes, periodic, quantities, global_indices)

        n_pairs = self._neighbors.length
        owner = self._neighbors
        finish = (lambda t: t.clone()) if copy else (lambda t: t)
        offsets_out = finish(_view(pair_offsets, (n_systems + 1,), "<u8", device, owner).view(torch.int64))
        if n_pairs == 0:
            pairs = torch.empty((0, 2), dtype=torch.int64, device=device)
            shifts = torch.empty((0, 3), dtype=torch.int32, device=device)
            distances = torch.empty((0,), dtype=work_dtype, device=device)
            vectors = torch.empty((0, 3), dtype=work_dtype, device=device)
        else:
            value = "<f4" if float_io else "<f8"
            pairs = _view(self._neighbors.pairs, (n_pairs, 2), "<u8", device, owner).view(torch.int64)
            shifts = _view(self._neighbors.shifts, (n_pairs, 3), "<i4", device, owner) if "S" in quantities else None
            distances = _view(self._neighbors.distances, (n_pairs,), value, device, owner) if "d" in quantities else None
            vectors = _view(self._neighbors.vectors, (n_pairs, 3), value, device, owner) if "D" in quantities else None
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
        return tuple(data), offsets_out

    def build(self, points, system_offsets, boxes=None, periodic=None, quantities="ij", global_indices=False):
        """The C call alone (``vesin_b200_neighbors_batch`` or its float32 twin):
        contiguous CUDA tensors of one floating-point type whose contents are
        complete. The result stays in the list; returns the device address of
        the n_systems + 1 pair offsets."""
        float_io = points.dtype == torch.float32
        offsets = np.ascontiguousarray(system_offsets, dtype=np.uint64)
        options = VesinOptions()
        options.cutoff = self.cutoff
        options.full = self.full_list
        options.return_shifts = "S" in quantities
        options.return_distances = "d" in quantities
        options.return_vectors = "D" in quantities
        error = ctypes.c_char_p()
        pair_offsets = ctypes.c_void_p()
        entry_point = self._lib.vesin_b200_neighbors_batch_f32 if float_io else self._lib.vesin_b200_neighbors_batch
        status = entry_point(
            points.data_ptr(),
            offsets.ctypes.data,
            len(offsets) - 1,
            boxes.data_ptr() if boxes is not None else None,
            periodic.data_ptr() if periodic is not None else None,
            VesinDevice(VesinCUDA, points.device.index or 0),
            options,
            bool(global_indices),
            ctypes.byref(self._neighbors),
            ctypes.byref(pair_offsets),
            ctypes.byref(error),
        )
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))
        return pair_offsets.value

    @property
    def n_pairs(self):
        return self._neighbors.length
