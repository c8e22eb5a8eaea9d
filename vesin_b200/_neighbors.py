"""Host-side mirror of the reference's Python calculator
(python/vesin/vesin/_neighbors.py:68-381): same class name, constructor
arguments, ``compute`` signature, quantities string and error behaviour, on
top of the CUDA engine's C ABI.

Inputs may be torch tensors on a CUDA device (outputs are torch tensors on the
same device, zero-copy views when ``copy=False``) or anything numpy can convert
(the data is copied to the current CUDA device, and the outputs come back as
numpy arrays). There is no CPU engine behind this class.
"""

import ctypes

import numpy as np
import torch

from ._c_api import (
    STAGE_NAMES,
    N_STAGES,
    VesinAutoAlgorithm,
    VesinBruteForce,
    VesinCellList,
    VesinCUDA,
    VesinDevice,
    VesinNeighborList,
    VesinOptions,
    VesinUnknownDevice,
    get_library,
)


class _DeviceArray:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so
    torch can wrap it without copying; keeps `owner` alive."""

    def __init__(self, ptr, shape, typestr, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {
            "shape": tuple(shape),
            "typestr": typestr,
            "data": (int(ptr), False),
            "version": 2,
            "strides": None,
        }


def _view(ptr, shape, typestr, device, owner):
    return torch.as_tensor(_DeviceArray(ptr, shape, typestr, owner), device=device)


class NeighborList:
    """A neighbor list calculator (CUDA engine)."""

    def __init__(self, cutoff, full_list, sorted=False, algorithm="auto", skin=0.0, n_threads=0, canonical=False):
        """Arguments as the reference's calculator; `canonical` (an addition)
        asks for the list sorted by (i, j, Sx, Sy, Sz) instead of by i only."""
        self._lib = get_library()
        self.canonical = bool(canonical)
        self.cutoff = float(cutoff)
        self.full_list = bool(full_list)
        self.sorted = bool(sorted)
        self.skin = float(skin)
        self.algorithm = algorithm
        self.n_threads = int(n_threads)
        if self.n_threads < 0:
            raise ValueError("n_threads must be zero or a positive integer")
        self._neighbors = VesinNeighborList()

    def __del__(self):
        try:
            if hasattr(self, "_lib") and hasattr(self, "_neighbors"):
                self._lib.vesin_free(ctypes.byref(self._neighbors))
        except (AttributeError, TypeError):
            pass  # interpreter shutdown: modules are already gone

    @property
    def algorithm(self):
        return self._algorithm

    @algorithm.setter
    def algorithm(self, value):
        algorithm = value.lower()
        self._algorithm = algorithm
        if algorithm == "auto":
            self._c_algorithm = VesinAutoAlgorithm
        elif algorithm == "brute_force":
            self._c_algorithm = VesinBruteForce
        elif algorithm == "cell_list":
            self._c_algorithm = VesinCellList
        else:
            raise ValueError(f"Unknown algorithm '{algorithm}'. Must be one of 'auto', 'brute_force', or 'cell_list'.")

    def compute(self, points, box, periodic, quantities="ij", copy=True):
        """Compute the neighbor list of the system (``points``, ``box``,
        ``periodic``) and return the requested ``quantities``: any of ``i``,
        ``j``, ``P`` (both indices), ``S`` (periodic shifts), ``d`` (distances)
        and ``D`` (vectors), as a tuple in the order given."""
        if not torch.cuda.is_available():
            raise RuntimeError("vesin_b200 needs a CUDA device: there is no CPU engine in this package")

        from_torch = isinstance(points, torch.Tensor)
        if from_torch:
            if points.device.type != "cuda":
                raise RuntimeError("torch inputs must live on a CUDA device (there is no CPU engine in this package)")
            device = points.device
            if points.requires_grad or (isinstance(box, torch.Tensor) and box.requires_grad):
                raise RuntimeError("NeighborList.compute does not support autograd for torch tensors")
            box = torch.as_tensor(box, device=device)
            initial_dtype = points.dtype
            if box.dtype != initial_dtype:
                raise RuntimeError(f"`points` and `box` must have the same dtype, got {points.dtype} and {box.dtype}")
        else:
            points = np.asarray(points)
            box = np.asarray(box)
            if box.dtype != points.dtype:
                raise RuntimeError(f"`points` and `box` must have the same dtype, got {points.dtype} and {box.dtype}")
            initial_dtype = points.dtype
            device = torch.device("cuda", torch.cuda.current_device())

        if isinstance(periodic, (bool, np.bool_)):
            periodic = [bool(periodic)] * 3

        if tuple(box.shape) != (3, 3):
            raise ValueError("`box` must be a 3x3 matrix")
        if len(points.shape) != 2 or points.shape[1] != 3:
            raise ValueError("`points` must be a nx3 array")

        # float32 data goes through the fp32 entry point: no upcast pass before
        # the call, no downcast pass after it (the decisions are fp64 either way)
        if from_torch:
            floating = initial_dtype.is_floating_point
            out_dtype = initial_dtype if floating else torch.float64
            float_io = initial_dtype == torch.float32 and not self.canonical  # the canonical entry point is fp64
            work_dtype = torch.float32 if float_io else torch.float64
            d_points = points.to(work_dtype).contiguous()
            d_box = box.to(work_dtype).contiguous()
            d_periodic = torch.as_tensor(periodic, device=device).to(torch.bool).contiguous()
        else:
            floating = np.issubdtype(initial_dtype, np.floating)
            out_dtype = initial_dtype if floating else np.float64
            float_io = initial_dtype == np.float32 and not self.canonical
            work_dtype = np.float32 if float_io else np.float64
            d_points = torch.from_numpy(np.ascontiguousarray(points, dtype=work_dtype)).to(device, non_blocking=False)
            d_box = torch.from_numpy(np.ascontiguousarray(box, dtype=work_dtype)).to(device)
            d_periodic = torch.from_numpy(np.ascontiguousarray(periodic, dtype=np.bool_)).to(device)
        if tuple(d_periodic.shape) != (3,):
            raise ValueError(
                "`periodic` must be a single boolean or a sequence of three "
                f"booleans, got {periodic} of type {type(periodic)}"
            )

        options = VesinOptions()
        options.cutoff = self.cutoff
        options.full = self.full_list
        options.sorted = self.sorted
        options.return_shifts = "S" in quantities
        options.return_distances = "d" in quantities
        options.return_vectors = "D" in quantities
        options.algorithm = self._c_algorithm
        options.skin = self.skin
        options.n_threads = self.n_threads

        c_device = VesinDevice(VesinCUDA, device.index or 0)
        if self._neighbors.device.type != VesinUnknownDevice and (
            self._neighbors.device.type != c_device.type or self._neighbors.device.device_id != c_device.device_id
        ):
            self._lib.vesin_free(ctypes.byref(self._neighbors))
            ctypes.memset(ctypes.byref(self._neighbors), 0, ctypes.sizeof(self._neighbors))

        # inputs produced on another stream of the caller must be complete:
        # the engine works on its own stream
        torch.cuda.current_stream(device).synchronize()
        error_message = ctypes.c_char_p()
        entry_point = self._lib.vesin_b200_neighbors_f32 if float_io else self._lib.vesin_neighbors
        if self.canonical:
            entry_point = self._lib.vesin_b200_neighbors_canonical
        status = entry_point(
            d_points.data_ptr(),
            d_points.shape[0],
            d_box.data_ptr(),
            d_periodic.data_ptr(),
            c_device,
            options,
            ctypes.byref(self._neighbors),
            ctypes.byref(error_message),
        )
        if status != 0:
            raise RuntimeError(error_message.value.decode("utf8"))

        n_pairs = self._neighbors.length
        torch_float = out_dtype if from_torch else torch.from_numpy(np.zeros(0, dtype=out_dtype)).dtype
        if n_pairs == 0:
            pairs = torch.empty((0, 2), dtype=torch.uint64, device=device)
            shifts = torch.empty((0, 3), dtype=torch.int32, device=device)
            distances = torch.empty((0,), dtype=torch_float, device=device)
            vectors = torch.empty((0, 3), dtype=torch_float, device=device)
        else:
            owner = self._neighbors
            pairs = _view(self._neighbors.pairs, (n_pairs, 2), "<u8", device, owner)
            shifts = distances = vectors = None
            if "S" in quantities:
                shifts = _view(self._neighbors.shifts, (n_pairs, 3), "<i4", device, owner)
            if "d" in quantities:
                distances = _view(self._neighbors.distances, (n_pairs,), "<f4" if float_io else "<f8", device, owner).to(torch_float)
            if "D" in quantities:
                vectors = _view(self._neighbors.vectors, (n_pairs, 3), "<f4" if float_io else "<f8", device, owner).to(torch_float)

        def finish(tensor):
            if from_torch:
                return tensor.clone() if copy else tensor
            return tensor.cpu().numpy()

        data = []
        for quantity in quantities:
            if quantity == "P":
                data.append(finish(pairs))
            if quantity == "i":
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

    def stage_times(self):
        """Device milliseconds per stage of the last build (needs
        ``vesin_b200.set_profiling(True)`` before the build)."""
        values = (ctypes.c_double * N_STAGES)()
        if self._lib.vesin_b200_stage_times(ctypes.byref(self._neighbors), values) != 0:
            return None
        return dict(zip(STAGE_NAMES, values))


def set_profiling(enabled):
    get_library().vesin_b200_set_profiling(int(bool(enabled)))
