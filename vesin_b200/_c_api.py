"""ctypes declarations of the C ABI (include/vesin.h, include/vesin_b200.h)
and the loader of the in-tree shared library. There is no fallback: when the
library is missing, loading fails with instructions to build it."""

import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
# VESIN_B200_LIBRARY points at another build of the same library (e.g. one made
# with extra compiler flags); the default is the in-tree build.
LIBRARY_PATH = os.environ.get("VESIN_B200_LIBRARY", os.path.join(HERE, "lib", "libvesin.so"))

VesinUnknownDevice = 0
VesinCPU = 1
VesinCUDA = 2

VesinAutoAlgorithm = 0
VesinBruteForce = 1
VesinCellList = 2

N_STAGES = 8
STAGE_NAMES = ("bounds", "bin", "scan_cells", "scatter", "count", "scan_rows", "emit", "halo")


class VesinDevice(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("device_id", ctypes.c_int)]


class VesinOptions(ctypes.Structure):
    _fields_ = [
        ("cutoff", ctypes.c_double),
        ("full", ctypes.c_bool),
        ("sorted", ctypes.c_bool),
        ("algorithm", ctypes.c_int),
        ("n_threads", ctypes.c_int32),
        ("return_shifts", ctypes.c_bool),
        ("return_distances", ctypes.c_bool),
        ("return_vectors", ctypes.c_bool),
        ("skin", ctypes.c_double),
    ]


class VesinB200Slab(ctypes.Structure):
    _fields_ = [("axis", ctypes.c_int), ("lower", ctypes.c_double), ("upper", ctypes.c_double)]


class VesinNeighborList(ctypes.Structure):
    _fields_ = [
        ("length", ctypes.c_size_t),
        ("device", VesinDevice),
        ("pairs", ctypes.c_void_p),
        ("shifts", ctypes.c_void_p),
        ("distances", ctypes.c_void_p),
        ("vectors", ctypes.c_void_p),
        ("opaque", ctypes.c_void_p),
    ]


EXPORTED_SYMBOLS = (
    "vesin_neighbors",
    "vesin_free",
    "vesin_list_libraries",
    "vesin_b200_set_profiling",
    "vesin_b200_stage_times",
    "vesin_b200_version",
    "vesin_b200_neighbors_no_alloc",
    "vesin_b200_neighbors_batch",
    "vesin_b200_neighbors_batch_f32",
    "vesin_b200_neighbors_slab",
    "vesin_b200_pack_halo",
    "vesin_b200_neighbors_f32",
    "vesin_b200_neighbors_canonical",
    "vesin_b200_neighbors_slab_f32",
    "vesin_b200_slab_geometry",
    "vesin_b200_sharded_unique_id",
    "vesin_b200_sharded_create",
    "vesin_b200_sharded_free",
    "vesin_b200_sharded_set_halo_capacity",
    "vesin_b200_sharded_neighbors",
    "vesin_b200_sharded_neighbors_f32",
    "vesin_b200_sharded_pack",
    "vesin_b200_sharded_build",
    "vesin_b200_sharded_stage_times",
    "vesin_b200_list_value_bytes",
    "vesin_b200_list_checksum",
)
UNIQUE_ID_BYTES = 128
NO_ALLOC_MAX_POINTS = 32768


def build_library(verbose=False):
    """Compile vesin_b200/lib/libvesin.so with nvcc for sm_100a."""
    subprocess.run(
        ["make", "-C", os.path.join(HERE, "csrc")] + ([] if verbose else ["-s"]),
        check=True,
    )


_LIBRARY = None


def get_library():
    global _LIBRARY
    if _LIBRARY is not None:
        return _LIBRARY
    if not os.path.exists(LIBRARY_PATH):
        raise ImportError(
            f"{LIBRARY_PATH} does not exist: build it with `make -C vesin_b200/csrc` "
            "(needs nvcc; there is no CPU fallback)"
        )
    lib = ctypes.CDLL(LIBRARY_PATH)
    lib.vesin_neighbors.restype = ctypes.c_int
    lib.vesin_neighbors.argtypes = [
        ctypes.c_void_p,  # points
        ctypes.c_size_t,  # n_points
        ctypes.c_void_p,  # box
        ctypes.c_void_p,  # periodic
        VesinDevice,
        VesinOptions,
        ctypes.POINTER(VesinNeighborList),
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_free.restype = None
    lib.vesin_free.argtypes = [ctypes.POINTER(VesinNeighborList)]
    lib.vesin_list_libraries.restype = None
    lib.vesin_list_libraries.argtypes = [ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_size_t)]
    lib.vesin_b200_set_profiling.restype = None
    lib.vesin_b200_set_profiling.argtypes = [ctypes.c_int]
    lib.vesin_b200_stage_times.restype = ctypes.c_int
    lib.vesin_b200_stage_times.argtypes = [ctypes.POINTER(VesinNeighborList), ctypes.POINTER(ctypes.c_double)]
    lib.vesin_b200_neighbors_no_alloc.restype = ctypes.c_int
    lib.vesin_b200_neighbors_no_alloc.argtypes = [
        ctypes.c_void_p,  # points
        ctypes.c_size_t,
        ctypes.c_void_p,  # box
        ctypes.c_void_p,  # periodic
        ctypes.c_int,  # device_id
        ctypes.c_double,  # cutoff
        ctypes.c_bool,  # full
        ctypes.c_size_t,  # capacity
        ctypes.c_void_p,  # pairs
        ctypes.c_void_p,  # shifts
        ctypes.c_void_p,  # distances
        ctypes.c_void_p,  # vectors
        ctypes.POINTER(ctypes.c_size_t),
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_b200_neighbors_batch.restype = ctypes.c_int
    lib.vesin_b200_neighbors_batch.argtypes = [
        ctypes.c_void_p,  # points (device)
        ctypes.c_void_p,  # system_offsets (host, size_t)
        ctypes.c_size_t,  # n_systems
        ctypes.c_void_p,  # boxes (device or NULL)
        ctypes.c_void_p,  # periodic (device or NULL)
        VesinDevice,
        VesinOptions,
        ctypes.c_bool,  # global_indices
        ctypes.POINTER(VesinNeighborList),
        ctypes.POINTER(ctypes.c_void_p),  # pair_offsets (out, device)
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_b200_neighbors_batch_f32.restype = ctypes.c_int
    lib.vesin_b200_neighbors_batch_f32.argtypes = lib.vesin_b200_neighbors_batch.argtypes
    lib.vesin_b200_neighbors_slab.restype = ctypes.c_int
    lib.vesin_b200_neighbors_slab.argtypes = [
        ctypes.c_void_p,  # points (device): owned first, then halo
        ctypes.c_size_t,  # n_points
        ctypes.c_size_t,  # n_owned
        ctypes.c_void_p,  # global_index (device, int64)
        ctypes.c_void_p,  # box (device)
        ctypes.c_void_p,  # periodic (device)
        VesinB200Slab,
        VesinDevice,
        VesinOptions,
        ctypes.POINTER(VesinNeighborList),
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_b200_neighbors_f32.restype = ctypes.c_int
    lib.vesin_b200_neighbors_f32.argtypes = lib.vesin_neighbors.argtypes
    lib.vesin_b200_neighbors_canonical.restype = ctypes.c_int
    lib.vesin_b200_neighbors_canonical.argtypes = lib.vesin_neighbors.argtypes
    lib.vesin_b200_neighbors_slab_f32.restype = ctypes.c_int
    lib.vesin_b200_neighbors_slab_f32.argtypes = lib.vesin_b200_neighbors_slab.argtypes
    lib.vesin_b200_slab_geometry.restype = ctypes.c_int
    lib.vesin_b200_slab_geometry.argtypes = [
        ctypes.c_void_p,  # box (host, 3x3 double)
        ctypes.c_void_p,  # periodic (host, 3 bool)
        ctypes.c_double,  # cutoff
        ctypes.POINTER(ctypes.c_int),  # axis
        ctypes.POINTER(ctypes.c_double),  # inverse_column (3)
        ctypes.POINTER(ctypes.c_double),  # reach
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_b200_sharded_unique_id.restype = ctypes.c_int
    lib.vesin_b200_sharded_unique_id.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_char_p)]
    lib.vesin_b200_sharded_create.restype = ctypes.c_int
    lib.vesin_b200_sharded_create.argtypes = [
        ctypes.c_void_p,  # id (128 bytes) or NULL
        ctypes.c_int,  # rank
        ctypes.c_int,  # world_size
        ctypes.c_int,  # device_id
        ctypes.POINTER(ctypes.c_void_p),  # handle (out)
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_b200_sharded_free.restype = None
    lib.vesin_b200_sharded_free.argtypes = [ctypes.c_void_p]
    lib.vesin_b200_sharded_set_halo_capacity.restype = ctypes.c_int
    lib.vesin_b200_sharded_set_halo_capacity.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_char_p)]
    sharded_build = [
        ctypes.c_void_p,  # handle
        ctypes.c_void_p,  # points (device): the points this rank owns
        ctypes.c_void_p,  # global_index (device, int64)
        ctypes.c_size_t,  # n_owned
        ctypes.c_void_p,  # box (HOST)
        ctypes.c_void_p,  # periodic (HOST)
        VesinOptions,
        ctypes.POINTER(VesinNeighborList),
        ctypes.POINTER(ctypes.c_char_p),
    ]
    for function in (lib.vesin_b200_sharded_neighbors, lib.vesin_b200_sharded_neighbors_f32, lib.vesin_b200_sharded_build):
        function.restype = ctypes.c_int
        function.argtypes = sharded_build
    lib.vesin_b200_sharded_pack.restype = ctypes.c_int
    lib.vesin_b200_sharded_pack.argtypes = [
        ctypes.c_void_p,  # handle
        ctypes.c_void_p,  # points (device)
        ctypes.c_void_p,  # global_index (device)
        ctypes.c_size_t,  # n_owned
        ctypes.c_void_p,  # box (HOST)
        ctypes.c_void_p,  # periodic (HOST)
        ctypes.c_double,  # cutoff
        ctypes.POINTER(ctypes.c_void_p),  # messages (out, 4 device addresses)
        ctypes.POINTER(ctypes.c_size_t),  # rows (out)
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_b200_sharded_stage_times.restype = ctypes.c_int
    lib.vesin_b200_sharded_stage_times.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
    lib.vesin_b200_list_value_bytes.restype = ctypes.c_int
    lib.vesin_b200_list_value_bytes.argtypes = [ctypes.POINTER(VesinNeighborList)]
    lib.vesin_b200_list_checksum.restype = ctypes.c_int
    lib.vesin_b200_list_checksum.argtypes = [
        ctypes.POINTER(VesinNeighborList),
        ctypes.POINTER(ctypes.c_uint64),  # checksum (4)
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_b200_pack_halo.restype = ctypes.c_int
    lib.vesin_b200_pack_halo.argtypes = [
        ctypes.c_void_p,  # points (device)
        ctypes.c_void_p,  # global_index (device)
        ctypes.c_size_t,
        ctypes.POINTER(ctypes.c_double),  # inverse_column (host, 3)
        ctypes.c_double,  # lower
        ctypes.c_double,  # upper
        ctypes.c_double,  # reach
        ctypes.c_void_p,  # to_lower (device)
        ctypes.c_void_p,  # to_upper (device)
        ctypes.c_size_t,  # capacity
        ctypes.c_void_p,  # counts (device, 3 x uint64)
        ctypes.POINTER(ctypes.c_char_p),
    ]
    lib.vesin_b200_version.restype = ctypes.c_char_p
    lib.vesin_b200_version.argtypes = []
    _LIBRARY = lib
    return lib
