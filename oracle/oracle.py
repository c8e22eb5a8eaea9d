"""
TEST INFRASTRUCTURE ONLY -- ctypes front-ends for the two CPU checkers.

* ``restated_neighbors``  : the plain-C restatement in ``vesin_oracle.c``
* ``reference_neighbors`` : the unmodified reference CPU path, compiled by
  ``oracle/Makefile`` into ``oracle/_ref/libvesin_ref.so`` and called through
  the reference's own C ABI (``vesin_neighbors`` with ``VesinDevice{CPU, 0}``,
  vesin/include/vesin.h:191-200)
* ``canonical`` : the comparison recipe of the reference's CPU/GPU consistency
  test (python/vesin/tests/test_gpu_consistency.py:17-26): lexicographic sort
  on (i, j, Sx, Sy, Sz), then element-wise comparison.

Nothing in the product package imports this module; only the tests, the smoke
check and the CPU legs of the benchmark do.
"""

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
RESTATED_PATH = os.path.join(HERE, "libvesin_oracle.so")
REFERENCE_PATH = os.path.join(HERE, "_ref", "libvesin_ref.so")


def build(force=False):
    """Compile the restatement (always) and the reference CPU path (when the
    reference tree is present). Prebuilt files are kept otherwise."""
    if force or not os.path.exists(RESTATED_PATH) or not os.path.exists(REFERENCE_PATH):
        subprocess.run(["make", "-s", "-C", HERE], check=True)


class _OracleList(ctypes.Structure):
    _fields_ = [
        ("length", ctypes.c_size_t),
        ("capacity", ctypes.c_size_t),
        ("pairs", ctypes.POINTER(ctypes.c_size_t)),
        ("shifts", ctypes.POINTER(ctypes.c_int32)),
        ("distances", ctypes.POINTER(ctypes.c_double)),
        ("vectors", ctypes.POINTER(ctypes.c_double)),
    ]


# Mirror of the reference C ABI structs (vesin/include/vesin.h:49-163), used
# only to drive the reference CPU library.
class _VesinOptions(ctypes.Structure):
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


class _VesinDevice(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("device_id", ctypes.c_int)]


class _VesinNeighborList(ctypes.Structure):
    _fields_ = [
        ("length", ctypes.c_size_t),
        ("device", _VesinDevice),
        ("pairs", ctypes.POINTER(ctypes.c_size_t)),
        ("shifts", ctypes.POINTER(ctypes.c_int32)),
        ("distances", ctypes.POINTER(ctypes.c_double)),
        ("vectors", ctypes.POINTER(ctypes.c_double)),
        ("opaque", ctypes.c_void_p),
    ]


_restated = None
_reference = None


def _restated_lib():
    global _restated
    if _restated is None:
        if not os.path.exists(RESTATED_PATH):
            build()
        lib = ctypes.CDLL(RESTATED_PATH)
        lib.vesin_oracle_neighbors.restype = ctypes.c_int
        lib.vesin_oracle_neighbors.argtypes = [
            ctypes.c_void_p,
            ctypes.c_size_t,
            ctypes.c_void_p,
            ctypes.c_void_p,
            ctypes.c_double,
            ctypes.c_int,
            ctypes.c_int,
            ctypes.c_int,
            ctypes.c_int,
            ctypes.POINTER(_OracleList),
            ctypes.c_char_p,
            ctypes.c_size_t,
        ]
        lib.vesin_oracle_free.restype = None
        lib.vesin_oracle_free.argtypes = [ctypes.POINTER(_OracleList)]
        _restated = lib
    return _restated


def reference_available():
    return os.path.exists(REFERENCE_PATH)


def _reference_lib():
    global _reference
    if _reference is None:
        lib = ctypes.CDLL(REFERENCE_PATH)
        lib.vesin_neighbors.restype = ctypes.c_int
        lib.vesin_neighbors.argtypes = [
            ctypes.c_void_p,
            ctypes.c_size_t,
            ctypes.c_void_p,
            ctypes.c_void_p,
            _VesinDevice,
            _VesinOptions,
            ctypes.POINTER(_VesinNeighborList),
            ctypes.POINTER(ctypes.c_char_p),
        ]
        lib.vesin_free.restype = None
        lib.vesin_free.argtypes = [ctypes.POINTER(_VesinNeighborList)]
        _reference = lib
    return _reference


def _prepare(points, box, periodic):
    points = np.ascontiguousarray(points, dtype=np.float64).reshape(-1, 3)
    box = np.ascontiguousarray(box, dtype=np.float64).reshape(3, 3)
    if isinstance(periodic, (bool, np.bool_)):
        periodic = [periodic] * 3
    periodic = np.ascontiguousarray(periodic, dtype=np.bool_).reshape(3)
    return points, box, periodic


def _collect(lst, n, quantities):
    out = {}
    pairs = np.ctypeslib.as_array(lst.pairs, shape=(n, 2)).astype(np.int64) if n else np.zeros((0, 2), np.int64)
    out["i"] = pairs[:, 0].copy()
    out["j"] = pairs[:, 1].copy()
    if "S" in quantities:
        out["S"] = np.ctypeslib.as_array(lst.shifts, shape=(n, 3)).copy() if n else np.zeros((0, 3), np.int32)
    if "d" in quantities:
        out["d"] = np.ctypeslib.as_array(lst.distances, shape=(n,)).copy() if n else np.zeros((0,), np.float64)
    if "D" in quantities:
        out["D"] = np.ctypeslib.as_array(lst.vectors, shape=(n, 3)).copy() if n else np.zeros((0, 3), np.float64)
    return out


def restated_neighbors(points, box, periodic, cutoff, full_list, quantities="ijSdD"):
    """Run the C restatement; returns a dict with keys i, j and any of S, d, D
    (unsorted: the order is the reference's single-thread order)."""
    lib = _restated_lib()
    points, box, periodic = _prepare(points, box, periodic)
    lst = _OracleList()
    err = ctypes.create_string_buffer(512)
    status = lib.vesin_oracle_neighbors(
        points.ctypes.data,
        points.shape[0],
        box.ctypes.data,
        periodic.ctypes.data,
        float(cutoff),
        int(full_list),
        int("S" in quantities),
        int("d" in quantities),
        int("D" in quantities),
        ctypes.byref(lst),
        err,
        len(err),
    )
    try:
        if status != 0:
            raise RuntimeError(err.value.decode("utf8"))
        return _collect(lst, lst.length, quantities)
    finally:
        lib.vesin_oracle_free(ctypes.byref(lst))


class ReferenceCPU:
    """The reference CPU path behind its own C ABI; keeps one
    ``VesinNeighborList`` so repeated calls re-use its allocations (this is
    what the timed CPU baseline uses)."""

    def __init__(self):
        self._lib = _reference_lib()
        self._list = _VesinNeighborList()

    def __del__(self):
        try:
            self._lib.vesin_free(ctypes.byref(self._list))
        except Exception:
            pass

    def run(self, points, box, periodic, cutoff, full_list, quantities="ijSdD", n_threads=0, sorted=False, skin=0.0):
        """Only runs the calculation; returns the number of pairs. With
        ``skin > 0`` the reference re-uses the candidates it cached on this
        list (vesin/src/verlet.cpp:82-191) while the points have moved little."""
        points, box, periodic = _prepare(points, box, periodic)
        options = _VesinOptions()
        options.cutoff = float(cutoff)
        options.full = bool(full_list)
        options.sorted = bool(sorted)
        options.algorithm = 0
        options.n_threads = int(n_threads)
        options.return_shifts = "S" in quantities
        options.return_distances = "d" in quantities
        options.return_vectors = "D" in quantities
        options.skin = float(skin)
        error = ctypes.c_char_p()
        status = self._lib.vesin_neighbors(
            points.ctypes.data,
            points.shape[0],
            box.ctypes.data,
            periodic.ctypes.data,
            _VesinDevice(1, 0),
            options,
            ctypes.byref(self._list),
            ctypes.byref(error),
        )
        if status != 0:
            raise RuntimeError(error.value.decode("utf8"))
        return self._list.length

    def compute(self, points, box, periodic, cutoff, full_list, quantities="ijSdD", n_threads=0, sorted=False, skin=0.0):
        n = self.run(points, box, periodic, cutoff, full_list, quantities, n_threads, sorted, skin)
        return _collect(self._list, n, quantities)


def reference_neighbors(points, box, periodic, cutoff, full_list, quantities="ijSdD", n_threads=0, sorted=False):
    return ReferenceCPU().compute(points, box, periodic, cutoff, full_list, quantities, n_threads, sorted)


def canonical(result):
    """Sort a result dict lexicographically on (i, j, Sx, Sy, Sz)."""
    i = np.asarray(result["i"]).astype(np.int64)
    j = np.asarray(result["j"]).astype(np.int64)
    n = i.shape[0]
    S = np.asarray(result["S"]).astype(np.int64) if "S" in result else np.zeros((n, 3), np.int64)
    order = np.lexsort((S[:, 2], S[:, 1], S[:, 0], j, i))
    return {k: np.asarray(v)[order] for k, v in result.items()}


def assert_same(got, expected, rtol, what=""):
    """Bit-exact (i, j, S); d and D within `rtol` relative to the cutoff-scale
    magnitude of the expected value (absolute floor rtol * max|expected|)."""
    got = canonical(got)
    expected = canonical(expected)
    assert got["i"].shape == expected["i"].shape, f"{what}: {got['i'].shape[0]} pairs, expected {expected['i'].shape[0]}"
    assert np.array_equal(got["i"], expected["i"]), f"{what}: first indices differ"
    assert np.array_equal(got["j"], expected["j"]), f"{what}: second indices differ"
    if "S" in expected:
        assert np.array_equal(got["S"], expected["S"]), f"{what}: shifts differ"
    for key in ("d", "D"):
        if key in expected and expected[key].size:
            scale = np.max(np.abs(expected[key]))
            err = np.max(np.abs(got[key].astype(np.float64) - expected[key]))
            assert err <= rtol * scale, f"{what}: {key} differs by {err:.3e} (allowed {rtol * scale:.3e})"
