"""CPU tests: the shared library loads, exports every symbol the headers
declare, and its argument checks (which need no GPU) behave like the
reference's (vesin/src/vesin.cpp:51-105). No compute call is made here."""

import ctypes
import os
import re

import pytest

import vesin_b200
from vesin_b200 import _c_api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(vesin_b200.LIBRARY_PATH):
        vesin_b200.build_library()
    return vesin_b200.get_library()


def _declared_symbols():
    names = set()
    for header in ("vesin.h", "vesin_b200.h"):
        with open(os.path.join(ROOT, "include", header)) as fd:
            text = fd.read()
        names.update(re.findall(r"VESIN_API\s+[\w\s\*]*?\b(vesin\w+)\s*\(", text))
    return names


def test_exports_every_declared_symbol(lib):
    declared = _declared_symbols()
    assert {"vesin_neighbors", "vesin_free", "vesin_list_libraries"} <= declared
    assert declared == set(_c_api.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None


def test_struct_layouts():
    assert ctypes.sizeof(_c_api.VesinOptions) == 32
    assert _c_api.VesinOptions.algorithm.offset == 12
    assert _c_api.VesinOptions.return_shifts.offset == 20
    assert _c_api.VesinOptions.skin.offset == 24
    assert ctypes.sizeof(_c_api.VesinDevice) == 8
    assert ctypes.sizeof(_c_api.VesinNeighborList) == 56
    assert _c_api.VesinNeighborList.pairs.offset == 16
    assert _c_api.VesinNeighborList.opaque.offset == 48


def test_argument_checks_without_gpu(lib):
    neighbors = _c_api.VesinNeighborList()
    options = _c_api.VesinOptions()
    options.cutoff = 2.0
    error = ctypes.c_char_p()
    device = _c_api.VesinDevice(_c_api.VesinCUDA, 0)
    fake = ctypes.c_void_p(16)  # never dereferenced by the checks below

    def call(points, box, opts, lst=ctypes.byref(neighbors), dev=device):
        error.value = None
        status = lib.vesin_neighbors(points, 1, box, fake, dev, opts, lst, ctypes.byref(error))
        return status, (error.value.decode() if error.value else None)

    assert lib.vesin_neighbors(fake, 1, fake, fake, device, options, ctypes.byref(neighbors), None) == 1
    assert call(None, fake, options) == (1, "`points` can not be a NULL pointer")
    assert call(fake, None, options) == (1, "`cell` can not be a NULL pointer")
    assert call(fake, fake, options, lst=None) == (1, "`neighbors` can not be a NULL pointer")
    options.cutoff = 0.0
    assert call(fake, fake, options) == (1, "cutoff must be a finite, positive number")
    options.cutoff = 5e-7
    assert call(fake, fake, options) == (1, "cutoff is too small")
    options.cutoff = 2.0
    options.n_threads = -2
    assert call(fake, fake, options) == (1, "n_threads must be zero or a positive integer")
    options.n_threads = 0
    assert call(fake, fake, options, dev=_c_api.VesinDevice(0, 0)) == (1, "got an unknown device type")
    lib.vesin_free(ctypes.byref(neighbors))
    assert bytes(neighbors) == bytes(56)


def test_calculator_fails_loudly_without_gpu():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    calculator = vesin_b200.NeighborList(cutoff=3.0, full_list=True)
    with pytest.raises(RuntimeError, match="needs a CUDA device"):
        calculator.compute([[0.0, 0.0, 0.0]], [[1.0, 0, 0], [0, 1.0, 0], [0, 0, 1.0]], True)
    with pytest.raises(ValueError, match="Unknown algorithm"):
        vesin_b200.NeighborList(cutoff=3.0, full_list=True, algorithm="magic")
    with pytest.raises(ValueError, match="n_threads must be zero or a positive integer"):
        vesin_b200.NeighborList(cutoff=3.0, full_list=True, n_threads=-1)
