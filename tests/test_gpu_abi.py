"""GPU tests of the C ABI contract itself, through raw ctypes calls: argument
checks and their messages (vesin/src/vesin.cpp:51-105,
vesin/src/vesin_cuda.cpp:831-854), ownership and re-use
(vesin/tests/memory.cpp), concurrent calls from many host threads
(vesin/tests/cuda.cpp:147-156), the pairs-per-point limit
(python/vesin/tests/test_cupy.py:292-336)."""

import ctypes
import threading

import numpy as np
import pytest

import known_answers as KA
from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def abi():
    import torch

    import vesin_b200
    from vesin_b200 import _c_api

    assert torch.cuda.is_available()
    return vesin_b200.get_library(), _c_api, torch


def _options(api, cutoff, full=True, S=True, d=True, D=True, algorithm=0, n_threads=0, skin=0.0, sorted=False):
    options = api.VesinOptions()
    options.cutoff = cutoff
    options.full = full
    options.sorted = sorted
    options.algorithm = algorithm
    options.n_threads = n_threads
    options.return_shifts = S
    options.return_distances = d
    options.return_vectors = D
    options.skin = skin
    return options


def _call(lib, api, points, n, box, periodic, options, neighbors, device=None, error=None):
    if error is None:
        error = ctypes.c_char_p()
        error_ref = ctypes.byref(error)
    else:
        error_ref = error
    if device is None:
        device = api.VesinDevice(api.VesinCUDA, 0)
    status = lib.vesin_neighbors(points, n, box, periodic, device, options, neighbors, error_ref)
    message = error.value.decode() if isinstance(error, ctypes.c_char_p) and error.value else None
    return status, message


def _device_inputs(torch, points, box, periodic, device="cuda:0"):
    return (
        torch.tensor(np.asarray(points, dtype=np.float64).reshape(-1, 3), device=device),
        torch.tensor(np.asarray(box, dtype=np.float64), device=device),
        torch.tensor(np.asarray(periodic, dtype=bool), device=device),
    )


def _download(torch, api, neighbors, device="cuda:0"):
    from vesin_b200._neighbors import _view

    n = neighbors.length
    result = {}
    if n == 0:
        return {"i": np.zeros(0, np.int64), "j": np.zeros(0, np.int64)}
    pairs = _view(neighbors.pairs, (n, 2), "<u8", torch.device(device), neighbors).view(torch.int64).cpu().numpy()
    result["i"], result["j"] = pairs[:, 0].copy(), pairs[:, 1].copy()
    if neighbors.shifts:
        result["S"] = _view(neighbors.shifts, (n, 3), "<i4", torch.device(device), neighbors).cpu().numpy()
    if neighbors.distances:
        result["d"] = _view(neighbors.distances, (n,), "<f8", torch.device(device), neighbors).cpu().numpy()
    if neighbors.vectors:
        result["D"] = _view(neighbors.vectors, (n, 3), "<f8", torch.device(device), neighbors).cpu().numpy()
    return result


def test_argument_checks(abi):
    lib, api, torch = abi
    p, b, per = _device_inputs(torch, [[0.0, 0, 0], [1.0, 1, 1]], np.eye(3) * 4, [True] * 3)
    neighbors = api.VesinNeighborList()
    ref = ctypes.byref(neighbors)
    good = _options(api, 2.0)

    # NULL error_message: immediate failure, nothing else touched
    assert lib.vesin_neighbors(p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), api.VesinDevice(2, 0), good, ref, None) == 1

    cases = [
        ((None, 2, b.data_ptr(), per.data_ptr(), good, ref), "`points` can not be a NULL pointer"),
        ((p.data_ptr(), 2, None, per.data_ptr(), good, ref), "`cell` can not be a NULL pointer"),
        ((p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), good, None), "`neighbors` can not be a NULL pointer"),
        ((p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), _options(api, float("nan")), ref), "cutoff must be a finite, positive number"),
        ((p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), _options(api, -3.0), ref), "cutoff must be a finite, positive number"),
        ((p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), _options(api, 1e-7), ref), "cutoff is too small"),
        ((p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), _options(api, 2.0, n_threads=-1), ref), "n_threads must be zero or a positive integer"),
        ((p.data_ptr(), 2, b.data_ptr(), None, good, ref), "failed to resolve attributes for pointer: periodic"),
    ]
    for arguments, expected in cases:
        status, message = _call(lib, api, *arguments)
        assert status == 1 and message == expected, (message, expected)

    fresh = api.VesinNeighborList()
    status, message = _call(lib, api, p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), good, ctypes.byref(fresh), device=api.VesinDevice(0, 0))
    assert status == 1 and message == "got an unknown device type"
    status, message = _call(lib, api, p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), good, ctypes.byref(fresh), device=api.VesinDevice(1, 0))
    assert status == 1 and "CUDA" in message  # no CPU engine in this library
    lib.vesin_free(ctypes.byref(fresh))
    lib.vesin_free(ref)

    # host memory where device memory is required
    host = np.zeros((2, 3))
    neighbors = api.VesinNeighborList()
    status, message = _call(lib, api, host.ctypes.data, 2, b.data_ptr(), per.data_ptr(), good, ctypes.byref(neighbors))
    assert status == 1 and message == "`points` pointer is not allocated on a CUDA device"
    lib.vesin_free(ctypes.byref(neighbors))

    # a list that already belongs to another device kind
    neighbors = api.VesinNeighborList()
    neighbors.device = api.VesinDevice(1, 0)
    status, message = _call(lib, api, p.data_ptr(), 2, b.data_ptr(), per.data_ptr(), good, ctypes.byref(neighbors))
    assert status == 1 and message == "`neighbors` device and data `device` do not match, free the neighbors first"


def test_success_leaves_error_message_untouched_and_free_zeroes(abi):
    lib, api, torch = abi
    case = KA.CUDA_TRICLINIC
    p, b, per = _device_inputs(torch, case["points"], case["box"], case["periodic"])
    neighbors = api.VesinNeighborList()
    error = ctypes.c_char_p()
    status = lib.vesin_neighbors(
        p.data_ptr(), 3, b.data_ptr(), per.data_ptr(), api.VesinDevice(2, 0), _options(api, 3.0, full=False), ctypes.byref(neighbors), ctypes.byref(error)
    )
    assert status == 0 and error.value is None
    assert neighbors.length == 5
    assert neighbors.pairs and neighbors.shifts and neighbors.distances and neighbors.vectors
    assert neighbors.device.type == 2 and neighbors.device.device_id == 0
    got = O.canonical(_download(torch, api, neighbors))
    assert np.array_equal(got["d"], np.array(case["distances"]))
    assert np.array_equal(got["D"], np.array(case["vectors"]))
    lib.vesin_free(ctypes.byref(neighbors))
    assert bytes(neighbors) == bytes(ctypes.sizeof(neighbors))
    lib.vesin_free(ctypes.byref(neighbors))  # freeing a zeroed list is fine
    lib.vesin_free(None)


def test_zero_points_and_skin_message(abi):
    lib, api, torch = abi
    p, b, per = _device_inputs(torch, [[0.0, 0, 0]], np.eye(3) * 4, [True] * 3)
    neighbors = api.VesinNeighborList()
    status, message = _call(lib, api, p.data_ptr(), 0, b.data_ptr(), per.data_ptr(), _options(api, 2.0), ctypes.byref(neighbors))
    assert status == 0 and message is None and neighbors.length == 0
    # a bad skin sets the message but the call carries on (vesin/src/vesin.cpp:80-82)
    status, message = _call(lib, api, p.data_ptr(), 1, b.data_ptr(), per.data_ptr(), _options(api, 2.0, skin=-1.0), ctypes.byref(neighbors))
    assert status == 0 and message == "skin must be a finite, non-negative number"
    # a positive skin gives the plain list (rebuilt on every call)
    status, message = _call(lib, api, p.data_ptr(), 1, b.data_ptr(), per.data_ptr(), _options(api, 4.5, skin=1.0), ctypes.byref(neighbors))
    assert status == 0 and neighbors.length == 6
    lib.vesin_free(ctypes.byref(neighbors))


def test_pairs_per_point_limit(abi, monkeypatch):
    lib, api, torch = abi
    rng = np.random.default_rng(0)
    p, b, per = _device_inputs(torch, rng.random((100, 3)) * 3.0, np.eye(3) * 3.0, [True] * 3)
    neighbors = api.VesinNeighborList()
    options = _options(api, 4.0)
    monkeypatch.delenv("VESIN_CUDA_MAX_PAIRS_PER_POINT", raising=False)
    status, message = _call(lib, api, p.data_ptr(), 100, b.data_ptr(), per.data_ptr(), options, ctypes.byref(neighbors))
    assert status == 1
    assert message.startswith("The number of neighbor pairs exceeds the maximum capacity of 12800 (max_pairs_per_point=128; n_points=100).")
    assert "VESIN_CUDA_MAX_PAIRS_PER_POINT" in message
    monkeypatch.setenv("VESIN_CUDA_MAX_PAIRS_PER_POINT", "100000")
    status, message = _call(lib, api, p.data_ptr(), 100, b.data_ptr(), per.data_ptr(), options, ctypes.byref(neighbors))
    assert status == 0
    expected = O.restated_neighbors(p.cpu().numpy(), b.cpu().numpy(), [True] * 3, 4.0, True, "ijSdD")
    O.assert_same(_download(torch, api, neighbors), expected, 1e-12, "dense box")
    for bad in ("abc", "-5", "0", "12x"):
        monkeypatch.setenv("VESIN_CUDA_MAX_PAIRS_PER_POINT", bad)
        status, message = _call(lib, api, p.data_ptr(), 100, b.data_ptr(), per.data_ptr(), options, ctypes.byref(neighbors))
        assert status == 1 and message == f"Invalid value for VESIN_CUDA_MAX_PAIRS_PER_POINT: '{bad}'"
    lib.vesin_free(ctypes.byref(neighbors))


def test_many_host_threads(abi):
    """Ten host threads, each with its own list, round-robin over the devices."""
    lib, api, torch = abi
    n_devices = torch.cuda.device_count()
    case = KA.CUDA_TRICLINIC
    system = W.diamond(4, seed=21)
    expected_big = O.canonical(O.restated_neighbors(*system, 4.2, False, "ijSdD"))
    failures = []

    def worker(thread_id):
        try:
            device_id = thread_id % n_devices
            name = f"cuda:{device_id}"
            for points, box, periodic, cutoff, want in (
                (case["points"], case["box"], case["periodic"], 3.0, None),
                (system[0], system[1], system[2], 4.2, expected_big),
            ):
                p, b, per = _device_inputs(torch, points, box, periodic, name)
                torch.cuda.synchronize(device_id)
                neighbors = api.VesinNeighborList()
                for _ in range(5):
                    status, message = _call(
                        lib, api, p.data_ptr(), p.shape[0], b.data_ptr(), per.data_ptr(), _options(api, cutoff, full=False),
                        ctypes.byref(neighbors), device=api.VesinDevice(2, device_id),
                    )
                    assert status == 0, message
                got = O.canonical(_download(torch, api, neighbors, name))
                if want is None:
                    assert neighbors.length == 5
                    assert np.array_equal(got["S"], np.array(case["shifts"], dtype=np.int32))
                else:
                    for key in want:
                        assert np.array_equal(got[key], want[key]), key
                lib.vesin_free(ctypes.byref(neighbors))
        except Exception as e:  # noqa: BLE001
            failures.append((thread_id, repr(e)))

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(10)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures


def test_list_libraries(abi):
    lib, api, torch = abi
    count = ctypes.c_size_t(0)
    empty = (ctypes.c_char_p * 1)()
    lib.vesin_list_libraries(empty, ctypes.byref(count))
    total = count.value
    assert total > 3
    names = (ctypes.c_char_p * total)()
    count = ctypes.c_size_t(total)
    lib.vesin_list_libraries(names, ctypes.byref(count))
    paths = [n.decode() for n in names[: count.value] if n]
    assert any("libvesin" in path for path in paths)


def test_deterministic_content(abi):
    """Two builds of the same system give the same canonical list."""
    from gpu_utils import gpu_compute

    system = W.diamond(6, seed=3)
    a = O.canonical(gpu_compute(*system, 5.0, True))
    b = O.canonical(gpu_compute(*system, 5.0, True))
    for key in a:
        assert np.array_equal(a[key], b[key])
