"""CPU tests of the engine's host-side planning (vesin_b200/csrc/plan.cpp): the
box normalisation, the cell grid, the stencil reach, the fp32 screen band and
the slab window. plan.cpp is plain C++, so the test compiles it with g++ next
to a small C interface (tests/plan_check.cpp) and calls it through ctypes.

What is checked are the properties the kernels rely on (and that the
reference's own grid has, vesin/src/cpu_cell_list.cpp:277-351): a sphere of
radius `cutoff` around any point of a cell stays inside the stencil, the
number of cells never exceeds the number of points, rows of periodic
directions reach the kernels bit for bit.
"""

import ctypes
import os
import subprocess
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class PlanSummary(ctypes.Structure):
    _fields_ = [
        ("H", ctypes.c_double * 9),
        ("Hinv", ctypes.c_double * 9),
        ("t0", ctypes.c_double * 3),
        ("scale", ctypes.c_double * 3),
        ("cell_vec", ctypes.c_double * 9),
        ("face_dist", ctypes.c_double * 3),
        ("origin", ctypes.c_double * 3),
        ("zero_shift", ctypes.c_double * 3),
        ("cutoff2", ctypes.c_double),
        ("cutoff2_lo", ctypes.c_double),
        ("cutoff2_hi", ctypes.c_double),
        ("periodic", ctypes.c_int * 3),
        ("n_cells", ctypes.c_int * 3),
        ("n_search", ctypes.c_int * 3),
        ("n_cells_total", ctypes.c_int),
        ("pencil", ctypes.c_int),
        ("n_units", ctypes.c_int),
        ("window_axis", ctypes.c_int),
        ("n_owned", ctypes.c_int),
    ]


@pytest.fixture(scope="module")
def planner():
    build = tempfile.mkdtemp(prefix="plan_check_")
    library = os.path.join(build, "libplan_check.so")
    subprocess.run(
        [
            "g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-I", os.path.join(ROOT, "vesin_b200", "csrc"),
            os.path.join(ROOT, "tests", "plan_check.cpp"), os.path.join(ROOT, "vesin_b200", "csrc", "plan.cpp"), "-o", library,
        ],
        check=True,
    )
    lib = ctypes.CDLL(library)
    lib.plan_check_make.restype = ctypes.c_int

    def make(box, periodic, lower, upper, n_points, cutoff, full=True, sorted_=False, max_cells=1 << 27, slab=None, n_owned=0):
        box = np.ascontiguousarray(box, dtype=np.float64).reshape(9)
        periodic = np.ascontiguousarray(periodic, dtype=bool)
        lower = np.ascontiguousarray(lower, dtype=np.float64)
        upper = np.ascontiguousarray(upper, dtype=np.float64)
        out = PlanSummary()
        error = ctypes.create_string_buffer(512)
        axis, slab_lower, slab_upper = slab if slab is not None else (-1, 0.0, 1.0)
        status = lib.plan_check_make(
            box.ctypes.data_as(ctypes.c_void_p), periodic.ctypes.data_as(ctypes.c_void_p), lower.ctypes.data_as(ctypes.c_void_p),
            upper.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(n_points), ctypes.c_double(cutoff), int(full), int(sorted_),
            ctypes.c_size_t(max_cells), int(axis), ctypes.c_double(slab_lower), ctypes.c_double(slab_upper), ctypes.c_size_t(n_owned),
            ctypes.byref(out), error, ctypes.c_size_t(512),
        )
        if status != 0:
            raise RuntimeError(error.value.decode())
        return out

    return make


def _random_box(rng, scale):
    box = rng.normal(0.0, 1.0, (3, 3)) * 0.3 + np.eye(3)
    return box * scale


def test_stencil_covers_the_cutoff(planner):
    rng = np.random.default_rng(5)
    for trial in range(200):
        scale = float(rng.choice([3.0, 12.0, 40.0, 150.0]))
        box = _random_box(rng, scale)
        periodic = rng.random(3) < 0.7
        cutoff = float(rng.uniform(0.8, 9.0))
        n_points = int(rng.choice([1, 7, 300, 40000]))
        lower = rng.normal(0, scale, 3)
        upper = lower + rng.uniform(0.0, 2.0 * scale, 3)
        plan = planner(box, periodic, lower, upper, n_points, cutoff)
        H = np.array(plan.H).reshape(3, 3)
        Hinv = np.array(plan.Hinv).reshape(3, 3)
        assert np.allclose(H @ Hinv, np.eye(3), atol=1e-9)
        for k in range(3):
            if periodic[k]:
                # rows of periodic directions enter the distance arithmetic: bit for bit the caller's
                assert np.array_equal(H[k], box[k])
            n_cells, n_search = plan.n_cells[k], plan.n_search[k]
            assert n_cells >= 1
            width = plan.face_dist[k] / n_cells  # distance between the two faces of a cell
            if periodic[k] or n_cells > 1:
                reach = n_search * width
                if periodic[k] or n_search < n_cells - 1:
                    assert reach >= cutoff, (trial, k, reach, cutoff)
            if not periodic[k] and n_cells == 1:
                assert n_search == 0
        assert plan.n_cells_total == plan.n_cells[0] * plan.n_cells[1] * plan.n_cells[2]
        assert plan.n_cells_total <= max(n_points, 1)
        assert 1 <= plan.pencil <= min(8, plan.n_cells[0])
        pencils = -(-plan.n_cells[0] // plan.pencil)
        assert plan.n_units == pencils * plan.n_cells[1] * plan.n_cells[2]
        # the fp32 screen brackets the exact bound
        assert plan.cutoff2 == cutoff * cutoff
        assert plan.cutoff2_lo < plan.cutoff2 < plan.cutoff2_hi
        assert all(z == 0.0 for z in plan.zero_shift)


def test_non_periodic_window_holds_the_points(planner):
    rng = np.random.default_rng(11)
    for _ in range(100):
        box = _random_box(rng, 20.0)
        periodic = np.array([True, False, bool(rng.integers(2))])
        lower = rng.normal(0, 30.0, 3)
        upper = lower + rng.uniform(0.1, 60.0, 3)
        plan = planner(box, periodic, lower, upper, 500, 3.0)
        Hinv = np.array(plan.Hinv).reshape(3, 3)
        corners = np.array([[x, y, z] for x in (lower[0], upper[0]) for y in (lower[1], upper[1]) for z in (lower[2], upper[2])])
        for k in range(3):
            if periodic[k]:
                continue
            t = corners @ Hinv[:, k]
            cell = np.floor((t - plan.t0[k]) * plan.scale[k])
            assert cell.min() >= 0 and cell.max() <= plan.n_cells[k] - 1


def test_errors_of_the_reference(planner):
    singular = np.array([[1.0, 0, 0], [2.0, 0, 0], [0, 0, 1.0]])
    with pytest.raises(RuntimeError, match="the box matrix is not invertible"):
        planner(singular, [True, True, True], [0, 0, 0], [1, 1, 1], 10, 2.0)
    # the same rows are harmless along non-periodic directions (vesin/src/types.hpp:41-72)
    plan = planner(singular, [True, False, False], [0, 0, 0], [1, 1, 1], 10, 2.0)
    assert np.allclose(np.array(plan.H).reshape(3, 3) @ np.array(plan.Hinv).reshape(3, 3), np.eye(3))
    plan = planner(np.zeros((3, 3)), [False, False, False], [-4, -4, -4], [4, 4, 4], 100, 2.0)
    assert np.array_equal(np.array(plan.H).reshape(3, 3), np.eye(3))


def test_cutoff_hundreds_of_times_the_box_is_refused(planner):
    """A stencil beyond 2^20 cells (a collapsed box, a wrong unit) is an error,
    not a kernel that walks billions of images; large but sane stencils pass."""
    plan = planner(np.eye(3) * 0.5, [True, True, True], [0, 0, 0], [0.4, 0.4, 0.4], 3, 0.6)
    assert plan.n_search[0] == 2
    plan = planner(np.eye(3), [True, True, True], [0, 0, 0], [1, 1, 1], 4, 40.0)  # 81^3 = 531 441 cells
    assert plan.n_search[0] >= 40
    with pytest.raises(RuntimeError, match="the cutoff is too large for this box"):
        planner(np.eye(3), [True, True, True], [0, 0, 0], [1, 1, 1], 4, 60.0)
    # non-periodic directions have no images: the same numbers are fine
    planner(np.eye(3), [False, False, False], [0, 0, 0], [1, 1, 1], 4, 60.0)


def test_huge_empty_box_does_not_allocate_by_volume(planner):
    plan = planner(np.eye(3) * 1.0e6, [True, True, True], [0, 0, 0], [10, 10, 10], 64, 3.0)
    assert plan.n_cells_total <= 64


def test_slab_window(planner):
    box = np.diag([40.0, 50.0, 120.0])
    periodic = [True, True, True]
    plan = planner(box, periodic, [0, 0, 0], [40, 50, 120], 100000, 5.9, slab=(2, 0.25, 0.5), n_owned=80000)
    layers = int(np.floor(0.25 * 120.0 / 5.9))
    assert plan.window_axis == 2 and plan.n_owned == 80000
    assert plan.n_cells[2] == layers + 2 and plan.n_search[2] == 1
    width = 0.25 / layers
    assert np.isclose(plan.t0[2], 0.25 - width) and np.isclose(plan.scale[2], 1.0 / width)
    assert width * 120.0 >= 5.9  # a layer is at least a cutoff thick
    with pytest.raises(RuntimeError, match="thinner than the cutoff"):
        planner(box, periodic, [0, 0, 0], [40, 50, 120], 1000, 6.0, slab=(2, 0.0, 0.04), n_owned=10)
    with pytest.raises(RuntimeError, match="longer than the box"):
        planner(np.diag([40.0, 50.0, 20.0]), periodic, [0, 0, 0], [40, 50, 20], 1000, 6.0, slab=(2, 0.0, 0.5), n_owned=10)
