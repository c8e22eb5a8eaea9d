"""
Seeded synthetic systems used by the tests and the benchmark.

These stand in for the shapes the reference benchmarks on (diamond supercells,
benchmarks/benchmark.py:189,206; a random liquid at fixed density,
python/benchmarks/bench-cuda-algorithms.py:20-26); no external data set is
involved. Every generator returns ``(points, box, periodic)`` as numpy arrays
(float64 points (N, 3), float64 box (3, 3) with one cell vector per row, bool
periodic (3,)).
"""

import numpy as np

DIAMOND_A = 3.567

_DIAMOND_BASIS = np.array(
    [
        [0.0, 0.0, 0.0],
        [0.0, 0.5, 0.5],
        [0.5, 0.0, 0.5],
        [0.5, 0.5, 0.0],
        [0.25, 0.25, 0.25],
        [0.25, 0.75, 0.75],
        [0.75, 0.25, 0.75],
        [0.75, 0.75, 0.25],
    ]
)


def diamond(n, seed=0, sigma=0.05, a=DIAMOND_A):
    """Diamond-carbon supercell: the 8-atom cubic cell replicated n x n x n,
    atom index ((ix*n + iy)*n + iz)*8 + b, positions jittered by a seeded
    Gaussian and NOT wrapped back (some atoms lie just outside the box).
    n=5 is the 1000-atom case, n=40 the 512000-atom case."""
    grid = np.arange(n, dtype=np.float64)
    cells = np.stack(np.meshgrid(grid, grid, grid, indexing="ij"), axis=-1).reshape(-1, 1, 3)
    points = ((cells + _DIAMOND_BASIS[None, :, :]) * a).reshape(-1, 3)
    points = points + np.random.default_rng(seed).normal(0.0, sigma, points.shape)
    box = np.eye(3) * (n * a)
    return np.ascontiguousarray(points), box, np.array([True, True, True])


def small_triclinic(n_atoms=64, seed=3):
    """Uniform-random atoms in a seeded triclinic cell with lengths in [6, 8]
    and angles in [60, 120] degrees (standard orientation: a along x, b in the
    xy plane). With a 9.0 cutoff several periodic images contribute per axis."""
    rng = np.random.default_rng(seed)
    while True:
        la, lb, lc = rng.uniform(6.0, 8.0, 3)
        alpha, beta, gamma = np.deg2rad(rng.uniform(60.0, 120.0, 3))
        cx = lc * np.cos(beta)
        cy = lc * (np.cos(alpha) - np.cos(beta) * np.cos(gamma)) / np.sin(gamma)
        cz2 = lc * lc - cx * cx - cy * cy
        if cz2 > 1e-6:
            break
    box = np.array(
        [
            [la, 0.0, 0.0],
            [lb * np.cos(gamma), lb * np.sin(gamma), 0.0],
            [cx, cy, np.sqrt(cz2)],
        ]
    )
    points = rng.random((n_atoms, 3)) @ box
    return np.ascontiguousarray(points), box, np.array([True, True, True])


def molecule_batch(n_systems=16384, seed=4, radius=6.0, min_sep=1.0, n_min=16, n_max=64):
    """Independent non-periodic molecules: seeded atom counts in [n_min, n_max],
    atoms drawn uniformly in a sphere with a minimum separation (dart throwing),
    stored as float32 values. Returns (points (sum n, 3) float64 holding
    float32-representable values, offsets (n_systems + 1,) int64)."""
    rng = np.random.default_rng(seed)
    counts = rng.integers(n_min, n_max + 1, n_systems)
    offsets = np.zeros(n_systems + 1, dtype=np.int64)
    np.cumsum(counts, out=offsets[1:])
    points = np.empty((offsets[-1], 3), dtype=np.float64)
    min_sep2 = min_sep * min_sep
    for k in range(n_systems):
        n = counts[k]
        accepted = np.empty((n, 3))
        filled = 0
        while filled < n:
            cand = rng.uniform(-radius, radius, (4 * n, 3))
            cand = cand[np.einsum("ij,ij->i", cand, cand) <= radius * radius]
            for c in cand:
                if filled == n:
                    break
                if filled:
                    diff = accepted[:filled] - c
                    if np.min(np.einsum("ij,ij->i", diff, diff)) < min_sep2:
                        continue
                accepted[filled] = c
                filled += 1
        points[offsets[k] : offsets[k + 1]] = accepted.astype(np.float32).astype(np.float64)
    return points, offsets


def liquid(n_atoms, seed=5, density=0.0334):
    """Uniform-random atoms in a periodic cube at Lennard-Jones-liquid number
    density, float32-representable coordinates. n_atoms = 16_777_216 is the
    slab-decomposed case."""
    length = float(np.float32((n_atoms / density) ** (1.0 / 3.0)))
    rng = np.random.default_rng(seed)
    points = np.empty((n_atoms, 3), dtype=np.float64)
    step = 1 << 22
    for start in range(0, n_atoms, step):
        stop = min(n_atoms, start + step)
        chunk = (rng.random((stop - start, 3), dtype=np.float32) * np.float32(length)).astype(np.float64)
        points[start:stop] = chunk
    box = np.eye(3) * length
    return points, box, np.array([True, True, True])


# ---------------------------------------------------------------------------
# Small systems for the parity matrix. They re-create the *kinds* of system the
# reference tests use (python/vesin/tests/_utils.py:114-222): a 1-D periodic
# chain, a 2-D periodic sheet, a 3-D crystal with large jitter, an isolated
# cluster, a flat 2-D periodic cell with a zero third vector, random points in
# a skewed box with every periodicity combination.
# ---------------------------------------------------------------------------


def chain_1d():
    spacing = 1.54
    points = np.zeros((8, 3))
    points[:, 0] = np.arange(8) * spacing
    return points, np.diag([8 * spacing, 18.0, 18.0]), np.array([True, False, False])


def sheet_2d():
    a1 = np.array([2.46, 0.0, 0.0])
    a2 = np.array([1.23, 2.13042249, 0.0])
    basis = [np.zeros(3), np.array([1.23, 0.71014083, 0.0])]
    points = [i * a1 + j * a2 + b for i in range(4) for j in range(4) for b in basis]
    box = np.array([4 * a1, 4 * a2, [0.0, 0.0, 18.0]])
    return np.array(points), box, np.array([True, True, False])


def jittered_crystal(seed=1234):
    points, box, periodic = diamond(2, seed=seed, sigma=1.0, a=3.5607451090903233)
    return points, box, periodic


def cluster(seed=7, n=40):
    rng = np.random.default_rng(seed)
    points = rng.normal(0.0, 2.5, (n, 3)) + np.array([11.0, -3.0, 4.0])
    return points, np.zeros((3, 3)), np.array([False, False, False])


def flat_cell():
    points = np.array([[0.0, 2.5, 0.0], [2.0, 0.0, 0.0]])
    return points, np.diag([4.0, 4.5, 0.0]), np.array([True, True, False])


def skewed_random(periodic, seed=0, n=100):
    rng = np.random.default_rng(seed)
    box = np.eye(3)[[2, 0, 1]] + 0.1 * rng.normal(size=(3, 3))
    points = rng.random((n, 3))
    return points, box, np.array(periodic, dtype=bool)


def random_rotation(seed):
    """Seeded proper or improper rotation matrix."""
    rng = np.random.default_rng(seed)
    q, _ = np.linalg.qr(rng.normal(size=(3, 3)))
    if np.linalg.det(q) < 0:
        q[:, 0] *= -1
    if rng.integers(2):
        q = -q
    return q


def transformed(system, seed, translate):
    points, box, periodic = system
    q = random_rotation(seed)
    points = points @ q.T
    if translate:
        points = points + np.random.default_rng(seed + 1).uniform(-100.0, 100.0, 3)
    return np.ascontiguousarray(points), np.ascontiguousarray(box @ q.T), periodic


SMALL_SYSTEMS = {
    "chain_1d": chain_1d,
    "sheet_2d": sheet_2d,
    "jittered_crystal": jittered_crystal,
    "cluster": cluster,
    "flat_cell": flat_cell,
}
