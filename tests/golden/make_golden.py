"""
Generates tests/golden/reference_cpu.npz from the UNMODIFIED reference CPU path
(oracle/_ref/libvesin_ref.so, built by oracle/Makefile from the reference
sources). Run it where the reference tree is available:

    python tests/golden/make_golden.py [/path/to/reference]

Inputs:
  * the seven extended-XYZ fixtures of the reference's Python tests
    (python/vesin/tests/data/*.xyz; systems without a cell get a zero box and
    no periodicity, as python/vesin/tests/_utils.py:197-206 does through ASE),
  * the generated small systems of vesin_b200.workloads, plain and under a
    seeded rotation / rotation + translation,
  * random points in a skewed box for all eight periodicity combinations
    (the shape of python/vesin/tests/test_numpy.py:231-269),
  * the 1e7-wide box case (test_numpy.py:328-338 shape, seeded here).

For each (system, cutoff, full/half) the file stores the inputs, the number of
pairs, a SHA-256 over the canonically sorted (i, j, S) int64 table, sum(d) and
sum(|D|); cases with at most MAX_FULL pairs also store the whole canonical
i, j, S, d, D arrays. The file is read by the CPU tests (to pin the C
restatement) and by the GPU tests (to pin the CUDA engine).
"""

import hashlib
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402
from vesin_b200 import workloads as W  # noqa: E402

MAX_FULL = 500
CUTOFFS = [3.0, 5.0, 7.0, 10.0]


def read_extxyz(path):
    """Minimal extended-XYZ reader: positions from columns 1-3 after the
    species, Lattice="..." (rows) and pbc="..." from the comment line."""
    with open(path) as fd:
        lines = fd.read().splitlines()
    n = int(lines[0])
    comment = lines[1]
    lattice = re.search(r'Lattice="([^"]*)"', comment)
    pbc = re.search(r'pbc="([^"]*)"', comment)
    if lattice:
        box = np.array([float(x) for x in lattice.group(1).split()]).reshape(3, 3)
        periodic = np.array([True, True, True])
    else:
        box = np.zeros((3, 3))
        periodic = np.array([False, False, False])
    if pbc:
        periodic = np.array([tok.upper().startswith("T") for tok in pbc.group(1).split()])
    points = np.array([[float(x) for x in line.split()[1:4]] for line in lines[2 : 2 + n]])
    return points, box, periodic


def digest(result):
    c = O.canonical(result)
    table = np.concatenate([c["i"][:, None], c["j"][:, None], c["S"].astype(np.int64)], axis=1)
    return c, hashlib.sha256(np.ascontiguousarray(table).tobytes()).hexdigest()


def main():
    if len(sys.argv) > 1:
        reference_root = sys.argv[1]
    elif os.environ.get("VESIN_REFERENCE_ROOT"):
        reference_root = os.environ["VESIN_REFERENCE_ROOT"]
    else:  # a checkout named "reference" beside this repository
        reference_root = os.path.join(os.path.dirname(ROOT), "reference")
    data_dir = os.path.join(reference_root, "python", "vesin", "tests", "data")
    O.build()
    assert O.reference_available(), "oracle/_ref/libvesin_ref.so is missing"

    systems = {}
    for name in ["water", "diamond", "naphthalene", "carbon", "slab", "Cd2I4O12", "rotated_box"]:
        systems["xyz_" + name] = read_extxyz(os.path.join(data_dir, name + ".xyz"))
    for name, make in W.SMALL_SYSTEMS.items():
        systems[name] = make()
    base = dict(systems)
    for k, (name, system) in enumerate(sorted(base.items())):
        systems[name + "@rot"] = W.transformed(system, 100 + k, translate=False)
        systems[name + "@rot+trans"] = W.transformed(system, 200 + k, translate=True)

    cases = []  # (case name, system, cutoff, full)
    for name, system in systems.items():
        for cutoff in CUTOFFS:
            for full in (False, True):
                cases.append((f"{name}|{cutoff}|{int(full)}", system, cutoff, full))
    for bits in range(8):
        periodic = [(bits >> 2) & 1, (bits >> 1) & 1, bits & 1]
        system = W.skewed_random(periodic, seed=bits)
        cases.append((f"skewed_{bits:03b}|0.35|1", system, 0.35, True))
        cases.append((f"skewed_{bits:03b}|0.35|0", system, 0.35, False))
    rng = np.random.default_rng(34)
    gigantic = (rng.normal(size=(3000, 3)) * 100.0, np.eye(3) * 1e7, np.array([True] * 3))
    cases.append(("gigantic|8.0|1", gigantic, 8.0, True))

    out = {}
    names = []
    cpu = O.ReferenceCPU()
    for name, (points, box, periodic), cutoff, full in cases:
        res = cpu.compute(points, box, periodic, cutoff, full, "ijSdD", n_threads=1)
        c, sha = digest(res)
        names.append(name)
        out[f"{name}/points"] = points
        out[f"{name}/box"] = box
        out[f"{name}/periodic"] = np.asarray(periodic, dtype=bool)
        out[f"{name}/n_pairs"] = np.int64(len(c["i"]))
        out[f"{name}/sha256"] = np.array(sha)
        out[f"{name}/sum_d"] = np.float64(c["d"].sum())
        out[f"{name}/sum_absD"] = np.float64(np.abs(c["D"]).sum())
        if len(c["i"]) <= MAX_FULL:
            for key in "ijSdD":
                out[f"{name}/{key}"] = c[key]
    out["names"] = np.array(names)
    path = os.path.join(HERE, "reference_cpu.npz")
    np.savez_compressed(path, **out)
    print(f"{len(names)} cases -> {path} ({os.path.getsize(path) / 1e6:.2f} MB)")


if __name__ == "__main__":
    main()
