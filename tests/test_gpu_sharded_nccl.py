"""The sharded build over real NCCL: one process per GPU, every rank calls
``ShardedNeighborList.compute`` (library: packing kernel, ncclSend / ncclRecv,
local build) on the points it owns; the union of the ranks' lists must be the
CPU oracle's list of the whole system, (i, j, S) bit for bit and d, D
bit-identical. Needs at least two GPUs; skipped otherwise (the same code with
the test as transport runs on one GPU in tests/test_gpu_slab.py)."""

import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from oracle import oracle as O
from vesin_b200 import workloads as W

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_SCRIPT = """
import os, sys
sys.path.insert(0, {root!r})
import numpy as np
import torch
import torch.distributed as dist
import vesin_b200
from vesin_b200 import workloads as W
from vesin_b200._sharded import owner_of, slab_geometry

local_rank = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local_rank)
device = torch.device("cuda", local_rank)
dist.init_process_group("nccl", device_id=device)
rank, world = dist.get_rank(), dist.get_world_size()
out = {out!r}

cases = [
    ("liquid_full", W.liquid(60000, seed=31), 6.0, True, np.float64),
    ("liquid_half", W.liquid(60000, seed=32), 6.0, False, np.float64),
    ("liquid_half_f32", W.liquid(60000, seed=33), 6.0, False, np.float32),
]
for name, (points, box, periodic), cutoff, full, dtype in cases:
    calculator = vesin_b200.ShardedNeighborList(cutoff=cutoff, full_list=full)
    # three builds on the same list: the second and third re-use what the first left
    # (output arrays, message buffers) on points that have moved
    for step in range(3):
        moved = (points + 0.05 * step * np.sin(points[:, ::-1])).astype(dtype)
        reference_points = moved.astype(np.float64)
        reference_box = box.astype(dtype).astype(np.float64)
        axis, _, _ = slab_geometry(reference_box, periodic, cutoff)
        mine = np.nonzero(owner_of(reference_points, reference_box, axis, world) == rank)[0]
        i, j, S, d, D = calculator.compute(
            torch.from_numpy(moved[mine]).to(device), torch.from_numpy(mine).to(device), box.astype(dtype), periodic, "ijSdD"
        )
        np.savez(
            os.path.join(out, f"{{name}}_step{{step}}_rank{{rank}}.npz"),
            i=i.cpu().numpy(), j=j.cpu().numpy(), S=S.cpu().numpy(), d=d.cpu().numpy(), D=D.cpu().numpy(),
            checksum=np.array(calculator.checksum(), dtype=np.uint64), n_owned=len(mine),
        )
    calculator.close()

# A rank that fails inside its build still takes part in the exchange: the last rank asks
# for a sorted list (refused by the slab build before anything is queued), the others get
# their lists as usual; the next build works on every rank.
points, box, periodic = W.liquid(60000, seed=34)
axis, _, _ = slab_geometry(box, periodic, 6.0)
mine = np.nonzero(owner_of(points, box, axis, world) == rank)[0]
calculator = vesin_b200.ShardedNeighborList(cutoff=6.0, full_list=True)
arguments = (torch.from_numpy(points[mine]).to(device), torch.from_numpy(mine).to(device), box, periodic, "ijSdD")
calculator.compute(*arguments)
plain_options = calculator._options
if rank == world - 1:
    def sorted_options(quantities):
        options = plain_options(quantities)
        options.sorted = True
        return options
    calculator._options = sorted_options
    try:
        calculator.compute(*arguments)
    except RuntimeError as e:
        assert "sorted" in str(e), str(e)
    else:
        raise AssertionError("a sorted slab build has to be refused")
    calculator._options = plain_options
else:
    calculator.compute(*arguments)
i, j, S, d, D = calculator.compute(*arguments)
np.savez(
    os.path.join(out, f"after_failure_rank{{rank}}.npz"),
    i=i.cpu().numpy(), j=j.cpu().numpy(), S=S.cpu().numpy(), d=d.cpu().numpy(), D=D.cpu().numpy(),
)
calculator.close()
dist.barrier()
dist.destroy_process_group()
"""


def _run(world, tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(RANK_SCRIPT.format(root=ROOT, out=str(tmp_path))))
    environment = dict(os.environ)
    environment["NCCL_NVLS_ENABLE"] = "0"
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
         "--master-port", str(29750 + world), str(script)],
        capture_output=True, text=True, timeout=900, env=environment,
    )
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_lists_over_nccl(world, tmp_path):
    import torch

    from vesin_b200._sharded import checksum_of_arrays

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, tmp_path)
    cases = [
        ("liquid_full", W.liquid(60000, seed=31), 6.0, True, np.float64),
        ("liquid_half", W.liquid(60000, seed=32), 6.0, False, np.float64),
        ("liquid_half_f32", W.liquid(60000, seed=33), 6.0, False, np.float32),
    ]
    for name, (points, box, periodic), cutoff, full, dtype in cases:
        for step in range(3):
            moved = (points + 0.05 * step * np.sin(points[:, ::-1])).astype(dtype).astype(np.float64)
            box_used = box.astype(dtype).astype(np.float64)
            parts = [np.load(tmp_path / f"{name}_step{step}_rank{rank}.npz") for rank in range(world)]
            got = {key: np.concatenate([part[key] for part in parts]) for key in "ijSdD"}
            expected = O.restated_neighbors(moved, box_used, periodic, cutoff, full, "ijSdD")
            got, expected = O.canonical(got), O.canonical(expected)
            label = f"{name} step {step} on {world} ranks"
            assert len(got["i"]) == len(expected["i"]), label
            for key in "ijS":
                assert np.array_equal(got[key], expected[key]), label
            assert np.array_equal(got["d"], expected["d"].astype(dtype)), label
            assert np.array_equal(got["D"], expected["D"].astype(dtype)), label
            total = [int(sum(int(part["checksum"][k]) for part in parts) % (1 << 64)) for k in range(3)]
            total.append(int(sum(int(part["checksum"][3]) for part in parts)))
            assert tuple(total) == checksum_of_arrays(expected["i"], expected["j"], expected["S"], expected["d"].astype(dtype)), label
    # the build after one rank's refused call
    points, box, periodic = W.liquid(60000, seed=34)
    parts = [np.load(tmp_path / f"after_failure_rank{rank}.npz") for rank in range(world)]
    got = O.canonical({key: np.concatenate([part[key] for part in parts]) for key in "ijSdD"})
    expected = O.canonical(O.restated_neighbors(points, box, periodic, 6.0, True, "ijSdD"))
    for key in "ijSdD":
        assert np.array_equal(got[key], expected[key]), f"after a refused call: {key}"
