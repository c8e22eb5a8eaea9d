"""CPU tests of the multi-GPU host logic: splitting a batch of systems over
ranks (no communication on the data path). The two-rank case runs as two
gloo processes, the way the GPU ranks would."""

import os
import subprocess
import sys
import textwrap

import numpy as np

from vesin_b200 import split_batch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_split_covers_every_system_once():
    rng = np.random.default_rng(0)
    for n_systems in (0, 1, 2, 7, 1000):
        counts = rng.integers(0, 65, n_systems)
        offsets = np.concatenate([[0], np.cumsum(counts)])
        for world in (1, 2, 3, 4, 8):
            chunks = split_batch(offsets, world)
            assert len(chunks) == world
            assert chunks[0][0] == 0 and chunks[-1][1] == n_systems
            for (a, b), (c, d) in zip(chunks[:-1], chunks[1:]):
                assert a <= b == c <= d
            if n_systems >= 100:
                sizes = [offsets[b] - offsets[a] for a, b in chunks]
                assert max(sizes) - min(sizes) <= 2 * 64, "chunks are balanced by points to within two systems"


def test_two_ranks_over_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(
        textwrap.dedent(
            f"""
            import sys
            sys.path.insert(0, {ROOT!r})
            import numpy as np
            import torch
            import torch.distributed as dist
            from vesin_b200 import split_batch

            dist.init_process_group("gloo")
            rank, world = dist.get_rank(), dist.get_world_size()
            counts = np.random.default_rng(3).integers(16, 65, 501)
            offsets = np.concatenate([[0], np.cumsum(counts)])
            first, last = split_batch(offsets, world)[rank]
            mine = torch.zeros(len(counts), dtype=torch.int64)
            mine[first:last] = 1
            dist.all_reduce(mine)
            assert bool((mine == 1).all()), "every system is built by exactly one rank"
            points = torch.tensor([int(offsets[last] - offsets[first])])
            gathered = [torch.zeros_like(points) for _ in range(world)]
            dist.all_gather(gathered, points)
            assert sum(int(g) for g in gathered) == int(offsets[-1])
            dist.destroy_process_group()
            """
        )
    )
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29731", str(script)],
        capture_output=True, text=True, timeout=240,
    )
    assert result.returncode == 0, result.stdout + result.stderr


def test_halo_exchange_over_gloo(tmp_path):
    """The halo exchange on CPU tensors with 2 and 3 gloo ranks: every rank must
    end up with exactly the halo the single-process reference selects."""
    script = tmp_path / "halo.py"
    script.write_text(
        textwrap.dedent(
            f"""
            import sys
            sys.path.insert(0, {ROOT!r})
            import numpy as np
            import torch
            import torch.distributed as dist
            from vesin_b200 import workloads
            from vesin_b200._sharded import choose_axis, exchange_halo, local_set, owner_of

            dist.init_process_group("gloo")
            rank, world = dist.get_rank(), dist.get_world_size()
            points, box, periodic = workloads.liquid(6000, seed=21)
            cutoff = 6.0
            axis = choose_axis(box, periodic)
            owner = owner_of(points, box, axis, world)
            mine = np.nonzero(owner == rank)[0]
            halo_points, halo_index = exchange_halo(
                torch.from_numpy(points[mine]), torch.from_numpy(mine), box, axis, cutoff
            )
            owned, halo = local_set(points, box, periodic, cutoff, rank, world)
            assert np.array_equal(owned, mine)
            assert np.array_equal(halo_index.numpy(), halo), (rank, len(halo_index), len(halo))
            assert np.array_equal(halo_points.numpy(), points[halo])
            dist.destroy_process_group()
            """
        )
    )
    for world, port in ((2, 29741), (3, 29742)):
        result = subprocess.run(
            [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
             "--master-port", str(port), str(script)],
            capture_output=True, text=True, timeout=300,
        )
        assert result.returncode == 0, result.stdout[-2000:] + result.stderr[-2000:]
