"""Batch sharding over ranks, exercised with two gloo processes on the CPU: the partition covers every pair once, the
per-shard results equal the slices of the single-process result bit for bit (no cross-sample arithmetic exists), and the
timing reduction is the maximum over ranks."""

import hashlib
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

from flashim_b200.sharding import Ranks, shard_pairs

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("total,world", [(64, 1), (64, 2), (64, 8), (7, 4), (3, 8), (0, 2)])
def test_partition_is_contiguous_and_complete(total, world):
    covered = []
    for rank in range(world):
        first, count = shard_pairs(total, rank, world)
        covered += list(range(first, first + count))
    assert covered == list(range(total))
    sizes = [shard_pairs(total, r, world)[1] for r in range(world)]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        shard_pairs(total, world, world)


def test_single_process_ranks_are_trivial():
    ranks = Ranks()
    assert (ranks.rank, ranks.world) == (0, 1)
    assert ranks.max(3.5) == 3.5 and ranks.sum(2.0) == 2.0 and ranks.gather_strings("a") == ["a"]
    ranks.barrier()


WORKER = textwrap.dedent("""
    import hashlib, sys, torch
    sys.path.insert(0, {root!r})
    import oracle
    from flashim_b200.sharding import Ranks, shard_pairs

    ranks = Ranks.from_env(backend="gloo")
    pairs = 5
    g = torch.Generator().manual_seed(4)
    level = oracle.make_refiner_level_weights(64, 1, g)
    images = torch.randn(2 * pairs, 8, 9, 64, generator=g).to(torch.bfloat16)   # two direction-images per pair
    first, count = shard_pairs(pairs, ranks.rank, ranks.world)
    mine = images[2 * first: 2 * (first + count)]
    out = oracle.refiner_level_ext(mine, level)
    digest = hashlib.sha256(out.contiguous().view(torch.int16).numpy().tobytes()).hexdigest()
    digests = ranks.gather_strings(f"{{first}}:{{count}}:{{digest}}")
    slowest = ranks.max(10.0 + ranks.rank)
    total = ranks.sum(float(count))
    ranks.barrier()
    if ranks.rank == 0:
        print("RESULT", slowest, total, "|".join(digests))
    ranks.close()
""")


@pytest.mark.timeout(300)
def test_two_gloo_ranks_reproduce_the_single_process_slices(tmp_path):
    import oracle

    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29731", str(script)],
        capture_output=True, text=True, env=env, timeout=280)
    assert result.returncode == 0, result.stderr[-2000:]
    line = next(l for l in result.stdout.splitlines() if l.startswith("RESULT"))
    _, slowest, total, digests = line.split(" ", 3)
    assert float(slowest) == 11.0 and float(total) == 5.0  # max over ranks, all pairs counted once
    # the single-process run, sliced the same way
    g = torch.Generator().manual_seed(4)
    level = oracle.make_refiner_level_weights(64, 1, g)
    images = torch.randn(10, 8, 9, 64, generator=g).to(torch.bfloat16)
    whole = oracle.refiner_level_ext(images, level)
    for entry in digests.split("|"):
        first, count, digest = entry.split(":")
        first, count = int(first), int(count)
        part = whole[2 * first: 2 * (first + count)].contiguous()
        assert hashlib.sha256(part.view(torch.int16).numpy().tobytes()).hexdigest() == digest
