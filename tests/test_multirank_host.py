"""Host-side multi-rank logic of the benchmark, run as two gloo ranks on the CPU (no GPU needed).

The data path has no collective (every rank owns a contiguous block of the (batch, head) units); what the ranks
share is the split of the units and the timing protocol: barrier, per-rank device time, MAX over ranks, whole-job aggregate.
"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    sys.path.insert(0, ROOT)
    import bench
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        assert bench.dist_env() == (rank, world, rank)
        bench.barrier(world)
        ms = bench.max_over_ranks(10.0 + 5.0 * rank, world, torch.device("cpu"))
        # strong scaling: the 128 (batch, head) units are dealt out in contiguous blocks, the aggregate is all of the work
        lo, nb = bench.shard_batches(bench.ATTN["B"], bench.ATTN["H"], rank, world)
        fwd, bwd = bench.attn_flops(**dict(bench.ATTN, B=nb))
        out[rank] = (ms, (fwd + bwd) * world / (ms * 1e-3) / 1e12, lo, nb)
    finally:
        dist.destroy_process_group()


def test_two_ranks_agree_on_the_slowest_time_and_the_aggregate():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, 29000 + os.getpid() % 2000, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0][0] == res[1][0] == 15.0                      # MAX over ranks, seen by both
    assert res[0][1] == pytest.approx(1.92414e12 / 15e-3 / 1e12, rel=1e-4)       # whole-job TFLOP/s: all 128 units / slowest rank
    assert (res[0][2], res[0][3]) == (0, 4) and (res[1][2], res[1][3]) == (4, 4)  # contiguous blocks that tile the batch


def test_flop_convention_of_the_headline_configurations():
    sys.path.insert(0, ROOT)
    import bench
    fwd, bwd = bench.attn_flops(B=8, H=16, S=4096, D=128)
    assert fwd == pytest.approx(0.5498e12, rel=1e-3) and bwd == pytest.approx(1.3744e12, rel=1e-3)
    fwd1, bwd1 = bench.attn_flops(B=2, H=12, S=512, D=64)
    assert fwd1 + bwd1 == pytest.approx(2.818e9, rel=1e-3)


def test_reference_arm_runs_on_rank_zero_only():
    sys.path.insert(0, ROOT)
    import bench

    class A:
        workload, steps, warmup, gpus = "softmax", 1, 0, 2
    assert bench.run_reference(A, rank=1, world=2) is None       # other ranks exit without work
    line = bench.run_reference(A, rank=0, world=2)
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0


def test_unit_blocks_tile_the_batch():
    sys.path.insert(0, ROOT)
    import bench
    for world in (1, 2, 4, 8):
        blocks = [bench.shard_batches(8, 16, r, world) for r in range(world)]
        assert [b[0] for b in blocks] == list(range(0, 8, 8 // world)) and all(b[1] == 8 // world for b in blocks)
    with pytest.raises(SystemExit):
        bench.shard_batches(8, 16, 0, 3)
