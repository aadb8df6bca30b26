"""Host-side multi-rank logic of the benchmark, run as two gloo ranks on the CPU (no GPU needed).

The data path has no collective (every rank owns its (batch, head) units); what the ranks share is the
timing protocol: barrier, per-rank device time, MAX over ranks, whole-job aggregate.
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
        fwd, bwd = bench.attn_flops(**bench.ATTN)
        out[rank] = (ms, (fwd + bwd) * world / (ms * 1e-3) / 1e12)
    finally:
        dist.destroy_process_group()


def test_two_ranks_agree_on_the_slowest_time_and_the_aggregate():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, 29000 + os.getpid() % 2000, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0][0] == res[1][0] == 15.0                      # MAX over ranks, seen by both
    assert res[0][1] == pytest.approx(2 * 1.92414e12 / 15e-3 / 1e12, rel=1e-4)   # whole-job TFLOP/s: both ranks' work


def test_flop_convention_matches_the_survey():
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
        workload, steps, warmup, gpus = "swiglu", 1, 0, 2
    assert bench.run_reference(A, rank=1, world=2) is None       # other ranks exit without work
    assert "unavailable" in bench.run_reference(A, rank=0, world=2)
