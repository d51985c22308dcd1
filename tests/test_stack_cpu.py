"""The sharded stack's host logic on CPU: two gloo ranks, the GEMV replaced by the oracle's FP32 dequantise-and-matmul
(test stand-in only; the product stack always runs the CUDA ops). Checks the row slicing, the all-gather layout
[P][M][N/P] -> [M][N] and that the gathered result equals the unsharded one."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROLES = (("a", 256, 64), ("b", 512, 96))


class HostKernel:
    """Oracle-backed stand-in with the op surface the stack calls."""

    @staticmethod
    def gemv(x, codes, scales, inverse, out, blocked=False):
        from oracle import decode_gemv_oracle as oc
        out.copy_(oc.gemv_fp32(x, oc.dequant_fp32("nvfp4", (codes, scales, inverse)), out.dtype))
        return out


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from crit_kernels_b200 import stack as stk
        dev = torch.device("cpu")
        sharded = stk.ShardedStack.random(2, ROLES, rank, world, dev, seed=3, kernel=HostKernel(), gather="nccl")
        whole = stk.ShardedStack.random(2, ROLES, 0, 1, dev, seed=3, kernel=HostKernel())
        assert sharded.projections[0].codes.shape[0] == ROLES[0][2] // world
        lo = rank * ROLES[0][2] // world
        assert torch.equal(sharded.projections[0].codes, whole.projections[0].codes[lo:lo + ROLES[0][2] // world])
        for m in (1, 3):
            got, want = sharded.run(m), whole.run(m)
            assert len(got) == len(want) == 4
            for g, w in zip(got, want):
                assert g.shape == w.shape and torch.equal(g, w)
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_two_ranks_gather_the_unsharded_result():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, 29517, results), nprocs=world, join=True)
        assert dict(results) == {0: "ok", 1: "ok"}


def test_rows_must_split_evenly():
    from crit_kernels_b200 import stack as stk
    with pytest.raises(ValueError):
        stk.ShardedStack.random(1, (("a", 256, 66),), 0, 4, torch.device("cpu"), kernel=HostKernel())
