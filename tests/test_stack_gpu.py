"""The column-sharded NVFP4 stack on 2, 4 and 8 GPUs: the gathered outputs are bit-identical to the single-GPU outputs
for every projection and M, eager and from the captured graph, also when the activations change from replay to replay
(a gathered buffer that a fast rank overwrote too early would show there). Needs at least two GPUs (skipped
otherwise); ranks are child processes over NCCL on 127.0.0.1."""
import datetime
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROLES = (("qkv", 1024, 1280), ("o", 1024, 1024), ("gate_up", 1024, 7168), ("down", 3584, 1024))


def _worker(rank, world, port, gather, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=90))
    try:
        from crit_kernels_b200 import stack as stk
        batch = 0
        if gather.startswith("batch"):
            gather, batch = "fused", int(gather[5:])
        sharded = stk.ShardedStack.random(2, ROLES, rank, world, dev, seed=5, gather=gather, batch=batch)
        whole = stk.ShardedStack.random(2, ROLES, 0, 1, dev, seed=5)
        for m in (1, 8, 16):
            got, want = sharded.run(m), whole.run(m)
            for i, (g, w) in enumerate(zip(got, want)):
                assert torch.equal(g.view(torch.int16), w.view(torch.int16)), (m, i)
            run = sharded.capture(m)
            run.replay()
            torch.cuda.synchronize()
            last = run.full["down"].permute(1, 0, 2).reshape(m, -1)
            assert torch.equal(last, want[-1])
            run.replay()                                     # a second replay: the arrival counters were re-armed
            torch.cuda.synchronize()
            assert torch.equal(run.full["down"].permute(1, 0, 2).reshape(m, -1), want[-1])
            # new activations before every replay, every role's output of every replay checked
            alone = stk.StackRun(whole, m)
            for rep in range(4):
                g = torch.Generator().manual_seed(1000 + 17 * rep + m)
                for role, k, _ in ROLES:
                    fresh = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev)
                    run.x[role].copy_(fresh)
                    alone.x[role].copy_(fresh)
                run.replay()
                keep = []
                alone.eager(keep)
                torch.cuda.synchronize()
                outs = run.outputs()
                for (role, _, _), w in zip(ROLES, keep[-len(ROLES):]):
                    assert torch.equal(outs[role].view(torch.int16), w.view(torch.int16)), (m, rep, role)
            del run          # a live graph that captured the group's collectives blocks the group's teardown
        results[rank] = "ok"
        torch.cuda.synchronize()
        dist.barrier()
    except BaseException:
        import traceback
        results[rank] = traceback.format_exc()       # the parent shows it: the teardown below may end the process
        raise
    finally:
        import threading
        guard = threading.Timer(30.0, lambda: os._exit(0 if results.get(rank) == "ok" else 1))
        guard.daemon = True
        guard.start()
        dist.destroy_process_group()
        guard.cancel()


@pytest.mark.parametrize("gather", ["fused", "fused-overlap", "nccl", "batch4", "batch2"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_stack_reproduces_the_single_gpu_bits(world, gather):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with mp.Manager() as manager:
        results = manager.dict()
        port = 29531 + world + {"fused": 10, "fused-overlap": 20, "nccl": 0, "batch4": 30, "batch2": 40}[gather]
        try:
            mp.spawn(_worker, args=(world, port, gather, results), nprocs=world, join=True)
        except Exception as error:          # a rank's own traceback says more than the spawner's
            assert dict(results) == {r: "ok" for r in range(world)}, f"{error}"
        assert dict(results) == {r: "ok" for r in range(world)}
