"""Several NVFP4 GEMVs in one launch (dg_encode_nvfp4_batch + dg_enqueue_batch) give, row for row, the bits of the same
GEMVs enqueued one by one: shapes that leave CTAs without rows, ragged K windows, both scale paths, every shape class
of M, with and without the (single-rank) all-gather epilogue, eager and replayed from a CUDA graph."""
import ctypes

import pytest
import torch

from crit_kernels_b200 import cabi
from oracle import workloads as wl
from tests import helpers as h

pytestmark = pytest.mark.gpu
SHAPES = ((1280, 2048), (96, 256), (7168, 1024), (1024, 3584), (130, 2080), (5, 32), (3000, 512))


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def encode(lib, items, m, world, flags, slot, dev):
    count = len(items)
    nbytes = lib.dg_batch_blob_bytes(count)
    host = torch.zeros(nbytes, dtype=torch.uint8)
    device = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    array = (cabi.Nvfp4BatchItem * count)(*items)
    flag_ptrs = (ctypes.c_void_p * 1)(flags.data_ptr()) if world else None
    code = lib.dg_encode_nvfp4_batch(ctypes.cast(array, ctypes.c_void_p), count, 1, 1, m, world, 0, flag_ptrs, slot,
                                     _ptr(device), _ptr(host))
    assert code == 0, code
    device.copy_(host)
    return host, device


@pytest.mark.parametrize("m", [1, 2, 4, 5, 8, 11, 16])
@pytest.mark.parametrize("world", [0, 1])
def test_a_batch_gives_the_bits_of_single_calls(m, world):
    dev = torch.device("cuda")
    lib = cabi.load()
    mats, xs, want = [], [], []
    for i, (n, k) in enumerate(SHAPES):
        codes, scales, inverse = (t.to(dev) for t in wl.cfg_nvfp4(n, k, seed=20 + i))
        if i == 2:
            scales = torch.cat([torch.zeros(2, dtype=torch.uint8, device=dev), scales.flatten()])[2:].view(n, k // 16)   # read directly
        x = wl.activations(m, k, seed=50 + i).to(dev)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        h.run("nvfp4", x, (codes, scales, inverse), out)
        mats.append((codes, scales, inverse))
        xs.append(x)
        want.append(out)
    torch.cuda.synchronize()
    got = [torch.full((max(world, 1), m, n), -1.0, dtype=torch.bfloat16, device=dev) for n, _ in SHAPES]
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    keep, items = [], []
    for (n, k), (codes, scales, inverse), x, g in zip(SHAPES, mats, xs, got):
        peers = (ctypes.c_void_p * 1)(g.data_ptr())
        keep.append(peers)
        items.append(cabi.Nvfp4BatchItem(x=x.data_ptr(), codes=codes.data_ptr(), scales=scales.data_ptr(),
                                         inverse=inverse.data_ptr(), out=g.data_ptr(),
                                         peer_out=ctypes.cast(peers, ctypes.POINTER(ctypes.c_void_p)),
                                         ldx=x.stride(0), ldo=n, blocked=0, N=n, K=k))
    host, device = encode(lib, items, m, world, flags, 0, dev)
    assert lib.dg_enqueue_batch(_ptr(host), None) == 0
    torch.cuda.synchronize()
    for g, w in zip(got, want):
        assert torch.equal(g[0].view(torch.int16), w.view(torch.int16)), (m, world, tuple(w.shape))
    assert int(flags.abs().sum()) == 0                        # the arrival counters are re-armed
    # replayed from a graph, twice
    for g in got:
        g.fill_(-1.0)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        assert lib.dg_enqueue_batch(_ptr(host), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    for _ in range(2):
        for g in got:
            g.fill_(-1.0)
        graph.replay()
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            assert torch.equal(g[0].view(torch.int16), w.view(torch.int16))
    assert lib.dg_take_status() == 0


def test_a_batch_refuses_what_single_calls_refuse():
    dev = torch.device("cuda")
    lib = cabi.load()
    n, k, m = 64, 256, 2
    codes, scales, inverse = (t.to(dev) for t in wl.cfg_nvfp4(n, k))
    x = wl.activations(m, k).to(dev)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    good = dict(x=x.data_ptr(), codes=codes.data_ptr(), scales=scales.data_ptr(), inverse=inverse.data_ptr(),
                out=out.data_ptr(), peer_out=None, ldx=x.stride(0), ldo=n, blocked=0, N=n, K=k)
    host = torch.zeros(lib.dg_batch_blob_bytes(1), dtype=torch.uint8)
    device = torch.zeros_like(host, device=dev)

    def code(m_rows=m, **changed):
        item = (cabi.Nvfp4BatchItem * 1)(cabi.Nvfp4BatchItem(**{**good, **changed}))
        return lib.dg_encode_nvfp4_batch(ctypes.cast(item, ctypes.c_void_p), 1, 1, 1, m_rows, 0, 0, None, 0,
                                         _ptr(device), _ptr(host))
    assert code() == 0
    assert code(K=k + 16) == 1 and code(N=0) == 1 and code(m_rows=17) == 1 and code(out=None) == 1
    assert code(codes=codes.data_ptr() + 1) == 1 and code(ldx=x.stride(0) + 1) == 1
    assert lib.dg_enqueue_batch(_ptr(torch.zeros(512, dtype=torch.uint8)), None) == 1     # not an encoded batch


def test_the_stack_in_batched_launches_reproduces_the_chain_of_single_launches():
    from crit_kernels_b200 import stack as stk
    dev = torch.device("cuda")
    roles = (("qkv", 1024, 1280), ("o", 1024, 1024), ("gate_up", 1024, 7168), ("down", 3584, 1024))
    chain = stk.ShardedStack.random(3, roles, 0, 1, dev, seed=5)
    for per_launch in (4, 3, 12):
        batched = chain.with_batch(per_launch)
        for m in (1, 8, 16):
            want = chain.run(m)
            if per_launch <= 4:
                got = batched.run(m)
                assert len(got) == len(want)
                for g, w in zip(got, want):
                    assert torch.equal(g.view(torch.int16), w.view(torch.int16)), (per_launch, m)
            run = batched.capture(m)
            for _ in range(2):
                run.replay()
                torch.cuda.synchronize()
                for (role, _, _), w in zip(roles, want[-4:]):
                    assert torch.equal(run.outputs()[role].view(torch.int16), w.view(torch.int16)), (per_launch, m, role)
