"""SwiGLU between the gate_up and down projections: the standalone kernel against the C oracle and the reference's own
kernel (bit for bit, FP32), and the down projection that forms its activations itself (dg_enqueue_nvfp4_swiglu)
against the two-step path (SwiGLU to BF16, then the GEMV): the same bits for every row count."""
import ctypes

import pytest
import torch

from crit_kernels_b200 import cabi
from oracle import build_oracle, build_ref
from oracle import decode_gemv_oracle as oc
from oracle import workloads as wl
from tests import helpers as h

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def gate_up_values(rows, inter, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, 2 * inter, generator=g) * 3
    x[0, :8] = torch.tensor([0.0, -0.0, 100.0, -100.0, 88.5, -87.5, 1e-30, -1e-30])   # the clamps of the exponential
    return x


@pytest.mark.parametrize("rows,inter", [(1, 28672), (16, 3584), (5, 1000), (3, 7), (130, 512)])
def test_swiglu_matches_the_oracle_and_the_reference_kernel(rows, inter):
    dev = torch.device("cuda")
    lib = cabi.load()
    host = gate_up_values(rows, inter, 3 + rows)
    gu = host.to(dev)
    out = torch.empty(rows, inter, device=dev)
    assert lib.dg_enqueue_swiglu(_ptr(gu), 2 * inter, 1, rows, inter, _ptr(out), inter, 1, None) == 0
    torch.cuda.synchronize()
    want = build_oracle.swiglu_f32(host)
    assert torch.equal(out.cpu().view(torch.int32), want.view(torch.int32))
    ref = build_ref.load_swiglu()
    if ref is not None:
        theirs = torch.empty(rows, inter, device=dev)
        assert ref.ref_swiglu(_ptr(gu), inter, rows, _ptr(theirs), None) == 0
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int32), theirs.view(torch.int32))
    # BF16 out: the FP32 value rounded once; BF16 in: the same function of the BF16 values
    half = torch.empty(rows, inter, dtype=torch.bfloat16, device=dev)
    assert lib.dg_enqueue_swiglu(_ptr(gu), 2 * inter, 1, rows, inter, _ptr(half), inter, 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(half, out.to(torch.bfloat16))
    gub = gu.to(torch.bfloat16)
    from_half = torch.empty(rows, inter, device=dev)
    assert lib.dg_enqueue_swiglu(_ptr(gub), 2 * inter, 0, rows, inter, _ptr(from_half), inter, 1, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(from_half.cpu().view(torch.int32), build_oracle.swiglu_f32(gub.float().cpu()).view(torch.int32))
    assert lib.dg_enqueue_swiglu(_ptr(gu), inter, 1, rows, inter, _ptr(out), inter, 1, None) == 1     # rows too close


@pytest.mark.parametrize("inter,k", [(520, 2048), (96, 256), (7168, 1024), (1001, 512), (5, 32)])
def test_gate_up_with_the_swiglu_epilogue_gives_the_bits_of_the_two_step_path(inter, k):
    dev = torch.device("cuda")
    lib = cabi.load()
    host = wl.cfg_nvfp4(2 * inter, k, seed=60)
    codes, scales, inverse = (t.to(dev) for t in host)
    inverse = (inverse * (torch.rand(2 * inter, device=dev) + 0.5)).contiguous()      # scales that differ per row
    for m in range(1, 17):
        x = wl.activations(m, k, seed=70 + m).to(dev)
        sums = torch.empty(m, 2 * inter, device=dev)
        h.run("nvfp4", x, (codes, scales, inverse), sums)                             # FP32 gate and up sums
        for out_dtype, kind in ((torch.bfloat16, 1), (torch.float32, 0)):
            want = torch.empty(m, inter, dtype=out_dtype, device=dev)
            assert lib.dg_enqueue_swiglu(_ptr(sums), 2 * inter, 1, m, inter, _ptr(want), inter,
                                         int(out_dtype == torch.float32), None) == 0
            got = torch.full((m, inter + 8), -1.0, dtype=out_dtype, device=dev)       # padded rows: nothing beside them
            code = lib.dg_enqueue_nvfp4_gate_up_swiglu(_ptr(x), x.stride(0), 1, _ptr(codes), _ptr(scales), 0,
                                                       _ptr(inverse), _ptr(got), inter + 8, kind, m, inter, k, None)
            assert code == 0, code
            torch.cuda.synchronize()
            assert torch.equal(got[:, :inter].contiguous().view(torch.int16 if kind else torch.int32),
                               want.view(torch.int16 if kind else torch.int32)), (m, out_dtype)
            assert bool((got[:, inter:] == -1.0).all())
    assert lib.dg_take_status() == 0
    # blocked scales take the same path; refusals as the GEMV's
    x = wl.activations(2, k, seed=3).to(dev)
    out = torch.empty(2, inter, dtype=torch.bfloat16, device=dev)
    args = lambda xx, i_, kk: (_ptr(xx), xx.stride(0), 1, _ptr(codes), _ptr(scales), 0, _ptr(inverse), _ptr(out), inter,
                               1, 2, i_, kk, None)
    assert lib.dg_enqueue_nvfp4_gate_up_swiglu(*args(x, inter, k)) == 0
    assert lib.dg_enqueue_nvfp4_gate_up_swiglu(*args(x, 0, k)) == 1
    assert lib.dg_enqueue_nvfp4_gate_up_swiglu(*args(x, inter, k + 16)) == 1
    torch.cuda.synchronize()
