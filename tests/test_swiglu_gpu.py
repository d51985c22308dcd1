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


@pytest.mark.parametrize("gate_f32", [True, False])
@pytest.mark.parametrize("n,k", [(520, 2048), (96, 256), (1024, 3584)])
def test_the_down_projection_forms_its_activations_with_the_bits_of_the_two_step_path(n, k, gate_f32):
    dev = torch.device("cuda")
    lib = cabi.load()
    codes, scales, inverse = (t.to(dev) for t in wl.cfg_nvfp4(n, k, seed=60))
    host_values = oc.values_of("nvfp4", wl.cfg_nvfp4(n, k, seed=60))
    for m in range(1, 17):
        gu = gate_up_values(m, k, 70 + m).to(dev)
        gu = gu if gate_f32 else gu.to(torch.bfloat16)
        x = torch.empty(m, k, dtype=torch.bfloat16, device=dev)
        assert lib.dg_enqueue_swiglu(_ptr(gu), 2 * k, int(gate_f32), m, k, _ptr(x), k, 0, None) == 0
        want = torch.empty(m, n, device=dev)
        h.run("nvfp4", x, (codes, scales, inverse), want)
        got = torch.full((m, n), -1.0, device=dev)
        scratch = torch.zeros(m, k, dtype=torch.bfloat16, device=dev)
        code = lib.dg_enqueue_nvfp4_swiglu(_ptr(gu), 2 * k, int(gate_f32), _ptr(scratch), _ptr(codes), _ptr(scales), 0,
                                           _ptr(inverse), _ptr(got), n, 0, m, n, k, None)
        assert code == 0, code
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), m
        assert oc.within_fp32_bound(got, x.cpu(), host_values), m          # and the product is the oracle's
    assert lib.dg_take_status() == 0
    # refusals: no scratch, gate_up rows too close or unaligned
    gu = gate_up_values(2, k, 1).to(dev)
    out = torch.empty(2, n, device=dev)
    scratch = torch.zeros(2, k, dtype=torch.bfloat16, device=dev)
    args = lambda g, ld, s: (_ptr(g), ld, 1, s, _ptr(codes), _ptr(scales), 0, _ptr(inverse), _ptr(out), n, 0, 2, n, k, None)
    assert lib.dg_enqueue_nvfp4_swiglu(*args(gu, 2 * k, None)) == 1
    assert lib.dg_enqueue_nvfp4_swiglu(*args(gu, 2 * k - 8, _ptr(scratch))) == 1
    assert lib.dg_enqueue_nvfp4_swiglu(*args(gu.view(-1)[1:], 2 * k, _ptr(scratch))) == 1
