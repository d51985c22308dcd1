"""The benchmark configurations at their full sizes: oracle parity on a seeded sample of rows (the FP64 oracle of a
whole 235 M-weight matrix would take minutes on the host), row invariance across every M of the configuration
bit for bit, and the size-independent properties the GEMV has: linearity in exact cases (a scaled input scales the
output by a power of two exactly; a zero input gives zero) and repeat-run equality."""
import pytest
import torch

from oracle import decode_gemv_oracle as oc
from oracle import workloads as wl
from tests import helpers as h

pytestmark = pytest.mark.gpu
dev = torch.device("cuda")

CONFIGS = {
    "c0_nvfp4": ("nvfp4", 4096, 4096, (1,), lambda: wl.cfg_nvfp4(4096, 4096, seed=10)),
    "c1_fp8": ("fp8", 28672, 8192, (1, 2, 4, 8, 16), lambda: wl.cfg_fp8(28672, 8192, seed=11)),
    "c2_mxfp8": ("mxfp8", 13824, 5120, (1, 4, 16), lambda: wl.cfg_mxfp8(13824, 5120, seed=12)),
    "c3_bf16": ("bf16", 8192, 8192, tuple(range(1, 17)), lambda: (wl.cfg_bf16(8192, 8192, seed=13),)),
    "c4_down_shard": ("nvfp4", 1024, 28672, (1, 8, 16), lambda: wl.cfg_nvfp4(1024, 28672, seed=14)),
    "c4_gate_up_shard": ("nvfp4", 7168, 8192, (1, 8, 16), lambda: wl.cfg_nvfp4(7168, 8192, seed=15)),
}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_configuration_at_full_size(name):
    fmt, n, k, ms, make = CONFIGS[name]
    host = make()
    t = tuple(a.to(dev) for a in host)
    x = wl.activations(16, k, seed=21).to(dev)
    outs = {}
    for m in ms:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        outs[m] = h.run(fmt, x[:m], t, out)
    top = max(ms)
    for m in ms:                                             # row i bit-identical across M (integer-exact)
        assert torch.equal(outs[m].view(torch.int16), outs[top][:m].view(torch.int16)), (name, m)
    # oracle on a seeded sample of rows: BF16 output, max relative error <= 1e-2 against the FP32-dequantised
    # reference path, and the FP32 output inside the reference's 2e-5 bound against the FP64 product
    rows = torch.randperm(n, generator=torch.Generator().manual_seed(5))[:192].sort().values
    sample = tuple(a[rows] for a in host)
    values = oc.values_of(fmt, sample)
    ref16 = oc.gemv_fp32(x[:top], oc.dequant_fp32(fmt, sample))
    found16 = outs[top][:, rows.to(dev)]
    assert oc.max_rel_error(found16, ref16.double()) <= 1e-2
    out32 = h.run(fmt, x[:top], t, torch.empty(top, n, device=dev))
    assert oc.within_fp32_bound(out32[:, rows.to(dev)], x[:top], values)
    assert torch.equal(out32.to(torch.bfloat16), outs[top])                      # one rounding
    # exact linearity: x * 2^-3 scales every FP32 sum by 2^-3 (no product or sum leaves the normal range here)
    scaled = h.run(fmt, (x[:top].float() * 0.125).to(torch.bfloat16), t, torch.empty(top, n, device=dev))
    assert torch.equal(scaled, out32 * 0.125)
    zero = h.run(fmt, torch.zeros_like(x[:1]), t, torch.full((1, n), 3.0, device=dev))
    assert bool((zero == 0).all())
    assert torch.equal(h.run(fmt, x[:top], t, torch.empty(top, n, device=dev)), out32)   # a repeat
