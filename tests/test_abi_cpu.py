"""Host-side checks that need no GPU: the C-ABI library loads and exports what include/decode_gemv_b200.h declares,
the launch planner is a pure function of the sizes, the refusals that come before any device work, and the package
surface."""
import ctypes
import os
import re

import pytest

from crit_kernels_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    with open(os.path.join(ROOT, "include", "decode_gemv_b200.h")) as f:
        return re.findall(r"DG_API\s+(?:unsigned\s+long\s+long|int)\s+(dg_\w+)\s*\(", f.read())


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 7 and set(names) == set(cabi.SIGNATURES)
    lib = ctypes.CDLL(cabi.library_path())
    for name in names:
        assert getattr(lib, name) is not None, name
    assert cabi.load().dg_version() >= 100


@pytest.mark.parametrize("fmt,n,k", [("fp8", 28672, 8192), ("mxfp8", 13824, 5120), ("bf16", 8192, 8192),
                                     ("nvfp4", 4096, 4096), ("nvfp4", 57344, 8192), ("nvfp4", 1024, 28672),
                                     ("nvfp4", 1, 32), ("bf16", 5, 8), ("fp8", 130, 2048)])
def test_plans_fit_the_device_and_do_not_depend_on_the_call(fmt, n, k):
    for m in range(1, 17):
        p = cabi.plan(fmt, m, n, k)
        assert p == cabi.plan(fmt, m, n, k)
        # one CTA per SM with all its shared memory, or two that share it (1 KB per CTA is the system's)
        assert 1 <= p["ctas"] <= 296 and p["ctas"] <= n
        assert p["stages"] >= 2 and p["smem_bytes"] <= (232448 if p["ctas"] <= 148 else 115712)
        # header + ring, then (FP8 / NVFP4 at few rows) the activations that stay resident behind it
        behind = p["smem_bytes"] - (256 + p["stages"] * p["stage_bytes"])
        assert 0 <= behind <= 96 * 1024 + 16 and (behind == 0 or fmt in ("fp8", "nvfp4"))
        assert 1 <= p["rows_per_warp"] <= 8 and 1 <= p["steps"] <= 8


def test_planner_keeps_small_activations_resident():
    """FP8 / NVFP4 at few rows: the whole [M][K] activations stay in shared memory behind the ring when they are small
    (whole 512-byte steps of every row, plus a flag byte per step), unless that costs the ring its third stage."""
    def behind(fmt, m, n, k):
        p = cabi.plan(fmt, m, n, k)
        return p["smem_bytes"] - (256 + p["stages"] * p["stage_bytes"]), p["stages"]
    assert behind("nvfp4", 1, 8192, 8192) == (8 * 2048 + 16, 3)
    assert behind("nvfp4", 2, 57344, 8192) == (8 * 2 * 2048 + 16, 3)
    assert behind("fp8", 4, 28672, 8192) == (16 * 4 * 1024 + 16, 3)
    assert behind("nvfp4", 1, 8192, 28672)[0] == 0           # 56 KB would leave two stages
    assert behind("nvfp4", 4, 8192, 8192)[0] == 8 * 4 * 2048 + 16
    assert behind("fp8", 5, 8192, 8192)[0] == 0 and behind("nvfp4", 5, 8192, 8192)[0] == 0   # kernels without the mode
    assert behind("mxfp8", 1, 8192, 8192)[0] == 0 and behind("bf16", 1, 8192, 8192)[0] == 0


def test_planner_refuses_what_the_kernels_refuse():
    lib = cabi.load()
    out = (ctypes.c_int * 6)()
    assert lib.dg_plan(3, 17, 96, 256, out) != 0      # 17 rows
    assert lib.dg_plan(3, 1, 96, 48, out) != 0        # NVFP4 K not a multiple of 32
    assert lib.dg_plan(1, 1, 96, 24, out) != 0        # FP8 K not a multiple of 16
    assert lib.dg_plan(2, 1, 96, 48, out) != 0        # MXFP8 K not a multiple of 32
    assert lib.dg_plan(0, 1, 96, 12, out) != 0        # BF16 K not a multiple of 8
    assert lib.dg_plan(0, 1, 0, 8, out) != 0          # no rows
    assert lib.dg_plan(7, 1, 96, 256, out) != 0       # unknown format


def test_enqueue_refuses_bad_sizes_before_touching_a_device():
    lib = cabi.load()
    p = ctypes.c_void_p(4096)   # never dereferenced: the size checks come first
    assert lib.dg_enqueue_nvfp4(p, 256, 1, p, p, 0, p, p, 96, 0, 17, 96, 256, None) == 1
    assert lib.dg_enqueue_nvfp4(p, 256, 1, p, p, 0, p, p, 96, 0, 1, 96, 48, None) == 1
    assert lib.dg_enqueue_fp8(p, 256, 1, p, p, p, p, 96, 0, 1, 96, 256, None) == 1        # both scales
    assert lib.dg_enqueue_fp8(p, 256, 1, p, None, None, p, 96, 0, 1, 96, 256, None) == 1  # neither
    assert lib.dg_enqueue_bf16(p, 256, p, p, 96, 0, 0, 96, 256, None) == 1
    assert lib.dg_enqueue_bf16(ctypes.c_void_p(4100), 256, p, p, 96, 0, 1, 96, 256, None) == 1   # x off 16 bytes


def test_package_surface_matches_the_reference():
    import crit_kernels_b200
    mod = crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)
    assert mod.CUDA_ROWS == 16
    for name in ("gemv", "gemv_fp8", "gemv_bf16", "hardware_decode"):
        assert callable(getattr(mod, name))
    with pytest.raises(AttributeError):
        mod.gemv_triton
    with pytest.raises(ValueError):
        crit_kernels_b200.get_kernel("crit-labs/mma-rows")
    import torch
    schema = str(torch.ops._decode_gemv_b200.gemv.default._schema)
    assert schema.startswith("_decode_gemv_b200::gemv(Tensor x, Tensor codes, Tensor scales, Tensor inverse, "
                             "bool blocked, Tensor(") and schema.endswith(" out) -> ()") and "!" in schema


def test_dequantizer_wrappers_refuse_wrong_output_types_before_any_device_work():
    """decode writes 16-bit outputs, decode_fp8 FP8 E4M3: the other types are refused by the package functions
    themselves (no GPU needed to see it)."""
    import torch
    import crit_kernels_b200
    k = crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)
    c = torch.zeros(2, 8, dtype=torch.uint8)
    s = torch.zeros(2, 1, dtype=torch.uint8)
    f = torch.ones(2)
    with pytest.raises(RuntimeError):
        k.decode(c, s, f, torch.empty(2, 16, dtype=torch.float32))
    with pytest.raises(RuntimeError):
        k.decode(c, s, f, torch.empty(2, 16, dtype=torch.float8_e4m3fn))
    with pytest.raises(RuntimeError):
        k.decode_fp8(c, s, f, torch.empty(2, 16, dtype=torch.bfloat16))
    assert {"decode", "decode_fp8"} <= set(k.__all__)
    with pytest.raises(AttributeError):
        k.gemv_triton
