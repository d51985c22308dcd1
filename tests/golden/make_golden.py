"""Generates tests/golden/decode_gemv_golden.npz from the reference's own test-side oracle.

The reference keeps no stored fixtures for decode-gemv: its tests compute every expected value at run time with a few
host functions (decode-gemv/tests/test_decode_gemv.py: `E2M1` :16-17, `values` :29-34, `fp8_values` :210-214,
`to_blocked` :280-287). That test module cannot be imported (it loads the built kernel at import), so this script
parses the file, executes only those definitions (pure torch, CPU) and records their outputs on seeded inputs drawn
with the reference's own generators (`matrix` :20-26, `fp8_matrix` :198-207, `activations` :37-38, with the device
moved to the CPU). The fixture pins oracle/decode_gemv_oracle.py to the reference. It also holds answers of the reference's C++ host
oracle (fp8-block-rows/tests/order/row_fp8.h, fp8_block.h) computed by oracle/_ref/ref_host_check (host_* entries).

Run where the reference checkout is present:
    python tests/golden/make_golden.py [path/to/reference]
The fixture travels with the repository; the GPU box never needs the reference.
"""
import ast
import os
import sys

import numpy as np
import torch

WANTED = {"E2M1", "matrix", "values", "activations", "fp8_matrix", "fp8_values", "to_blocked"}


def load_reference_functions(path):
    with open(path) as f:
        tree = ast.parse(f.read())
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in WANTED:
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id in WANTED for t in node.targets):
            keep.append(node)
    space = {"torch": torch, "dev": torch.device("cpu")}
    exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), space)
    missing = WANTED - set(space)
    if missing:
        raise SystemExit(f"reference test file lacks {sorted(missing)}")
    return space


def host_oracle_vectors(root):
    """Answers of the reference's header-only C++ host oracle (fp8-block-rows/tests/order/row_fp8.h `decode`,
    `project`; fp8_block.h `quantize_group`, `e8m0`), run through oracle/_ref/ref_host_check on seeded inputs: an
    implementation that shares no code with torch, as a second pin of the Python oracle."""
    import struct
    import subprocess
    import tempfile
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from oracle import build_ref
    if not build_ref.build_host_check(root, verbose=False):
        raise SystemExit("the reference's host oracle headers were not found")
    g = torch.Generator().manual_seed(41)
    rows, width, tokens, groups = 24, 160, 5, 64
    codes = torch.randint(0, 256, (rows, width), generator=g, dtype=torch.uint8)
    codes[(codes & 127) == 127] = 0x38                                       # no NaN codes (the oracle rejects them)
    scales = ((torch.rand(rows, generator=g) * 1.5 + 0.5) / 64).to(torch.bfloat16).view(torch.int16)
    x = torch.randn(tokens, width, generator=g).to(torch.bfloat16).view(torch.int16)
    values = torch.randn(groups, 32, generator=g) * 0.02
    values[0] = 0                                                             # an all-zero group
    values[1] *= 2.0 ** -20                                                   # small
    values[2] *= 2.0 ** 12                                                    # large
    values[3, 0] = 0.0625                                                     # an exact power of two as the maximum
    values[3, 1:] *= 0.5
    with tempfile.TemporaryDirectory() as tmp:
        src, dst = os.path.join(tmp, "in.bin"), os.path.join(tmp, "out.bin")
        with open(src, "wb") as f:
            f.write(struct.pack("<4i", rows, width, tokens, groups))
            for t in (codes, scales, x, values.float()):
                f.write(t.contiguous().numpy().tobytes())
        subprocess.run([build_ref.HOST_CHECK, src, dst], check=True)
        raw = open(dst, "rb").read()
    table = np.frombuffer(raw, dtype="<f4", count=256, offset=0)
    projected = np.frombuffer(raw, dtype="<f8", count=tokens * rows, offset=1024).reshape(tokens, rows)
    rest = np.frombuffer(raw, dtype=np.uint8, offset=1024 + 8 * tokens * rows).reshape(groups, 8 + 32)
    pair = rest[:, :8].copy().view("<f4")
    return {"host_codes": codes.numpy(), "host_scales_bf16": scales.numpy(), "host_x_bf16": x.numpy(),
            "host_decode": table.copy(), "host_project": projected.copy(), "host_mx_values": values.float().numpy(),
            "host_mx_scale": pair[:, 0].copy(), "host_mx_e8m0": pair[:, 1].copy(), "host_mx_codes": rest[:, 8:].copy()}


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CRIT_KERNELS_REFERENCE", "")
    if not root:
        raise SystemExit("give the reference checkout: CRIT_KERNELS_REFERENCE=<path> or the path as the argument")
    ref = load_reference_functions(os.path.join(root, "decode-gemv", "tests", "test_decode_gemv.py"))
    out = {"e2m1_table": ref["E2M1"].numpy()}
    # every E4M3 byte as torch decodes it (the reference decodes with view(float8_e4m3fn), :211)
    out["e4m3_all"] = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).double().numpy()
    for tag, (n, k, m) in {"a": (96, 256, 16), "b": (130, 544, 5), "c": (40, 1024, 3)}.items():
        c, s, i = ref["matrix"](n, k)
        x = ref["activations"](m, k)
        v = ref["values"](c, s, i)
        out[f"nvfp4_{tag}_codes"] = c.numpy()
        out[f"nvfp4_{tag}_scales"] = s.view(torch.uint8).numpy()
        out[f"nvfp4_{tag}_inverse"] = i.numpy()
        out[f"nvfp4_{tag}_x"] = x.float().numpy()            # bf16 values, exactly representable in FP32
        out[f"nvfp4_{tag}_values"] = v.numpy()
        out[f"nvfp4_{tag}_exact"] = (x.double() @ v.t()).numpy()
        out[f"nvfp4_{tag}_blocked"] = ref["to_blocked"](s.view(torch.uint8)).numpy()
        # what the reference's test expects of its dequantizers decode / decode_fp8 (test_decode_gemv.py:131-140)
        if tag == "c":
            continue
        unit = ref["values"](c, s, torch.ones_like(i)).float()
        product = unit * i[:, None]
        out[f"nvfp4_{tag}_decode_bf16"] = product.to(torch.bfloat16).view(torch.int16).numpy()
        out[f"nvfp4_{tag}_decode_f16"] = product.to(torch.float16).view(torch.int16).numpy()
        factor = i * 64
        out[f"nvfp4_{tag}_decode_fp8"] = (unit * factor[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn) \
            .view(torch.uint8).numpy()
    for tag, (n, k, m, mx) in {"row": (96, 256, 16, False), "mx": (70, 512, 7, True)}.items():
        c, s = ref["fp8_matrix"](n, k, mx)
        x = ref["activations"](m, k)
        v = ref["fp8_values"](c, s)
        out[f"fp8_{tag}_codes"] = c.numpy()
        out[f"fp8_{tag}_scales"] = s.numpy()
        out[f"fp8_{tag}_x"] = x.float().numpy()
        out[f"fp8_{tag}_values"] = v.numpy()
        out[f"fp8_{tag}_exact"] = (x.double() @ v.t()).numpy()
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(64, 512, generator=g) * 0.05).to(torch.bfloat16)   # test_decode_gemv.py:92-93, smaller
    x = ref["activations"](16, 512)
    out["bf16_w"] = w.float().numpy()
    out["bf16_x"] = x.float().numpy()
    out["bf16_exact"] = (x.double() @ w.double().t()).numpy()
    out.update(host_oracle_vectors(root))
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "decode_gemv_golden.npz"), **out)
    print("wrote", os.path.join(here, "decode_gemv_golden.npz"), sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
