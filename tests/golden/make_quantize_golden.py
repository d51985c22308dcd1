"""Generates tests/golden/quantize_golden.npz from the reference's own test-side quantizers.

The reference states its activation quantizers as torch expressions in its test file (mma-rows/tests/
test_mma_rows.py: `fp8_rows` :80-83, `BOUNDS` / `TIES` :86-87, `nvfp4_quantize` :90-104, `to_blocked` :21-27,
`activations` :57-58, `INPUT_SCALE` :18) and checks its kernels against them bit for bit on CUDA tensors (:153-174).
This script parses that file, executes only those definitions and evaluates them on the reference test's own inputs.
It must run on a CUDA device: torch divides a CUDA tensor by a constant as a product with the FP32 reciprocal, a CPU
tensor by a true division, and the quantizers' bits are those of the CUDA form.

    python tests/golden/make_quantize_golden.py path/to/mma-rows/tests/test_mma_rows.py [out.npz]
"""
import ast
import os
import sys

import numpy as np
import torch

WANTED = {"E2M1", "INPUT_SCALE", "to_blocked", "activations", "fp8_rows", "BOUNDS", "TIES", "nvfp4_quantize"}


def load_reference_functions(path):
    import math
    with open(path) as f:
        tree = ast.parse(f.read())
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in WANTED:
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id in WANTED for t in node.targets):
            keep.append(node)
    space = {"torch": torch, "math": math, "dev": torch.device("cuda")}
    exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), space)
    missing = WANTED - set(space)
    if missing:
        raise SystemExit(f"reference test file lacks {sorted(missing)}")
    return space


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device (see the module docstring)")
    ref = load_reference_functions(sys.argv[1])
    out = sys.argv[2] if len(sys.argv) > 2 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                             "quantize_golden.npz")
    data = {"input_scale": np.float32(ref["INPUT_SCALE"])}
    # the reference test's own case (test_mma_rows.py:155-156, :168-174)
    x = ref["activations"](37, 2048, seed=3) * 4
    x[3, :100] = 0
    q, scale = ref["fp8_rows"](x)
    codes, scales = ref["nvfp4_quantize"](x, ref["INPUT_SCALE"])
    data.update(a_x=x.view(torch.int16).cpu().numpy(), a_q=q.view(torch.uint8).cpu().numpy(),
                a_scale=scale.cpu().numpy(),
                a_codes=(codes[:, 0::2] | (codes[:, 1::2] << 4)).cpu().numpy(),
                a_block_scales=scales.view(torch.uint8).cpu().numpy(),
                a_blocked=ref["to_blocked"](scales.view(torch.uint8)).cpu().numpy())
    # its ragged FP8 cases (:162-167): K = 1001 and K = 20000 of a [5][20480] batch
    xk = ref["activations"](5, 20480, seed=6) * 2
    data["b_x"] = xk.view(torch.int16).cpu().numpy()
    for k in (1001, 20000):
        q, scale = ref["fp8_rows"](xk[:, :k])
        data[f"b_q_{k}"] = q.view(torch.uint8).cpu().numpy()
        data[f"b_scale_{k}"] = scale.cpu().numpy()
    # a wider spread of magnitudes (tiny and huge blocks, exact ties of the E2M1 grid)
    g = torch.Generator().manual_seed(11)
    wide = torch.randn(9, 512, generator=g) * torch.exp2(torch.randint(-30, 12, (9, 32), generator=g).float()
                                                         ).repeat_interleave(16, dim=1)
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.25, -0.75, -1.75, -3.5, 0.0, 1.0, -6.0])
    wide[8, :16] = ties * (6.0 / ref["INPUT_SCALE"])
    wide = wide.to(torch.bfloat16).to(ref["dev"])
    q, scale = ref["fp8_rows"](wide)
    codes, scales = ref["nvfp4_quantize"](wide, ref["INPUT_SCALE"])
    data.update(c_x=wide.view(torch.int16).cpu().numpy(), c_q=q.view(torch.uint8).cpu().numpy(),
                c_scale=scale.cpu().numpy(), c_codes=(codes[:, 0::2] | (codes[:, 1::2] << 4)).cpu().numpy(),
                c_block_scales=scales.view(torch.uint8).cpu().numpy())
    np.savez_compressed(out, **data)
    print(f"wrote {out}: {sorted(data)}")


if __name__ == "__main__":
    main()
