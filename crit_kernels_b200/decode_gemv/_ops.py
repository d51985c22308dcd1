"""Loads the torch op library and exposes its namespace as `ops` (the role of kernel-builder's generated _ops.py in
the reference package, decode-gemv/torch-ext/decode_gemv/__init__.py:14)."""
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_OPS_LIB = os.path.join(_HERE, "_decode_gemv_b200.so")

if not os.path.exists(_OPS_LIB):
    raise ImportError(f"{_OPS_LIB} is missing: build it with `python -m crit_kernels_b200.builder` "
                      "(there is no fallback path)")
torch.ops.load_library(_OPS_LIB)
ops = torch.ops._decode_gemv_b200


def add_op_namespace_prefix(op_name: str) -> str:
    return f"_decode_gemv_b200::{op_name}"
