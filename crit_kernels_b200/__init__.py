"""B200-native decode GEMVs: a drop-in for the `crit-labs/decode-gemv` kernel package.

`get_kernel("crit-labs/decode-gemv", version=1)` returns the `decode_gemv` module with the reference's surface
(`gemv`, `gemv_fp8`, `gemv_bf16`, `hardware_decode`, `CUDA_ROWS`), as `kernels.get_kernel` does for the reference
(crit-kernels README.md:32-36, decode-gemv/tests/test_decode_gemv.py:14). This function is the loader: the
`build/<variant>/` tree with `metadata.json` that the real `kernels` package loads is kernel-builder's output and is
not produced by this package's builder.
"""
from __future__ import annotations

import importlib

REPO_ID = "crit-labs/decode-gemv"
VERSION = 1


def get_kernel(repo_id: str = REPO_ID, version: int | None = None, **_):
    """The module a caller of the reference gets from kernels.get_kernel(repo_id, version=...)."""
    if repo_id != REPO_ID:
        raise ValueError(f"this package provides {REPO_ID!r} only, not {repo_id!r}")
    if version not in (None, VERSION):
        raise ValueError(f"{REPO_ID} is at version {VERSION}, not {version}")
    return importlib.import_module(__name__ + ".decode_gemv")


def build(verbose: bool = False):
    """Compiles the CUDA library and the torch op library in-tree (needs nvcc and g++, no GPU)."""
    from . import builder
    return builder.build(verbose=verbose)
