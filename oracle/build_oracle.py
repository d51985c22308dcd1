"""TEST INFRASTRUCTURE ONLY. Compiles the C part of the oracle (oracle/swiglu_oracle.c) with gcc into
oracle/_ref/libswiglu_oracle.so (git-ignored, shipped to the GPU box) and loads it.

    python -m oracle.build_oracle
"""
import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libswiglu_oracle.so")
SRC = os.path.join(HERE, "swiglu_oracle.c")


def build(verbose=True):
    if os.path.exists(LIB) and os.path.getmtime(LIB) > os.path.getmtime(SRC):
        return True
    os.makedirs(OUT_DIR, exist_ok=True)
    # no contraction of a * b + c into an FMA the source does not name, no reassociation
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", SRC, "-o", LIB, "-lm"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return True


def swiglu_f32(gate_up):
    """gate_up: float32 torch tensor [rows][2 * inter] -> float32 [rows][inter], the reference's bits."""
    import torch
    build(verbose=False)
    lib = ctypes.CDLL(LIB)
    lib.swiglu_f32.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.swiglu_f32.restype = None
    g = gate_up.detach().cpu().float().contiguous()
    rows, two = g.shape
    out = torch.empty(rows, two // 2, dtype=torch.float32)
    lib.swiglu_f32(g.data_ptr(), two // 2, rows, out.data_ptr())
    return out


if __name__ == "__main__":
    build()
