"""In-tree build of the B200 decode-GEMV libraries (the stand-in for kernel-builder's build of build.toml).

  lib/libdecode_gemv_b200.so          the kernels and their C ABI (include/decode_gemv_b200.h); nvcc, sm_100a only,
                                      CUDA runtime linked statically, no torch
  decode_gemv/_decode_gemv_b200.so    the torch op library over that ABI (torch-ext/torch_binding.cpp); g++

Objects land in build/obj and are rebuilt only when a source or header is newer. Run `python -m
crit_kernels_b200.builder` (or call build()); nvcc cross-compiles, so no GPU is needed.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")
ABI_LIB = os.path.join(HERE, "lib", "libdecode_gemv_b200.so")
OPS_LIB = os.path.join(HERE, "decode_gemv", "_decode_gemv_b200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{done.stdout}\n{done.stderr}")
    return done.stdout + done.stderr


def build_abi(verbose=False, ptxas_info=False):
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(ABI_LIB), exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "decode_gemv_b200.h"))
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs, objects = [], []
    for src in sources:
        obj = os.path.join(OBJ, src[:-3] + ".o")
        objects.append(obj)
        if _newer(obj, [os.path.join(CSRC, src)] + headers):
            flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])
            jobs.append([NVCC] + flags + ["-c", os.path.join(CSRC, src), "-o", obj])
    logs = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            logs = list(pool.map(lambda c: _run(c, verbose), jobs))
    if jobs or _newer(ABI_LIB, objects):
        _run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-Xcompiler",
              "-fPIC", "-o", ABI_LIB] + objects, verbose)
    return "\n".join(logs)


def build_ops(verbose=False):
    import torch
    from torch.utils.cpp_extension import include_paths
    src = os.path.join(HERE, "torch-ext", "torch_binding.cpp")
    deps = [src, os.path.join(HERE, "torch-ext", "torch_binding.h"), os.path.join(ROOT, "include", "decode_gemv_b200.h"),
            ABI_LIB]
    if not _newer(OPS_LIB, deps):
        return
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", 
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in include_paths()] + [f"-I{os.path.join(CUDA_HOME, 'include')}"]
    cmd += [src, "-o", OPS_LIB, f"-L{os.path.dirname(ABI_LIB)}", "-ldecode_gemv_b200", f"-L{torch_lib}", "-lc10",
            "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", f"-L{os.path.join(CUDA_HOME, 'lib64')}", "-lcudart",
            "-Wl,-rpath,$ORIGIN/../lib", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)


def build(verbose=False, ptxas_info=False):
    log = build_abi(verbose, ptxas_info)
    build_ops(verbose)
    return log


if __name__ == "__main__":
    out = build(verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    if "--ptxas-info" in sys.argv:
        print(out)
