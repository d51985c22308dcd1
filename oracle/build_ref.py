"""TEST INFRASTRUCTURE ONLY. Builds oracle/_ref/libdecode_gemv_ref.so: the reference's own CUDA source
(decode-gemv/decode_gemv_cuda/decode_gemv.cu, two files, no build system) compiled for sm_100a from where it lies in
the reference checkout, plus oracle/ref_shim.cu; oracle/_ref/libmma_rows_ref.so, the same for the reference's
activation quantizers (mma-rows/mma_rows_cuda/mma_rows.cu + fp4_mma.cu, plus oracle/ref_quant_shim.cu);
oracle/_ref/libint_block_ref.so for its SwiGLU (int-block-experts/int_block_cuda/int_block.cu, oracle/ref_swiglu_shim.cu); and
oracle/_ref/ref_host_check, a small program over the reference's header-only C++ host oracle (see build_host_check).
No reference source is copied; only binaries land in oracle/_ref/ (git-ignored, shipped to the GPU box). Without the
checkout this is a no-op and whatever was built earlier is used.

    CRIT_KERNELS_REFERENCE=path/to/reference python -m oracle.build_ref      (or the path as the first argument)
"""
import ctypes
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libdecode_gemv_ref.so")
NVCC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


REFERENCE = os.environ.get("CRIT_KERNELS_REFERENCE", "")   # the reference checkout; empty: use what is built
QUANT_LIB = os.path.join(OUT_DIR, "libmma_rows_ref.so")


def build(reference=REFERENCE, verbose=True):
    src_dir = os.path.join(reference, "decode-gemv", "decode_gemv_cuda")
    src = os.path.join(src_dir, "decode_gemv.cu")
    shim = os.path.join(HERE, "ref_shim.cu")
    if not reference or not os.path.exists(src):
        return os.path.exists(LIB)
    if os.path.exists(LIB) and os.path.getmtime(LIB) > max(os.path.getmtime(src), os.path.getmtime(shim)):
        return True
    os.makedirs(OUT_DIR, exist_ok=True)
    # -gencode ...100a: the reference switches to the hardware E2M1 conversion on this target (decode_gemv.cu:10-14)
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-Xcompiler", "-fvisibility=hidden", "-cudart", "static", f"-I{src_dir}", src, shim, "-o", LIB]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return True


def build_quantizers(reference=REFERENCE, verbose=True):
    """oracle/_ref/libmma_rows_ref.so: the reference's quantize_fp8_rows / quantize_nvfp4 kernels, unmodified."""
    src_dir = os.path.join(reference, "mma-rows", "mma_rows_cuda")
    sources = [os.path.join(src_dir, "mma_rows.cu"), os.path.join(src_dir, "fp4_mma.cu")]
    shim = os.path.join(HERE, "ref_quant_shim.cu")
    if not reference or not all(os.path.exists(f) for f in sources):
        return os.path.exists(QUANT_LIB)
    if os.path.exists(QUANT_LIB) and os.path.getmtime(QUANT_LIB) > max(os.path.getmtime(f) for f in sources + [shim]):
        return True
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-Xcompiler", "-fvisibility=hidden", "-cudart", "static", f"-I{src_dir}"] + sources + [shim, "-o", QUANT_LIB]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return True


def load_quantizers():
    """The reference's quantizer library, or None when it was never built."""
    if not os.path.exists(QUANT_LIB):
        return None
    lib = ctypes.CDLL(QUANT_LIB)
    p, i, ll, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.ref_quantize_fp8_rows.argtypes = [p, ll, i, i, p, ll, p, p]
    lib.ref_quantize_nvfp4.argtypes = [p, ll, i, i, f, f, p, p, p]
    lib.ref_quantize_fp8_rows.restype = lib.ref_quantize_nvfp4.restype = i
    return lib


SWIGLU_LIB = os.path.join(OUT_DIR, "libint_block_ref.so")


def build_swiglu(reference=REFERENCE, verbose=True):
    """oracle/_ref/libint_block_ref.so: the reference's int-block-experts kernels (one file), for its swiglu."""
    src_dir = os.path.join(reference, "int-block-experts", "int_block_cuda")
    src, shim = os.path.join(src_dir, "int_block.cu"), os.path.join(HERE, "ref_swiglu_shim.cu")
    if not reference or not os.path.exists(src):
        return os.path.exists(SWIGLU_LIB)
    if os.path.exists(SWIGLU_LIB) and os.path.getmtime(SWIGLU_LIB) > max(os.path.getmtime(src), os.path.getmtime(shim)):
        return True
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-Xcompiler", "-fvisibility=hidden", "-cudart", "static", f"-I{src_dir}", src, shim, "-o", SWIGLU_LIB]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return True


def load_swiglu():
    """The reference's SwiGLU library, or None when it was never built."""
    if not os.path.exists(SWIGLU_LIB):
        return None
    lib = ctypes.CDLL(SWIGLU_LIB)
    lib.ref_swiglu.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lib.ref_swiglu.restype = ctypes.c_int
    return lib


HOST_CHECK = os.path.join(OUT_DIR, "ref_host_check")


def build_host_check(reference=REFERENCE, verbose=True):
    """oracle/_ref/ref_host_check: oracle/ref_host_check.cpp over the reference's header-only C++ host oracle
    (fp8-block-rows/tests/order/row_fp8.h, fp8_block.h), included from where it lies. g++ -std=c++20, no other
    dependency. Used by tests/golden/make_golden.py only."""
    inc = os.path.join(reference, "fp8-block-rows", "tests", "order")
    src = os.path.join(HERE, "ref_host_check.cpp")
    if not reference or not os.path.exists(os.path.join(inc, "row_fp8.h")):
        return os.path.exists(HOST_CHECK)
    if os.path.exists(HOST_CHECK) and os.path.getmtime(HOST_CHECK) > os.path.getmtime(src):
        return True
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++20", "-O2", f"-I{inc}", src, "-o", HOST_CHECK]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return True


def load():
    """The reference library, or None when it was never built."""
    if not os.path.exists(LIB):
        return None
    lib = ctypes.CDLL(LIB)
    p, i = ctypes.c_void_p, ctypes.c_int
    lib.ref_enqueue_nvfp4.argtypes = [p, i, i, p, p, i, p, p, i, i, i, i, i, p]
    lib.ref_enqueue_fp8.argtypes = [p, i, i, p, p, p, p, i, i, i, i, i, p]
    lib.ref_enqueue_bf16.argtypes = [p, i, p, p, i, i, i, i, i, p]
    for f in (lib.ref_enqueue_nvfp4, lib.ref_enqueue_fp8, lib.ref_enqueue_bf16, lib.ref_hardware_decode):
        f.restype = i
    return lib


if __name__ == "__main__":
    where = sys.argv[1] if len(sys.argv) > 1 else REFERENCE
    if not where:
        raise SystemExit("give the reference checkout: CRIT_KERNELS_REFERENCE=<path> or the path as the argument")
    ok = build(where)
    build_quantizers(where)
    build_swiglu(where)
    build_host_check(where)
    print("built" if ok else "reference checkout not found; nothing built")
