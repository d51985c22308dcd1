"""The kernels' lane reduction adds each value exactly as the plain xor-shuffle tree 16, 8, 4, 2, 1 does: a small CUDA
program (tests/lane_reduce_check.cu, built here with nvcc) runs both on the same random values for 1 to 64 values per
lane and compares the bits. Row invariance alone would not notice a butterfly that is consistently different from the
stated order."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_the_value_splitting_butterfly_has_the_bits_of_the_plain_tree(tmp_path):
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    binary = str(tmp_path / "lane_reduce_check")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
                    os.path.join(HERE, "lane_reduce_check.cu"), "-o", binary], check=True)
    done = subprocess.run([binary], capture_output=True, text=True, timeout=120)
    assert done.returncode == 0 and done.stdout.strip().endswith("ok"), done.stdout + done.stderr
