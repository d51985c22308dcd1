// Test program (compiled by tests/test_lane_reduce_gpu.py with nvcc): the kernels' lane reduction (dg::LaneReduce, a
// value-splitting butterfly) against the plain xor-shuffle tree 16, 8, 4, 2, 1 applied to every value on its own,
// on random FP32 values of mixed magnitudes, compared bit for bit, for V values per lane, V = 1 .. 64.
#include <cstdio>
#include <cstdint>
#include <vector>

#include "../crit_kernels_b200/csrc/dg_kernel.cuh"

template <int V>
__global__ void reduce_both(const float* in, float* fast, float* plain) {   // one warp; in [32][V]
  const int lane = threadIdx.x;
  float val[V], tree[V];
#pragma unroll
  for (int v = 0; v < V; ++v) val[v] = tree[v] = in[lane * V + v];
#pragma unroll
  for (int v = 0; v < V; ++v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tree[v] += __shfl_xor_sync(0xffffffffu, tree[v], o);
    if (lane == 0) plain[v] = tree[v];
  }
  constexpr int NOUT = (V + 31) / 32;
  float total[NOUT];
  dg::LaneReduce<V, 16, NOUT>::run(val, lane, total);
#pragma unroll
  for (int i = 0; i < NOUT; ++i) {
    const int v = dg::lane_value<V>(lane, i);
    if (v >= 0) fast[v] = total[i];
  }
}

template <int V>
bool check(const std::vector<float>& host, float* in, float* fast, float* plain) {
  cudaMemcpy(in, host.data(), 32 * V * sizeof(float), cudaMemcpyHostToDevice);
  cudaMemset(fast, 0xff, 64 * sizeof(float));
  cudaMemset(plain, 0x00, 64 * sizeof(float));
  reduce_both<V><<<1, 32>>>(in, fast, plain);
  uint32_t a[64], b[64];
  if (cudaMemcpy(a, fast, V * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
  if (cudaMemcpy(b, plain, V * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
  for (int v = 0; v < V; ++v)
    if (a[v] != b[v]) {
      printf("V=%d value %d: butterfly %08x, tree %08x\n", V, v, a[v], b[v]);
      return false;
    }
  return true;
}

template <int V>
bool all(const std::vector<float>& host, float* in, float* fast, float* plain) {
  if constexpr (V == 0) return true;
  else return check<V>(host, in, fast, plain) && all<V - 1>(host, in, fast, plain);
}

int main() {
  std::vector<float> host(32 * 64);
  uint32_t state = 12345u;
  for (float& x : host) {                       // values whose sums round: mixed signs and exponents
    state = state * 1664525u + 1013904223u;
    const int e = (int)((state >> 8) % 24) - 12;
    state = state * 1664525u + 1013904223u;
    x = ((int)(state >> 9) - (1 << 22)) * (1.0f / (1 << 22)) * (float)(1u << (e + 12)) / 4096.0f;
  }
  float *in, *fast, *plain;
  cudaMalloc(&in, 32 * 64 * sizeof(float));
  cudaMalloc(&fast, 64 * sizeof(float));
  cudaMalloc(&plain, 64 * sizeof(float));
  const bool ok = all<64>(host, in, fast, plain) && cudaDeviceSynchronize() == cudaSuccess;
  printf(ok ? "ok\n" : "FAIL\n");
  return ok ? 0 : 1;
}
