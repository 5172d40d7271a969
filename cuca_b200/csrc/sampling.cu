// Token selection on the device. Greedy: the first maximum wins, as in
// src/provider/local/sampler.rs:44-54 of the reference.
#include "common.cuh"

namespace {

// Monotonic map of a float to an unsigned key (larger float, larger key); NaN maps to 0.
__device__ __forceinline__ unsigned ordered_key(float v) {
  if (v != v) return 0u;
  unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(256)
argmax_kernel(const float* __restrict__ logits, size_t row_stride, int V, int* __restrict__ out) {
  __shared__ unsigned long long red[8];
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  unsigned long long best = 0ull;
  for (int i = threadIdx.x; i < V; i += 256) {
    unsigned long long k = ((unsigned long long)ordered_key(row[i]) << 32) | (unsigned)(0xFFFFFFFFu - (unsigned)i);
    best = k > best ? k : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) best = red[i] > best ? red[i] : best;
    // a row without any value above -inf selects id 0, as the reference does
    unsigned key = (unsigned)(best >> 32);
    unsigned idx = 0xFFFFFFFFu - (unsigned)(best & 0xFFFFFFFFull);
    out[blockIdx.x] = (key <= ordered_key(-INFINITY) || best == 0ull) ? 0 : (int)idx;
  }
}

}  // namespace

// out[r] = index of the first maximum of logits[r, 0..V)
CUCA_API int cuca_argmax(const float* logits, size_t row_stride, int n_rows, int V, int* out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(V > 0, "argmax: empty vocabulary");
  argmax_kernel<<<n_rows, 256, 0, stream>>>(logits, row_stride, V, out);
  CUCA_CHECK_LAUNCH("argmax");
  return 0;
}
