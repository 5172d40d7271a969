// Paged causal grouped-query attention, plain form: one warp per (row, query
// head), keys in tiles of 32 absolute positions with an online softmax. It
// serves the true 32-bit path and is the fall-back of the bfloat16 path for
// head sizes its tensor-core kernels refuse. A row's arithmetic depends only
// on its own position and keys: tiles start at multiples of 32 key positions,
// so cutting a prompt or batching it differently gives the same bits.
#include "common.cuh"
#include <math.h>

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ kpool, const T* __restrict__ vpool, int n_blocks, int bs,
                         const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                         const int* __restrict__ tables, int table_stride, int nh, int nkv, int d,
                         float scale, int window, int* err) {
  extern __shared__ float qs[];  // [4][d]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y;
  const int head = blockIdx.x * 4 + warp;
  const int seq = seq_of_row[row];
  if (seq < 0 || head >= nh) return;
  const int P = positions[row];
  const int kvh = head / (nh / nkv);
  float* qv = qs + warp * d;
  const T* qrow = q + (size_t)row * q_stride + (size_t)head * d;
  for (int i = lane; i < d; i += 32) qv[i] = to_f32(qrow[i]);
  __syncwarp();

  int lo = 0;
  if (window > 0 && P - (window - 1) > 0) lo = P - (window - 1);
  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  const int* table = tables + (size_t)seq * table_stride;

  for (int t0 = (lo / 32) * 32; t0 <= P; t0 += 32) {
    int kp = t0 + lane;
    bool valid = kp >= lo && kp <= P;
    long long base = -1;
    if (valid) {
      int blk = table[kp / bs];
      if (blk < 0 || blk >= n_blocks) {
        if (err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
        valid = false;
      } else {
        base = (((long long)blk * nkv + kvh) * bs + (kp % bs)) * d;
      }
    }
    float s = -INFINITY;
    if (valid) {
      const T* kr = kpool + base;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qv[i], to_f32(kr[i]), dot);
      s = dot * scale;
    }
    float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;  // a tile with no readable key
    float p = valid ? expf(s - m_new) : 0.f;
    float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] *= corr;
    for (int j = 0; j < 32; ++j) {
      float pj = __shfl_sync(0xffffffffu, p, j);
      long long bj = __shfl_sync(0xffffffffu, base, j);
      if (bj < 0) continue;
      const T* vr = vpool + bj;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        int dim = c * 32 + lane;
        if (dim < d) acc[c] = fmaf(pj, to_f32(vr[dim]), acc[c]);
      }
    }
    m = m_new;
  }
  float inv = l > 0.f ? 1.f / l : 0.f;
  T* o = out + (size_t)row * out_stride + (size_t)head * d;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    int dim = c * 32 + lane;
    if (dim < d) o[dim] = from_f32<T>(acc[c] * inv);
  }
}

}  // namespace

// The largest head size any attention kernel of this library takes (the plain kernel's; the tensor-core forms take
// fewer). A part asks at construction, so that a model with larger heads is refused when it is built, not at its
// first step.
CUCA_API int cuca_attention_max_head_dim() { return 256; }

// q: rows of `q_stride` elements whose first nh*d hold the (rotated) query
// heads; out: [n_rows, out_stride]; pools [n_blocks][nkv][bs][d]. Row r is at
// position positions[r] of sequence seq_of_row[r] (< 0: padding, skipped) and
// sees keys max(0, P - window + 1)..P of that sequence (window 0: all).
CUCA_API int cuca_attention_generic(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                    const void* kpool, const void* vpool, int n_blocks, int bs,
                                    const int* positions, const int* seq_of_row, const int* tables,
                                    int table_stride, int n_rows, int nh, int nkv, int d, float scale,
                                    int window, int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(d > 0 && d <= cuca_attention_max_head_dim(), "attention: head size %d is outside 1..%d", d, cuca_attention_max_head_dim());
  CUCA_REQUIRE(nkv > 0 && nh % nkv == 0, "attention: %d query heads do not group over %d key heads", nh, nkv);
  CUCA_REQUIRE(n_rows <= 65535, "attention: %d rows in one step exceed the launch limit 65535", n_rows);
  dim3 grid((nh + 3) / 4, n_rows);
  size_t smem = (size_t)4 * d * sizeof(float);
  if (dtype == CUCA_F32)
    cuca_launch(attention_generic_kernel<float>, grid, dim3(128), smem, stream, true, (const float*)q, q_stride,
                (float*)out, out_stride, (const float*)kpool, (const float*)vpool, n_blocks, bs, positions,
                seq_of_row, tables, table_stride, nh, nkv, d, scale, window, err);
  else if (dtype == CUCA_BF16)
    cuca_launch(attention_generic_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, true,
                (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)kpool,
                (const __nv_bfloat16*)vpool, n_blocks, bs, positions, seq_of_row, tables, table_stride, nh, nkv, d,
                scale, window, err);
  else
    CUCA_REQUIRE(false, "attention: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("attention_generic");
  return 0;
}
