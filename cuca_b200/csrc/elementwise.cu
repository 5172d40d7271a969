// Memory-bound kernels of the step: embedding gather, RMSNorm (with optional
// row gather), rotary encoding fused with the paged key/value write, SwiGLU.
// All arithmetic is 32-bit; the residual stream is 32-bit in every mode.
#include "common.cuh"
#include <stdarg.h>
#include <string>

static thread_local std::string g_last_error;
void cuca_set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}
CUCA_API const char* cuca_last_error() { return g_last_error.c_str(); }
CUCA_API int cuca_abi_version() { return 4; }

#include <stdlib.h>
static int g_pdl = -1;
bool cuca_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("CUCA_PDL");
    g_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pdl != 0;
}
// 1: kernels are launched as programmatic dependents of their predecessors (default); 0: plain stream order.
CUCA_API int cuca_set_pdl(int on) { g_pdl = on ? 1 : 0; return 0; }

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ x, int E, int V, int* err) {
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.x;
  int tok = tokens[row];
  if (tok < 0 || tok >= V) {
    if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
    for (int i = threadIdx.x; i < E; i += blockDim.x) x[(size_t)row * E + i] = 0.f;
    return;
  }
  const T* src = table + (size_t)tok * E;
  float* dst = x + (size_t)row * E;
  // 16 bytes per thread and round where the row allows it (a 4096-wide row in two rounds instead of sixteen rounds
  // of one value each: at eight rows the kernel is all latency)
  if (sizeof(T) == 2 && (E & 7) == 0 && (((size_t)src) & 15) == 0 && (((size_t)dst) & 15) == 0) {
    for (int i = threadIdx.x; i < (E >> 3); i += blockDim.x) {
      const uint4 w = reinterpret_cast<const uint4*>(src)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
      const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]),
                   d = __bfloat1622float2(h[3]);
      reinterpret_cast<float4*>(dst)[2 * i] = make_float4(a.x, a.y, b.x, b.y);
      reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
    }
    return;
  }
  if (sizeof(T) == 4 && (E & 3) == 0 && (((size_t)src) & 15) == 0 && (((size_t)dst) & 15) == 0) {
    for (int i = threadIdx.x; i < (E >> 2); i += blockDim.x)
      reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
    return;
  }
  for (int i = threadIdx.x; i < E; i += blockDim.x) dst[i] = to_f32(src[i]);
}

// Embedding rows of `tokens[n_rows]` into the 32-bit stream x[n_rows, E].
CUCA_API int cuca_embed(const void* table, int table_dtype, const int* tokens, float* x,
                        int n_rows, int E, int V, int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(E > 0 && V > 0, "embed: bad sizes E=%d V=%d", E, V);
  if (table_dtype == CUCA_F32)
    embed_kernel<float><<<n_rows, 256, 0, stream>>>((const float*)table, tokens, x, E, V, err);
  else if (table_dtype == CUCA_BF16)
    embed_kernel<__nv_bfloat16><<<n_rows, 256, 0, stream>>>((const __nv_bfloat16*)table, tokens, x, E, V, err);
  else
    CUCA_REQUIRE(false, "embed: unknown dtype %d", table_dtype);
  CUCA_CHECK_LAUNCH("embed");
  return 0;
}

// ---------------------------------------------------------------- RMSNorm
// One block per output row. Every thread takes four consecutive values at a time and the block is as wide as
// the row needs (up to 1024 threads), so all loads of a row are in flight together. The reduction order depends
// only on E, so a row's result does not depend on what else is in the batch.
static inline int norm_block(int E) {
  int t = ((E + 3) / 4 + 31) / 32 * 32;
  return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

__device__ __forceinline__ float block_sum_1024(float s, float* red) {
  s = warp_sum(s);
  const int nw = (blockDim.x + 31) >> 5;
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < nw; ++i) tot += red[i];
  return tot;
}

// four consecutive outputs with one store where the address allows it
__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
  if ((((size_t)o) & 15) == 0) *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
  else { o[0] = a; o[1] = b; o[2] = c; o[3] = d; }
}
__device__ __forceinline__ void store4(__nv_bfloat16* o, float a, float b, float c, float d) {
  if ((((size_t)o) & 7) == 0) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  } else {
    o[0] = __float2bfloat16_rn(a); o[1] = __float2bfloat16_rn(b); o[2] = __float2bfloat16_rn(c); o[3] = __float2bfloat16_rn(d);
  }
}

// PARTIAL: x[row] += sum over slices first (written back), see below.
// VL: value groups per thread and round. A block of B threads with VL groups each does exactly the arithmetic
// of a block of B * VL threads with one group each (thread t plays the lanes t, t + B, ...: the same warp
// shuffles, the same order across warps), so many-row launches can use narrow blocks with bit-equal results.
template <typename TW, typename TO, bool PARTIAL, int VL>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ partial, int n_slices,
                               size_t slice_stride, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int E, float eps) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  int orow = blockIdx.x;
  int irow = rows ? rows[orow] : orow;
  if (irow < 0) return;
  float* xr = x + (size_t)irow * E;
  const float* pr = PARTIAL ? partial + (size_t)irow * E : nullptr;
  TO* o = out + (size_t)orow * E;
  float s = 0.f;
  const bool vec = (E & 3) == 0 && (((size_t)xr) & 15) == 0 && (!PARTIAL || ((((size_t)pr) | (slice_stride * 4)) & 15) == 0);
  if (vec) {
    const int nvec = E >> 2;
    // One value group (four floats) per thread and round. The first two rounds (rows up to 8192 wide) stay in
    // registers between the two passes; wider rows are read again.
    auto take = [&](int i) {
      float4 v = reinterpret_cast<const float4*>(xr)[i];
      if (PARTIAL) {
        for (int k0 = 0; k0 < n_slices; k0 += 4) {  // four slices' loads in flight at once, added in slice order
          float4 q[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            q[u] = k0 + u < n_slices ? __ldcg(reinterpret_cast<const float4*>(pr + (k0 + u) * slice_stride) + i)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < 4; ++u) { v.x += q[u].x; v.y += q[u].y; v.z += q[u].z; v.w += q[u].w; }
        }
        reinterpret_cast<float4*>(xr)[i] = v;
      }
      s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s); s = fmaf(v.z, v.z, s); s = fmaf(v.w, v.w, s);
      return v;
    };
    auto put = [&](int i, float4 v, float r) {
      const int e = i << 2;
      const float w0 = to_f32(w[e]), w1 = to_f32(w[e + 1]), w2 = to_f32(w[e + 2]), w3 = to_f32(w[e + 3]);
      store4(o + e, v.x * r * w0, v.y * r * w1, v.z * r * w2, v.w * r * w3);
    };
    const int VB = blockDim.x * VL;  // virtual block width
    float4 v0[VL], v1[VL];
    float sk[VL];
#pragma unroll
    for (int k = 0; k < VL; ++k) {
      const int i0 = threadIdx.x + blockDim.x * k, i1 = i0 + VB;
      s = 0.f;
      v0[k] = v1[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i0 < nvec) v0[k] = take(i0);
      if (i1 < nvec) v1[k] = take(i1);
      for (int i = i1 + VB; i < nvec; i += VB) take(i);
      sk[k] = s;
    }
    // reduction in the order of the virtual block: warp sums, then the warps in ascending order
    const int real_warps = blockDim.x >> 5;
#pragma unroll
    for (int k = 0; k < VL; ++k) {
      float wsum = warp_sum(sk[k]);
      if ((threadIdx.x & 31) == 0) red[(threadIdx.x >> 5) + real_warps * k] = wsum;
    }
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < real_warps * VL; ++i) tot += red[i];
    const float r = rsqrtf(tot / (float)E + eps);
#pragma unroll
    for (int k = 0; k < VL; ++k) {
      const int i0 = threadIdx.x + blockDim.x * k, i1 = i0 + VB;
      if (i0 < nvec) put(i0, v0[k], r);
      if (i1 < nvec) put(i1, v1[k], r);
      for (int i = i1 + VB; i < nvec; i += VB) put(i, reinterpret_cast<const float4*>(xr)[i], r);
    }
  } else {
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
      float v = xr[i];
      if (PARTIAL) {
        for (int k = 0; k < n_slices; ++k) v += __ldcg(pr + k * slice_stride + i);
        xr[i] = v;
      }
      s = fmaf(v, v, s);
    }
    float r = rsqrtf(block_sum_1024(s, red) / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = from_f32<TO>(xr[i] * r * to_f32(w[i]));
  }
}

// out[r] = x[rows ? rows[r] : r] * rsqrt(mean(x^2) + eps) * w
CUCA_API int cuca_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype,
                          const int* rows, int n_rows, int E, float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(E > 0, "rmsnorm: bad width %d", E);
  float* xm = const_cast<float*>(x);  // not written without PARTIAL
  // many rows: a quarter of the threads per block, four value groups each (bit-equal to the wide block)
  const bool narrow = norm_block(E) == 1024 && n_rows >= 64 && (E & 3) == 0;
#define LAUNCH(TW, TO)                                                                                          \
  do {                                                                                                          \
    if (narrow)                                                                                                 \
      cuca_launch(rmsnorm_kernel<TW, TO, false, 4>, dim3(n_rows), dim3(256), 0, stream, true, xm,               \
                  (const float*)nullptr, 0, (size_t)0, (const TW*)w, (TO*)out, rows, E, eps);                   \
    else                                                                                                        \
      cuca_launch(rmsnorm_kernel<TW, TO, false, 1>, dim3(n_rows), dim3(norm_block(E)), 0, stream, true, xm,     \
                  (const float*)nullptr, 0, (size_t)0, (const TW*)w, (TO*)out, rows, E, eps);                   \
  } while (0)
  if (w_dtype == CUCA_F32 && out_dtype == CUCA_F32) LAUNCH(float, float);
  else if (w_dtype == CUCA_F32 && out_dtype == CUCA_BF16) LAUNCH(float, __nv_bfloat16);
  else if (w_dtype == CUCA_BF16 && out_dtype == CUCA_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == CUCA_BF16 && out_dtype == CUCA_F32) LAUNCH(__nv_bfloat16, float);
  else CUCA_REQUIRE(false, "rmsnorm: unknown dtypes %d %d", w_dtype, out_dtype);
#undef LAUNCH
  CUCA_CHECK_LAUNCH("rmsnorm");
  return 0;
}

// ---------------------------------------------------------------- rotary + paged K/V write
// qkv: [T, (nh + 2 nkv) d]. q and k heads are rotated (first `rot` values of a
// head, pairs (i, i + rot/2)); q in place, k and v go to their page (nkv = 0:
// the layer owns no keys, only q is rotated):
// pool[block][kv head][row in block][d], block = table[seq][pos / bs].
template <typename T>
__global__ void __launch_bounds__(256)
rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                  const int* __restrict__ seq_of_row, const int* __restrict__ tables,
                  int table_stride, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                  int table_rows, int rot, T* __restrict__ kpool, T* __restrict__ vpool,
                  int n_blocks, int bs, int nh, int nkv, int d, int* err) {
  // one block per row; its threads walk all heads of the row: rotated pairs, pass-through values, v copies
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int seq = seq_of_row[row];
  if (seq < 0) return;
  const int pos = positions[row];
  const int half = rot / 2;
  T* base = qkv + (size_t)row * (nh + 2 * nkv) * d;
  long long page_off = -1;  // offset of this position's row in a pool, per kv head add kvh * bs * d
  if (nkv > 0) {
    int blk = pos >= 0 ? tables[(size_t)seq * table_stride + pos / bs] : -1;
    if (blk < 0 || blk >= n_blocks) {
      if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
    } else {
      page_off = ((long long)blk * nkv * bs + (pos % bs)) * d;
    }
  }
  const bool in_table = pos >= 0 && pos < table_rows;
  if (!in_table && half > 0 && threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
  const float* cr = cos_t + (size_t)(in_table ? pos : 0) * half;
  const float* sr = sin_t + (size_t)(in_table ? pos : 0) * half;
  // q and k heads: `half` rotated pairs + (d - rot) values that pass through
  const int per_head = half + (d - rot);
  const int qk_items = (nh + nkv) * per_head;
  for (int idx = threadIdx.x; idx < qk_items; idx += blockDim.x) {
    const int head = idx / per_head, i = idx % per_head;
    T* src = base + (size_t)head * d;
    T* dst = nullptr;  // k heads go to their page; q heads are rotated in place
    const bool is_k = head >= nh;
    if (is_k) {
      if (page_off < 0) continue;
      dst = kpool + page_off + (size_t)(head - nh) * bs * d;
    }
    if (i < half) {
      float c = in_table ? cr[i] : 1.f, sn = in_table ? sr[i] : 0.f;
      float a = to_f32(src[i]), b = to_f32(src[i + half]);
      T ra = from_f32<T>(a * c - b * sn), rb = from_f32<T>(a * sn + b * c);
      if (is_k) { dst[i] = ra; dst[i + half] = rb; }
      else { src[i] = ra; src[i + half] = rb; }
    } else if (is_k) {
      const int e = rot + (i - half);
      dst[e] = src[e];
    }
  }
  if (nkv > 0 && page_off >= 0) {
    const T* vsrc = base + (size_t)(nh + nkv) * d;
    for (int idx = threadIdx.x; idx < nkv * d; idx += blockDim.x) {
      const int kvh = idx / d, e = idx % d;
      vpool[page_off + (size_t)kvh * bs * d + e] = vsrc[idx];
    }
  }
}

// The same for bf16 rows whose heads are rotated whole (rot = d) with d a multiple of 16: a thread takes eight
// pairs (16 bytes of each half of a head, eight cosines and sines) or 16 bytes of v at a time. Same arithmetic,
// element by element, as the kernel above.
__global__ void __launch_bounds__(256)
rope_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_row, const int* __restrict__ tables, int table_stride,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_rows,
                      __nv_bfloat16* __restrict__ kpool, __nv_bfloat16* __restrict__ vpool, int n_blocks, int bs,
                      int nh, int nkv, int d, int* err) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int seq = seq_of_row[row];
  if (seq < 0) return;
  const int pos = positions[row];
  const int half = d / 2;
  __nv_bfloat16* base = qkv + (size_t)row * (nh + 2 * nkv) * d;
  long long page_off = -1;
  if (nkv > 0) {
    int blk = pos >= 0 ? tables[(size_t)seq * table_stride + pos / bs] : -1;
    if (blk < 0 || blk >= n_blocks) {
      if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
    } else {
      page_off = ((long long)blk * nkv * bs + (pos % bs)) * d;
    }
  }
  const bool in_table = pos >= 0 && pos < table_rows;
  if (!in_table && threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
  const float* cr = cos_t + (size_t)(in_table ? pos : 0) * half;
  const float* sr = sin_t + (size_t)(in_table ? pos : 0) * half;
  const int per_head = half / 8;  // items of eight pairs
  const int qk_items = (nh + nkv) * per_head;
  const int v_items = (nkv > 0 && page_off >= 0) ? nkv * d / 8 : 0;
  for (int idx = threadIdx.x; idx < qk_items + v_items; idx += blockDim.x) {
    if (idx >= qk_items) {
      const int e = (idx - qk_items) * 8, kvh = e / d;
      const uint4 v = *reinterpret_cast<const uint4*>(base + (size_t)(nh + nkv) * d + e);
      *reinterpret_cast<uint4*>(vpool + page_off + (size_t)kvh * bs * d + (e - kvh * d)) = v;
      continue;
    }
    const int head = idx / per_head, i = (idx - head * per_head) * 8;
    __nv_bfloat16* src = base + (size_t)head * d;
    const bool is_k = head >= nh;
    if (is_k && page_off < 0) continue;
    __nv_bfloat16* dst = is_k ? kpool + page_off + (size_t)(head - nh) * bs * d : src;
    uint4 ua = *reinterpret_cast<const uint4*>(src + i), ub = *reinterpret_cast<const uint4*>(src + i + half);
    float c[8], sn[8];
    if (in_table) {
      *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cr + i);
      *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cr + i + 4);
      *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sr + i);
      *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sr + i + 4);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { c[j] = 1.f; sn[j] = 0.f; }
    }
    const __nv_bfloat16* pa = reinterpret_cast<const __nv_bfloat16*>(&ua);
    const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&ub);
    uint4 oa, ob;
    __nv_bfloat16* qa = reinterpret_cast<__nv_bfloat16*>(&oa);
    __nv_bfloat16* qb = reinterpret_cast<__nv_bfloat16*>(&ob);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = __bfloat162float(pa[j]), b = __bfloat162float(pb[j]);
      qa[j] = __float2bfloat16_rn(a * c[j] - b * sn[j]);
      qb[j] = __float2bfloat16_rn(a * sn[j] + b * c[j]);
    }
    *reinterpret_cast<uint4*>(dst + i) = oa;
    *reinterpret_cast<uint4*>(dst + i + half) = ob;
  }
}

CUCA_API int cuca_rope_store(void* qkv, int dtype, const int* positions, const int* seq_of_row,
                             const int* tables, int table_stride, const float* cos_t, const float* sin_t,
                             int table_rows, int rot, void* kpool, void* vpool, int n_blocks, int bs,
                             int n_rows, int nh, int nkv, int d, int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "rope_store: rotary size %d does not fit head size %d", rot, d);
  CUCA_REQUIRE(bs > 0 && nh > 0 && nkv >= 0 && d > 0, "rope_store: bad sizes");
  dim3 grid(n_rows);
  int threads = 256;
  const bool aligned = (((uintptr_t)qkv | (uintptr_t)kpool | (uintptr_t)vpool | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) == 0;
  if (dtype == CUCA_BF16 && rot == d && d % 16 == 0 && aligned)
    cuca_launch(rope_store_vec_kernel, grid, dim3(threads), 0, stream, true, (__nv_bfloat16*)qkv, positions, seq_of_row,
                tables, table_stride, cos_t, sin_t, table_rows, (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, n_blocks,
                bs, nh, nkv, d, err);
  else if (dtype == CUCA_F32)
    cuca_launch(rope_store_kernel<float>, grid, dim3(threads), 0, stream, true, (float*)qkv, positions, seq_of_row,
                tables, table_stride, cos_t, sin_t, table_rows, rot, (float*)kpool, (float*)vpool, n_blocks, bs, nh,
                nkv, d, err);
  else if (dtype == CUCA_BF16)
    cuca_launch(rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, true, (__nv_bfloat16*)qkv,
                positions, seq_of_row, tables, table_stride, cos_t, sin_t, table_rows, rot, (__nv_bfloat16*)kpool,
                (__nv_bfloat16*)vpool, n_blocks, bs, nh, nkv, d, err);
  else
    CUCA_REQUIRE(false, "rope_store: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("rope_store");
  return 0;
}

// ---------------------------------------------------------------- SwiGLU (unfused form)
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int ff, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  size_t r = i / ff;
  int j = (int)(i % ff);
  float g = to_f32(gu[r * 2 * ff + j]);
  float u = to_f32(gu[r * 2 * ff + ff + j]);
  out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

// out[r, j] = silu(gu[r, j]) * gu[r, ff + j]
CUCA_API int cuca_swiglu(const void* gu, void* out, int dtype, int n_rows, int ff, cudaStream_t stream) {
  size_t total = (size_t)n_rows * ff;
  if (total == 0) return 0;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == CUCA_F32) swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)out, ff, total);
  else if (dtype == CUCA_BF16)
    swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, ff, total);
  else CUCA_REQUIRE(false, "swiglu: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("swiglu");
  return 0;
}

// ---------------------------------------------------------------- stream += delta
template <typename T>
__global__ void add_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] += to_f32(delta[i]);
}

CUCA_API int cuca_add_to_stream(float* x, const void* delta, int dtype, size_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == CUCA_F32) add_kernel<float><<<blocks, 256, 0, stream>>>(x, (const float*)delta, total);
  else if (dtype == CUCA_BF16) add_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(x, (const __nv_bfloat16*)delta, total);
  else CUCA_REQUIRE(false, "add_to_stream: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("add_to_stream");
  return 0;
}

// ---------------------------------------------------------------- table updates
__global__ void scatter_int_kernel(int* __restrict__ dst, const int* __restrict__ idx, const int* __restrict__ val,
                                   int n, long long limit) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && idx[i] >= 0 && (long long)idx[i] < limit) dst[idx[i]] = val[i];
}

// dst[idx[i]] = val[i] for i < n; entries outside 0..limit-1 are skipped
CUCA_API int cuca_scatter_int(int* dst, const int* idx, const int* val, int n, long long limit, cudaStream_t stream) {
  if (n == 0) return 0;
  scatter_int_kernel<<<(n + 255) / 256, 256, 0, stream>>>(dst, idx, val, n, limit);
  CUCA_CHECK_LAUNCH("scatter_int");
  return 0;
}

// ---------------------------------------------------------------- consumers of partial sums (decode)
// A contraction over few tokens is cut along K over several CTAs. Instead of adding the slices up itself (a
// second pass through global memory at the end of a short kernel), it leaves them as [slice][row][feature]
// 32-bit sums, and the next kernel, which reads every value anyway, adds them in slice order.

// x[row] += sum over slices; out[orow] = RMSNorm(x[row]) * w (the RMSNorm kernel above with PARTIAL).
CUCA_API int cuca_add_partials_rmsnorm(float* x, const float* partial, int n_slices, size_t slice_stride,
                                       const float* w, void* out, int out_dtype, const int* rows, int n_rows, int E,
                                       float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(E > 0 && n_slices >= 1, "add_partials_rmsnorm: bad sizes");
  if (out_dtype == CUCA_BF16)
    cuca_launch(rmsnorm_kernel<float, __nv_bfloat16, true, 1>, dim3(n_rows), dim3(norm_block(E)), 0, stream, true, x,
                partial, n_slices, slice_stride, w, (__nv_bfloat16*)out, rows, E, eps);
  else if (out_dtype == CUCA_F32)
    cuca_launch(rmsnorm_kernel<float, float, true, 1>, dim3(n_rows), dim3(norm_block(E)), 0, stream, true, x, partial,
                n_slices, slice_stride, w, (float*)out, rows, E, eps);
  else
    CUCA_REQUIRE(false, "add_partials_rmsnorm: unknown dtype %d", out_dtype);
  CUCA_CHECK_LAUNCH("add_partials_rmsnorm");
  return 0;
}

// x += sum over slices: for a reader of the stream that does not add the slices itself.
__global__ void add_partials_kernel(float* __restrict__ x, const float* __restrict__ partial, int n_slices,
                                    size_t slice_stride, size_t total) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = x[i];
  for (int k = 0; k < n_slices; ++k) v += __ldcg(partial + k * slice_stride + i);
  x[i] = v;
}

CUCA_API int cuca_add_partials(float* x, const float* partial, int n_slices, size_t slice_stride, size_t total,
                               cudaStream_t stream) {
  if (total == 0) return 0;
  cuca_launch(add_partials_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, true, x, partial,
              n_slices, slice_stride, total);
  CUCA_CHECK_LAUNCH("add_partials");
  return 0;
}

// The q/k/v projection arrives as partial sums [slice][row][(nh + 2 nkv) d]: add them (and the bias), rotate q
// and k in 32-bit, write q as bf16 to q_out[row][nh d] and k, v to their pages.
__global__ void rope_store_partial_kernel(const float* __restrict__ partial, int n_slices, size_t slice_stride,
                                          const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ q_out,
                                          const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                                          const int* __restrict__ tables, int table_stride,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          int table_rows, int rot, __nv_bfloat16* __restrict__ kpool,
                                          __nv_bfloat16* __restrict__ vpool, int n_blocks, int bs, int nh, int nkv,
                                          int d, int* err) {
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.x;
  int head = blockIdx.y;
  int seq = seq_of_row[row];
  if (seq < 0) return;
  int pos = positions[row];
  const size_t width = (size_t)(nh + 2 * nkv) * d;
  const float* src = partial + (size_t)row * width + (size_t)head * d;
  const __nv_bfloat16* b = bias ? bias + (size_t)head * d : nullptr;
  auto value = [&](int i) {
    float v = b ? __bfloat162float(b[i]) : 0.f;
    for (int k0 = 0; k0 < n_slices; k0 += 4) {  // four slices' loads in flight at once, added in slice order
      float q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = k0 + u < n_slices ? __ldcg(src + (k0 + u) * slice_stride + i) : 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) v += q[u];
    }
    return v;
  };
  bool is_v = head >= nh + nkv;
  bool is_k = !is_v && head >= nh;
  __nv_bfloat16* dst;
  if (is_k || is_v) {
    int blk = pos >= 0 ? tables[(size_t)seq * table_stride + pos / bs] : -1;
    if (blk < 0 || blk >= n_blocks) {
      if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
      return;
    }
    int kvh = is_k ? head - nh : head - nh - nkv;
    dst = (is_k ? kpool : vpool) + (((size_t)blk * nkv + kvh) * bs + (pos % bs)) * d;
  } else {
    dst = q_out + (size_t)row * nh * d + (size_t)head * d;
  }
  if (is_v) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = __float2bfloat16_rn(value(i));
    return;
  }
  int half = rot / 2;
  bool in_table = pos >= 0 && pos < table_rows;
  if (!in_table && half > 0 && threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float c = in_table ? cos_t[(size_t)pos * half + i] : 1.f;
    float s = in_table ? sin_t[(size_t)pos * half + i] : 0.f;
    float a = value(i), bb = value(i + half);
    dst[i] = __float2bfloat16_rn(a * c - bb * s);
    dst[i + half] = __float2bfloat16_rn(a * s + bb * c);
  }
  for (int i = rot + threadIdx.x; i < d; i += blockDim.x) dst[i] = __float2bfloat16_rn(value(i));
}

CUCA_API int cuca_rope_store_partial(const float* partial, int n_slices, size_t slice_stride, const void* bias,
                                     void* q_out, const int* positions, const int* seq_of_row, const int* tables,
                                     int table_stride, const float* cos_t, const float* sin_t, int table_rows,
                                     int rot, void* kpool, void* vpool, int n_blocks, int bs, int n_rows, int nh,
                                     int nkv, int d, int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "rope_store_partial: rotary size %d does not fit head size %d", rot, d);
  CUCA_REQUIRE(bs > 0 && nh > 0 && nkv >= 0 && d > 0 && n_slices >= 1, "rope_store_partial: bad sizes");
  dim3 grid(n_rows, nh + 2 * nkv);
  int threads = d / 2 >= 64 ? 64 : 32;
  cuca_launch(rope_store_partial_kernel, grid, dim3(threads), 0, stream, true, partial, n_slices, slice_stride,
              (const __nv_bfloat16*)bias, (__nv_bfloat16*)q_out, positions, seq_of_row, tables, table_stride, cos_t,
              sin_t, table_rows, rot, (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, n_blocks, bs, nh, nkv, d, err);
  CUCA_CHECK_LAUNCH("rope_store_partial");
  return 0;
}

// ---------------------------------------------------------------- random weights
// Element i of a tensor is a function of (key, i) alone, so the same values come out on the host and on the
// device, whole or in pieces: outputs 3i, 3i+1, 3i+2 of a SplitMix64 stream that starts at `key` give twelve
// 16-bit fields whose sum is near-normal (Irwin-Hall); v = (2 sum - 12 * 65535) * scale, then mean + v, each a
// single 32-bit rounding (no fused multiply-add, so the host restates it exactly).
__device__ __forceinline__ unsigned long long splitmix_out(unsigned long long state) {
  unsigned long long z = state;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, size_t n, size_t first, unsigned long long key, float mean,
                                     float scale) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long e = first + i;
  int sum = 0;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    unsigned long long h = splitmix_out(key + (3ull * e + (unsigned long long)j + 1ull) * 0x9E3779B97F4A7C15ull);
    sum += (int)(h & 0xFFFF) + (int)((h >> 16) & 0xFFFF) + (int)((h >> 32) & 0xFFFF) + (int)(h >> 48);
  }
  float v = __fadd_rn(mean, __fmul_rn((float)(2 * sum - 12 * 65535), scale));
  out[i] = from_f32<T>(v);
}

// out[i] = mean + normal(first + i) * std for i < n (`first`: the element number out[0] has in its tensor).
CUCA_API int cuca_random_normal(void* out, int dtype, size_t n, size_t first, unsigned long long key, float mean,
                                float scale, cudaStream_t stream) {
  if (n == 0) return 0;
  CUCA_REQUIRE(n < ((size_t)1 << 40), "random_normal: %zu elements in one call", n);
  unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == CUCA_F32)
    random_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, first, key, mean, scale);
  else if (dtype == CUCA_BF16)
    random_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, first, key, mean, scale);
  else
    CUCA_REQUIRE(false, "random_normal: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("random_normal");
  return 0;
}
