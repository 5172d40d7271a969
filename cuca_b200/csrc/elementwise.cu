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
  for (int i = threadIdx.x; i < E; i += blockDim.x) x[(size_t)row * E + i] = to_f32(src[i]);
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
// One block of 256 threads per output row; the reduction order depends only
// on E, so a row's result does not depend on what else is in the batch.
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int E, float eps) {
  __shared__ float red[8];
  pdl_trigger();
  pdl_wait();
  int orow = blockIdx.x;
  int irow = rows ? rows[orow] : orow;
  if (irow < 0) return;
  const float* xr = x + (size_t)irow * E;
  float s = 0.f;
  for (int i = threadIdx.x; i < E; i += 256) {
    float v = xr[i];
    s = fmaf(v, v, s);
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  float r = rsqrtf(tot / (float)E + eps);
  TO* o = out + (size_t)orow * E;
  for (int i = threadIdx.x; i < E; i += 256) o[i] = from_f32<TO>(xr[i] * r * to_f32(w[i]));
}

// out[r] = x[rows ? rows[r] : r] * rsqrt(mean(x^2) + eps) * w
CUCA_API int cuca_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype,
                          const int* rows, int n_rows, int E, float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(E > 0, "rmsnorm: bad width %d", E);
#define LAUNCH(TW, TO) \
  cuca_launch(rmsnorm_kernel<TW, TO>, dim3(n_rows), dim3(256), 0, stream, true, x, (const TW*)w, (TO*)out, rows, E, eps)
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
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const int* __restrict__ seq_of_row, const int* __restrict__ tables,
                                  int table_stride, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  int table_rows, int rot, T* __restrict__ kpool, T* __restrict__ vpool,
                                  int n_blocks, int bs, int nh, int nkv, int d, int* err) {
  pdl_trigger();
  pdl_wait();
  int row = blockIdx.x;
  int head = blockIdx.y;  // 0..nh-1 q, nh..nh+nkv-1 k, then v
  int seq = seq_of_row[row];
  if (seq < 0) return;
  int pos = positions[row];
  T* src = qkv + (size_t)row * (nh + 2 * nkv) * d + (size_t)head * d;
  bool is_v = head >= nh + nkv;
  bool is_k = !is_v && head >= nh;
  T* dst = nullptr;
  if (is_k || is_v) {
    int blk = pos >= 0 ? tables[(size_t)seq * table_stride + pos / bs] : -1;
    if (blk < 0 || blk >= n_blocks) {
      if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
      return;
    }
    int kvh = is_k ? head - nh : head - nh - nkv;
    dst = (is_k ? kpool : vpool) + (((size_t)blk * nkv + kvh) * bs + (pos % bs)) * d;
  }
  if (is_v) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
    return;
  }
  int half = rot / 2;
  bool in_table = pos >= 0 && pos < table_rows;
  if (!in_table && half > 0 && threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float c = in_table ? cos_t[(size_t)pos * half + i] : 1.f;
    float s = in_table ? sin_t[(size_t)pos * half + i] : 0.f;
    float a = to_f32(src[i]), b = to_f32(src[i + half]);
    T ra = from_f32<T>(a * c - b * s);
    T rb = from_f32<T>(a * s + b * c);
    if (is_k) {
      if (dst) { dst[i] = ra; dst[i + half] = rb; }
    } else {
      src[i] = ra; src[i + half] = rb;
    }
  }
  if (is_k && dst)
    for (int i = rot + threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
}

CUCA_API int cuca_rope_store(void* qkv, int dtype, const int* positions, const int* seq_of_row,
                             const int* tables, int table_stride, const float* cos_t, const float* sin_t,
                             int table_rows, int rot, void* kpool, void* vpool, int n_blocks, int bs,
                             int n_rows, int nh, int nkv, int d, int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "rope_store: rotary size %d does not fit head size %d", rot, d);
  CUCA_REQUIRE(bs > 0 && nh > 0 && nkv >= 0 && d > 0, "rope_store: bad sizes");
  dim3 grid(n_rows, nh + 2 * nkv);
  int threads = d / 2 >= 64 ? 64 : 32;
  if (dtype == CUCA_F32)
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
