// Plain CUDA-core contraction out = A[M,K] * W[N,K]^T with 32-bit accumulation:
// the true 32-bit path of every projection, and the bfloat16 path's stand-in
// for shapes the tensor-core kernel refuses. Each output element sums its K
// products in ascending order with fused multiply-adds, whatever M and the tile
// variant are, so a row's result never depends on the rest of the batch.
//
// Epilogues: store (optional bias), add into the 32-bit residual stream, or
// SwiGLU over a stacked [gate; up] weight (rows 0..N-1 gate, N..2N-1 up).
#include "common.cuh"

#define EPI_STORE 0
#define EPI_RESIDUAL 1
#define EPI_SWIGLU 2

namespace {

constexpr int BK = 16;
constexpr int BN = 64;

template <typename TI, typename TO, int TM, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* __restrict__ A, const TI* __restrict__ W, const TI* __restrict__ bias,
                 TO* __restrict__ out, int M, int N, int K, int lda, int ldo) {
  constexpr int BM = 16 * TM;
  constexpr bool DUAL = EPI == EPI_SWIGLU;
  __shared__ float As[BK][BM + 1];
  __shared__ float Bs[DUAL ? 2 : 1][BK][BN + 1];
  pdl_trigger();
  pdl_wait();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][4];
  float acc2[DUAL ? TM : 1][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll
  for (int i = 0; i < (DUAL ? TM : 1); ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc2[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // A tile: BM x BK
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      int r = e / BK, c = e % BK;
      int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
    }
    for (int e = threadIdx.x; e < BN * BK; e += 256) {
      int r = e / BK, c = e % BK;
      int gn = n0 + r, gk = k0 + c;
      bool ok = gn < N && gk < K;
      Bs[0][c][r] = ok ? to_f32(W[(size_t)gn * K + gk]) : 0.f;
      if (DUAL) Bs[DUAL ? 1 : 0][c][r] = ok ? to_f32(W[(size_t)(gn + N) * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[0][kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      if (DUAL) {
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[DUAL ? 1 : 0][kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc2[DUAL ? i : 0][j] = fmaf(a[i], b[j], acc2[DUAL ? i : 0][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      size_t o = (size_t)gm * ldo + gn;
      if (EPI == EPI_SWIGLU) {
        float u = acc2[DUAL ? i : 0][j];
        out[o] = from_f32<TO>(v / (1.f + expf(-v)) * u);
      } else {
        if (bias) v += to_f32(bias[gn]);
        if (EPI == EPI_RESIDUAL) out[o] = from_f32<TO>(to_f32(out[o]) + v);
        else out[o] = from_f32<TO>(v);
      }
    }
  }
}

template <typename TI, typename TO, int EPI>
void launch(const void* A, const void* W, const void* bias, void* out, int M, int N, int K, int lda, int ldo,
            cudaStream_t stream) {
  if (M <= 16) {
    dim3 grid((N + BN - 1) / BN, (M + 15) / 16);
    cuca_launch(gemm_simt_kernel<TI, TO, 1, EPI>, grid, dim3(256), 0, stream, true, (const TI*)A, (const TI*)W,
                (const TI*)bias, (TO*)out, M, N, K, lda, ldo);
  } else {
    dim3 grid((N + BN - 1) / BN, (M + 63) / 64);
    cuca_launch(gemm_simt_kernel<TI, TO, 4, EPI>, grid, dim3(256), 0, stream, true, (const TI*)A, (const TI*)W,
                (const TI*)bias, (TO*)out, M, N, K, lda, ldo);
  }
}

}  // namespace

// out = epilogue(A[M,K] W[N,K]^T). in_dtype: A, W and bias; out_dtype: out.
// epilogue 0 store, 1 out (32-bit) += result, 2 SwiGLU (W has 2N rows).
CUCA_API int cuca_gemm_simt(const void* A, const void* W, const void* bias, void* out, int in_dtype, int out_dtype,
                   int M, int N, int K, int lda, int ldo, int epilogue, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  CUCA_REQUIRE(K > 0 && lda >= K && ldo >= N, "gemm: bad sizes M=%d N=%d K=%d lda=%d ldo=%d", M, N, K, lda, ldo);
  CUCA_REQUIRE(epilogue != EPI_RESIDUAL || out_dtype == CUCA_F32, "gemm: the residual stream is 32-bit");
  CUCA_REQUIRE(epilogue != EPI_SWIGLU || bias == nullptr, "gemm: SwiGLU takes no bias");
#define GO(TI, TO)                                                                               \
  do {                                                                                           \
    if (epilogue == EPI_STORE) launch<TI, TO, EPI_STORE>(A, W, bias, out, M, N, K, lda, ldo, stream);       \
    else if (epilogue == EPI_RESIDUAL) launch<TI, float, EPI_RESIDUAL>(A, W, bias, out, M, N, K, lda, ldo, stream); \
    else if (epilogue == EPI_SWIGLU) launch<TI, TO, EPI_SWIGLU>(A, W, bias, out, M, N, K, lda, ldo, stream); \
    else CUCA_REQUIRE(false, "gemm: unknown epilogue %d", epilogue);                               \
  } while (0)
  if (in_dtype == CUCA_F32 && out_dtype == CUCA_F32) GO(float, float);
  else if (in_dtype == CUCA_BF16 && out_dtype == CUCA_BF16) GO(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == CUCA_BF16 && out_dtype == CUCA_F32) GO(__nv_bfloat16, float);
  else CUCA_REQUIRE(false, "gemm: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef GO
  CUCA_CHECK_LAUNCH("gemm_simt");
  return 0;
}
