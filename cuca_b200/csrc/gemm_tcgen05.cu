// bfloat16 contraction on the 5th-generation tensor cores: out = epilogue(X[M,K] W[N,K]^T).
//
// The weight is the MMA's 128-row operand and the tokens are its N dimension
// (16..256), so one kernel serves a 2048-token prefill and a handful of decode
// rows: D[feature, token] accumulates in tensor memory, one TMEM lane per
// output feature. Both operands are K-major, as stored: TMA brings 128 x 64
// weight tiles and BN x 64 activation tiles (128-byte swizzle) into a ring of
// shared-memory stages; one thread issues tcgen05.mma (kind::f16, 32-bit
// accumulate) and tcgen05.commit hands each stage back to the producer. The
// epilogue reads TMEM with tcgen05.ld and fuses bias, the add into the 32-bit
// residual stream, or SwiGLU (gate and up tiles accumulate side by side in
// TMEM, so the same thread holds both values of a feature).
//
// Decode shapes have fewer 128-row tiles than the GPU has SMs, so K is split
// over several CTAs: each writes its 32-bit partial tile to a workspace and the
// last one to arrive adds the partials in split order (the result does not
// depend on arrival order) and runs the epilogue.
//
// Every wait on an mbarrier is bounded; on a timeout the kernel records
// CUCA_ERR_WAIT_TIMEOUT, lets copies in flight land, frees its TMEM and returns.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <string.h>

#define EPI_STORE 0
#define EPI_RESIDUAL 1
#define EPI_SWIGLU 2

namespace {

constexpr int TILE_N = 128;  // weight rows (output features) per CTA = TMEM lanes
constexpr int TILE_K = 64;   // bf16 elements per stage row = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false (and the error word set) if the phase did not complete in WAIT_LIMIT_NS.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = global_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (global_ns() - t0 > WAIT_LIMIT_NS) {
      if (err) atomicExch(err, CUCA_ERR_WAIT_TIMEOUT);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte swizzle,
// 8-row groups 1024 bytes apart; the tile base is 1024-byte aligned.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                  // leading byte offset: unused with a swizzled K-major tile
  d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                  // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                  // 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);
}

struct Params {
  void* out;
  const __nv_bfloat16* bias;
  float* workspace;
  int* counters;
  int* err;
  int M, N, K;   // tokens, output features, reduction
  int ldo;
  int epilogue;
  int out_f32;
  int splits;
  int ksteps_per_split;
};

template <int BN, bool DUAL>
struct Cfg {
  static constexpr int W_BYTES = TILE_N * TILE_K * 2 * (DUAL ? 2 : 1);
  static constexpr int X_BYTES = BN * TILE_K * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  // decode-sized tiles keep under half of an SM's shared memory, so the CTAs of the next contraction can move
  // in and prefetch their weights while this one drains; prefill-sized tiles take most of it
  static constexpr int SMEM_BUDGET = (BN <= 64 ? 108 : 200) * 1024;
  static constexpr int STAGES = (SMEM_BUDGET / STAGE_BYTES) > 8 ? 8 : (SMEM_BUDGET / STAGE_BYTES);
  static constexpr int NCOLS = BN * (DUAL ? 2 : 1);
  static constexpr int TMEM_COLS = NCOLS < 32 ? 32 : NCOLS;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + __expf(-g)) * u; }

template <bool DUAL>
__device__ __forceinline__ void write_out(const Params& p, int n, int m, float v, float u) {
  if (m >= p.M || n >= p.N) return;
  size_t o = (size_t)m * p.ldo + n;
  if (DUAL) {
    ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(silu_mul(v, u));
    return;
  }
  if (p.bias) v += __bfloat162float(p.bias[n]);
  if (p.epilogue == EPI_RESIDUAL) atomicAdd((float*)p.out + o, v);  // result unused: a fire-and-forget reduction;
                                                                   // one CTA owns each element, so the sum is exact
  else if (p.out_f32) ((float*)p.out)[o] = v;
  else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v);
}

template <int BN, bool DUAL>
__global__ void __launch_bounds__(128, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
  using C = Cfg<BN, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* accum_full = empty + C::STAGES;
  uint32_t* tmem_slot = (uint32_t*)(accum_full + 1);
  int* flag = (int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TILE_N;
  const int m0 = blockIdx.y * BN;
  const int split = blockIdx.z;
  const int total_ksteps = (p.K + TILE_K - 1) / TILE_K;
  const int ks_begin = split * p.ksteps_per_split;
  int ks_end = ks_begin + p.ksteps_per_split;
  if (ks_end > total_ksteps) ks_end = total_ksteps;
  const int nk = ks_end - ks_begin;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum_full, 1);
    *flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------ producer: TMA loads into the stage ring
    // Weights are never written by a kernel, so the first ring of weight tiles is requested before waiting
    // for the predecessor; activations only after it.
    const int pre = nk < C::STAGES ? nk : C::STAGES;
    for (int i = 0; i < pre; ++i) {
      uint8_t* st = smem + i * C::STAGE_BYTES;
      mbar_expect_tx(&full[i], C::STAGE_BYTES);
      int kc = (ks_begin + i) * TILE_K;
      tma_load_2d(st, &tmW, &full[i], kc, n0);
      if (DUAL) tma_load_2d(st + TILE_N * TILE_K * 2, &tmW, &full[i], kc, p.N + n0);
    }
    pdl_wait();
    for (int i = 0; i < pre; ++i)
      tma_load_2d(smem + i * C::STAGE_BYTES + C::W_BYTES, &tmX, &full[i], (ks_begin + i) * TILE_K, m0);
    for (int i = pre; i < nk; ++i) {
      int s = i % C::STAGES;
      uint32_t ph = (i / C::STAGES) & 1;
      if (!mbar_wait(&empty[s], ph ^ 1, p.err)) { ok = false; break; }
      uint8_t* st = smem + s * C::STAGE_BYTES;
      mbar_expect_tx(&full[s], C::STAGE_BYTES);
      int kc = (ks_begin + i) * TILE_K;
      tma_load_2d(st, &tmW, &full[s], kc, n0);
      if (DUAL) tma_load_2d(st + TILE_N * TILE_K * 2, &tmW, &full[s], kc, p.N + n0);
      tma_load_2d(st + C::W_BYTES, &tmX, &full[s], kc, m0);
    }
  } else if (warp == 1 && lane == 0) {
    pdl_wait();
    // ------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = instr_desc(BN);
    for (int i = 0; i < nk; ++i) {
      int s = i % C::STAGES;
      uint32_t ph = (i / C::STAGES) & 1;
      if (!mbar_wait(&full[s], ph, p.err)) { ok = false; break; }
      tc_fence_after();
      uint32_t wa = smem_u32(smem + s * C::STAGE_BYTES);
      uint64_t adesc = smem_desc(wa);
      uint64_t adesc2 = smem_desc(wa + TILE_N * TILE_K * 2);
      uint64_t bdesc = smem_desc(wa + C::W_BYTES);
#pragma unroll
      for (int k = 0; k < TILE_K / UMMA_K; ++k) {
        uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
        uint64_t koff = (uint64_t)(k * UMMA_K * 2 >> 4);
        umma_bf16(tmem_base, adesc + koff, bdesc + koff, idesc, acc);
        if (DUAL) umma_bf16(tmem_base + BN, adesc2 + koff, bdesc + koff, idesc, acc);
      }
      umma_commit(&empty[s]);
    }
    umma_commit(accum_full);
  } else {
    pdl_wait();
  }
  __syncwarp();

  // ---------------------------------------------------- epilogue: all four warps, one TMEM lane per thread
  if (nk > 0 && !mbar_wait(accum_full, 0, p.err)) ok = false;
  tc_fence_after();
  if (!ok) atomicExch(flag, 1);
  __syncthreads();
  const bool failed = *flag != 0;
  const int feature = n0 + warp * 32 + lane;
  const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);

  if (!failed) {
    if (p.splits == 1) {
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float v[16], u[16];
        if (nk > 0) {
          tmem_ld16(lane_addr + c, v);
          if (DUAL) tmem_ld16(lane_addr + BN + c, u);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = u[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) write_out<DUAL>(p, feature, m0 + c + j, v[j], DUAL ? u[j] : 0.f);
      }
    } else {
      // partial tile -> workspace[tile][split][column][lane]; the last CTA of the tile reduces in split order
      const int tile = blockIdx.y * gridDim.x + blockIdx.x;
      float* ws = p.workspace + ((size_t)tile * p.splits + split) * C::NCOLS * TILE_N;
#pragma unroll 1
      for (int c = 0; c < C::NCOLS; c += 16) {
        float v[16];
        if (nk > 0) tmem_ld16(lane_addr + c, v);
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) ws[(size_t)(c + j) * TILE_N + threadIdx.x] = v[j];
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        int arrived = atomicAdd(&p.counters[tile], 1);
        *flag = (arrived == p.splits - 1) ? 2 : 0;
      }
      __syncthreads();
      if (*flag == 2) {
        __threadfence();
        const float* base = p.workspace + (size_t)tile * p.splits * C::NCOLS * TILE_N;
#pragma unroll 1
        for (int c = 0; c < BN; c += 8) {
          if (m0 + c >= p.M) break;
          float v[8], u[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = u[j] = 0.f;
          // split order: the sum does not depend on who arrived last; four splits' loads are in flight at once
          for (int s0 = 0; s0 < p.splits; s0 += 4) {
            float a[4][8], b[4][8];
#pragma unroll
            for (int ss = 0; ss < 4; ++ss) {
              const bool live = s0 + ss < p.splits;
              const float* part = base + (size_t)(s0 + ss) * C::NCOLS * TILE_N + threadIdx.x;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                a[ss][j] = live ? __ldcg(part + (size_t)(c + j) * TILE_N) : 0.f;
                if (DUAL) b[ss][j] = live ? __ldcg(part + (size_t)(BN + c + j) * TILE_N) : 0.f;
              }
            }
#pragma unroll
            for (int ss = 0; ss < 4; ++ss)
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                v[j] += a[ss][j];
                if (DUAL) u[j] += b[ss][j];
              }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) write_out<DUAL>(p, feature, m0 + c + j, v[j], u[j]);
        }
        if (threadIdx.x == 0) p.counters[tile] = 0;  // ready for the next launch
      }
    }
  } else {
    // let copies in flight land before the shared memory is handed to another CTA
    unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ------------------------------------------------------------------ host side
int device_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t rows, cols, stride;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && stride == o.stride && box_rows == o.box_rows;
  }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.stride;
    h = h * 1000003u ^ k.box_rows;
    return h;
  }
};

// Tensor map of a row-major bf16 matrix [rows, cols] with `stride` elements between rows; box = box_rows x 64.
bool tensor_map(const void* ptr, uint64_t rows, uint64_t cols, uint64_t stride, uint32_t box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, stride, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {stride * 2};
  cuuint32_t box[2] = {(cuuint32_t)TILE_K, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

template <int BN, bool DUAL>
int launch_tc(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, dim3 grid, cudaStream_t stream) {
  using C = Cfg<BN, DUAL>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) {
      cuca_set_error("gemm_tc: cannot reserve %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e));
      return 2;
    }
    configured = true;
  }
  cuca_launch(gemm_tc_kernel<BN, DUAL>, grid, dim3(128), C::SMEM, stream, true, tmW, tmX, p);
  CUCA_CHECK_LAUNCH("gemm_tc");
  return 0;
}

}  // namespace

// 1 when the tensor-core kernel takes this problem, else 0 with the reason in cuca_last_error().
CUCA_API int cuca_gemm_tc_supported(const void* A, const void* W, int M, int N, int K, int lda) {
  if (K % 8 != 0 || lda % 8 != 0) { cuca_set_error("gemm_tc: K=%d and lda=%d must be multiples of 8 (16-byte rows for TMA)", K, lda); return 0; }
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) { cuca_set_error("gemm_tc: operands must be 16-byte aligned"); return 0; }
  if (M <= 0 || N <= 0) { cuca_set_error("gemm_tc: empty problem"); return 0; }
  return 1;
}

// out = epilogue(A[M,K] W[N,K]^T), bf16 operands. workspace/counters: scratch for split-K
// (ws_bytes of 32-bit partials; n_counters zeroed ints, left zeroed). max_splits <= 1 disables split-K.
CUCA_API int cuca_gemm_tc(const void* A, const void* W, const void* bias, void* out, int out_dtype, int M, int N,
                          int K, int lda, int ldo, int epilogue, void* workspace, size_t ws_bytes, int* counters,
                          int n_counters, int max_splits, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (!cuca_gemm_tc_supported(A, W, M, N, K, lda)) return 1;
  CUCA_REQUIRE(epilogue != EPI_RESIDUAL || out_dtype == CUCA_F32, "gemm_tc: the residual stream is 32-bit");
  CUCA_REQUIRE(epilogue != EPI_SWIGLU || (bias == nullptr && out_dtype == CUCA_BF16), "gemm_tc: SwiGLU writes bf16, no bias");
  const bool dual = epilogue == EPI_SWIGLU;
  int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  // more, narrower token tiles when the wide ones would leave SMs idle (the weight tile is re-read from L2)
  while (bn > 64 && ((N + TILE_N - 1) / TILE_N) * ((M + bn - 1) / bn) < device_sms()) bn >>= 1;
  CUtensorMap tmW, tmX;
  CUCA_REQUIRE(tensor_map(W, (uint64_t)N * (dual ? 2 : 1), K, K, TILE_N, &tmW), "gemm_tc: weight tensor map failed");
  CUCA_REQUIRE(tensor_map(A, M, K, lda, bn, &tmX), "gemm_tc: activation tensor map failed");
  dim3 grid((N + TILE_N - 1) / TILE_N, (M + bn - 1) / bn, 1);
  const int tiles = grid.x * grid.y;
  const int ksteps = (K + TILE_K - 1) / TILE_K;
  int splits = 1;
  if (workspace && counters && max_splits > 1 && tiles < device_sms() && bn <= 64) {
    splits = device_sms() / tiles;
    if (splits > max_splits) splits = max_splits;
    if (splits > ksteps / 4) splits = ksteps / 4;  // at least four K steps per CTA
    size_t per_tile = (size_t)(dual ? 2 : 1) * bn * TILE_N * sizeof(float);
    while (splits > 1 && (per_tile * tiles * splits > ws_bytes)) --splits;
    if (tiles > n_counters || splits < 1) splits = 1;
  }
  Params p;
  p.out = out; p.bias = (const __nv_bfloat16*)bias; p.workspace = (float*)workspace; p.counters = counters;
  p.err = err; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.epilogue = epilogue; p.out_f32 = out_dtype == CUCA_F32;
  p.splits = splits;
  p.ksteps_per_split = (ksteps + splits - 1) / splits;
  // every split must own at least one K step
  while (splits > 1 && (splits - 1) * p.ksteps_per_split >= ksteps) {
    --splits;
    p.splits = splits;
    p.ksteps_per_split = (ksteps + splits - 1) / splits;
  }
  grid.z = splits;
#define GO(BN_)                                                                  \
  case BN_:                                                                      \
    return dual ? launch_tc<BN_, true>(tmW, tmX, p, grid, stream) : launch_tc<BN_, false>(tmW, tmX, p, grid, stream);
  switch (bn) {
    GO(16) GO(32) GO(64) GO(128) GO(256)
  }
#undef GO
  return 1;
}
