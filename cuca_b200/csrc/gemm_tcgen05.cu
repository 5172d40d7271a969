// bfloat16 contraction on the 5th-generation tensor cores: out = epilogue(X[M,K] W[N,K]^T).
//
// A persistent, warp-specialised kernel: two threads (of two warps, taking stages in turn: one thread alone requests
// about 16 KB per 0.45 us, less than an SM's share of the memory's rate) stream tiles with TMA (128-byte swizzle)
// into a ring of shared-memory stages; over few tokens the weights carry the L2 hint "evict first", since a decode
// step reads each weight once and far more of them than L2 holds; one thread issues tcgen05.mma (kind::f16, 32-bit accumulate) into one of two TMEM
// accumulators, and four warps drain the other accumulator with tcgen05.ld and run the epilogue (store, bias,
// add into the 32-bit residual stream, or SwiGLU), so the epilogue of one tile overlaps the main loop of the
// next. tcgen05.commit hands stages back to the producer and accumulators to the epilogue.
//
// Two orientations share the code. Up to 256 tokens (decode, short portions; SwiGLU up to 64), the weight is the 128-row
// MMA operand and the tokens are the N dimension (16..256): D[feature, token], one TMEM lane per output feature. Above, the tokens
// are the 128-row operand and 256 weight rows the N dimension: D[token, feature], so a thread owns a run of
// consecutive features of one token and stores vectors. For SwiGLU the gate and up tiles accumulate side by
// side in TMEM, so one thread holds both values of a feature.
//
// Work is cut in units of one 64-wide K step of one tile. With plenty of tiles, CTAs take whole tiles in
// turn. With few tiles (decode: 32 to 1002 tiles of 64 K steps on 148 SMs) the units are dealt out evenly
// ("stream-K"): a CTA's share may start and end inside a tile; partial tiles go to a workspace and the last CTA
// to arrive adds the parts in K order (the result does not depend on arrival order) and runs the epilogue.
// Over many tokens there are two more forms of a tile: the tall one (256 tokens x 256 weight rows in one CTA, see
// Cfg) and the two-SM one (a cluster of two CTAs on such a tile, tcgen05.mma.cta_group::2, see gemm_pair_kernel),
// which also produces the K slices left unadded (EPI_PARTIAL) from 129 to 512 tokens.
//
// The kernel is a programmatic dependent: it requests its first ring of weight tiles before waiting for its
// predecessor, since weights are never written. Every wait on an mbarrier is bounded; on a timeout the kernel
// records CUCA_ERR_WAIT_TIMEOUT, every role stops, copies in flight land, TMEM is freed and the kernel returns.
#include "tcgen05.cuh"
#include <mutex>
#include <unordered_map>
#include <string.h>
#include <stdlib.h>

#define EPI_STORE 0
#define EPI_RESIDUAL 1
#define EPI_SWIGLU 2
#define EPI_PARTIAL 3  // out = 32-bit [slices][M][N]: every K slice of a tile stores its partial sum, nothing is added up

namespace {

constexpr int SWAP_MAX_TOKENS = 256;  // up to here the weights are the 128-row operand and the tokens the columns
// SwiGLU: up to here. Beyond, its two accumulators leave no room in the tensor memory for a second tile's, and the
// token-row forms are as fast or faster (measured on the Llama-3.1-8B widths, us: 65..128 tokens 46.0-46.5 against
// 46.4-49.4 this way; 129..256 tokens 55.4-59.3 in the tall form against 56.7-65.7).
constexpr int SWAP_MAX_TOKENS_SWIGLU = 64;
constexpr int NPROD = 2;       // one thread requests about 16 KB per 0.45 us: too little for an SM's share of the memory's rate

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
  int tile_rows; // rows of the 128-row operand one tile covers: 128, or 256 for the tall form (two row blocks)
  int tiles_a;   // tiles along the 128-row operand
  int tiles;     // all tiles
  int ksteps;    // K steps per tile
  int stream_k;  // 0: whole tiles in turn; 1: units dealt out evenly; 2: per_tile even K slices of every tile
  // tokens as rows but fewer tiles than SMs (mode 0): instead of whole tiles, `pieces` column pieces of
  // `piece_w` output columns over all of K, one per CTA
  int pieces, piece_w;
  int per_tile;  // mode 2: CTAs per tile
  int max_parts; // workspace slots per tile
  int tma_out;   // many tokens: whole tiles leave through shared memory and the copy engine (tensor map of `out`)
  int ordered_add;  // mode 2 into the 32-bit stream over many tokens: the K slices of a tile add themselves in turn
  int skew;         // ... and slice k + 1 has `skew` K steps more than slice k, so that it finishes when slice k has added
  int slab_rows;    // pairs of CTAs leaving K slices unadded: rows of one slice's slab in `out` (a multiple of 32, >= M)
};

constexpr int STAGING_BUF = 32 * 128;  // 32 rows of 128 bytes

// SWAP: weight rows on the 128 lanes, BN tokens as columns. Otherwise tokens on the lanes, 256 weight rows
// (SwiGLU: 128 gate + 128 up) as columns.
// TALL (many tokens only): a tile is 256 tokens x 256 weight rows, two row blocks that share every stage's weight
// tile. A CTA then takes in 64 KB per K step for twice the arithmetic (32 KB per 128 x 256 block instead of 48):
// the main loop of the 128-row form runs at the pace of its loads (64 bytes per clock from L2 into an SM), this
// one at the pace of its MMAs. The two accumulators fill all 512 TMEM columns, so a tile's epilogue (eight warps,
// one per 32 rows of either block) no longer runs under the next tile's main loop.
template <int BN, bool DUAL, bool SWAP, bool TALL = false>
struct Cfg {
  static_assert(!TALL || (!SWAP && BN == 256), "the tall form is for many tokens and 256 weight rows");
  static constexpr int ROW_BLOCKS = TALL ? 2 : 1;
  static constexpr int A_BYTES = TILE_A * TILE_K * 2 * ((SWAP && DUAL) || TALL ? 2 : 1);
  static constexpr int B_ROWS = BN;  // many tokens: 256 weight rows a stage, or 128 for launches of column pieces up to 128 wide
  static constexpr int B_BYTES = B_ROWS * TILE_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // deep rings in both orientations: the more weight bytes in flight, the closer the stream runs to the memory's
  // rate (measured: 200 KB of stages beat 108 KB with room for the next kernel's CTAs)
#ifndef CUCA_SWAP_SMEM_KB
#define CUCA_SWAP_SMEM_KB 200
#endif
  static constexpr int SMEM_BUDGET = (SWAP ? ((BN == 64 && DUAL && CUCA_SWAP_SMEM_KB < 124) ? 124 : CUCA_SWAP_SMEM_KB) : 192) * 1024;
  static constexpr int STAGES = (SMEM_BUDGET / STAGE_BYTES) > 12 ? 12 : (SMEM_BUDGET / STAGE_BYTES);
  static constexpr int MMA_N = BN;                                 // N of one tcgen05.mma
  static constexpr int NCOLS = (SWAP ? BN * (DUAL ? 2 : 1) : BN) * ROW_BLOCKS;  // accumulator columns of one tile
  // tiles whose accumulators TMEM holds at once: two, so that one tile's epilogue runs under the next one's main
  // loop; one in the tall form, whose accumulators fill all 512 columns
  static constexpr int ACC_BUFS = TALL ? 1 : 2;
  static constexpr int TMEM_COLS = ACC_BUFS * NCOLS < 32 ? 32 : ACC_BUFS * NCOLS;
  static constexpr int EPI_WARPS = 4 * ROW_BLOCKS;
  static constexpr int PROD2_WARP = 2 + EPI_WARPS;                   // the second producer's warp
  static constexpr int THREADS = 32 * (PROD2_WARP + 1);              // warp 0 producer, warp 1 MMA, epilogue warps, producer
  static constexpr int STAGING_BUFS = TALL ? 1 : 2;                  // staging buffers per epilogue warp
  static constexpr int OUT_COLS = SWAP ? BN : (DUAL ? BN / 2 : BN);  // output columns of one tile
  // many tokens: each epilogue warp stages its 32 rows x 128 bytes of output twice over for the copy engine
  static constexpr int STAGING = SWAP ? 0 : EPI_WARPS * STAGING_BUFS * STAGING_BUF;
  static constexpr int SMEM = STAGES * STAGE_BYTES + STAGING + 1024 /*alignment*/ + 512 /*barriers*/;
};

// One CTA's run of work: segments (tile, K steps [ks0, ks1)) in the order every role walks them.
struct Segment {
  int tile, ks0, ks1, part, nparts;
  int a0, b0;  // first row of the 128-row operand, first output column (of the column operand)
  int w;       // output columns
};
struct SegmentWalk {
  const Params& p;
  long long u, u_end;   // stream-K: unit cursor
  int tile_cursor;      // whole tiles: next tile
  int out_cols;         // output columns of a whole tile
  bool piece_done;
  __device__ SegmentWalk(const Params& prm, int cols) : p(prm), out_cols(cols), piece_done(false) {
    const long long U = (long long)p.tiles * p.ksteps, G = gridDim.x;
    u = (long long)blockIdx.x * U / G;
    u_end = ((long long)blockIdx.x + 1) * U / G;
    tile_cursor = blockIdx.x;
  }
  __device__ void origin(Segment& s) const {
    s.a0 = (s.tile % p.tiles_a) * p.tile_rows;
    s.b0 = (s.tile / p.tiles_a) * out_cols;
    s.w = out_cols;
  }
  __device__ bool next(Segment& s) {
    if (!p.stream_k) {
      s.ks0 = 0; s.ks1 = p.ksteps; s.part = 0; s.nparts = 1;
      if (!p.pieces) {
        if (tile_cursor >= p.tiles) return false;
        s.tile = tile_cursor;
        origin(s);
        tile_cursor += gridDim.x;
        return true;
      }
      // column piece number blockIdx.x: neighbouring CTAs take the same columns of different row blocks
      if (piece_done) return false;
      piece_done = true;
      s.tile = p.tiles;  // no whole tile
      s.a0 = ((int)blockIdx.x % p.tiles_a) * TILE_A;
      s.b0 = ((int)blockIdx.x / p.tiles_a) * p.piece_w;
      s.w = p.piece_w;
      return true;
    }
    if (p.stream_k == 2) {
      // one K slice of one tile per CTA
      if (tile_cursor < 0) return false;
      s.tile = (int)blockIdx.x / p.per_tile;
      origin(s);
      s.part = (int)blockIdx.x % p.per_tile;
      s.nparts = p.per_tile;
      if (p.skew > 0) {
        const int n = p.per_tile, tri = p.skew * n * (n - 1) / 2;
        const int base = (p.ksteps - tri) / n;
        s.ks0 = s.part * base + p.skew * s.part * (s.part - 1) / 2;
        s.ks1 = s.part == n - 1 ? p.ksteps : s.ks0 + base + p.skew * s.part;
      } else {
        s.ks0 = (int)((long long)s.part * p.ksteps / p.per_tile);
        s.ks1 = (int)((long long)(s.part + 1) * p.ksteps / p.per_tile);
      }
      tile_cursor = -1;
      return true;
    }
    if (u >= u_end) return false;
    const long long K = p.ksteps, U = (long long)p.tiles * K, G = gridDim.x;
    s.tile = (int)(u / K);
    origin(s);
    s.ks0 = (int)(u % K);
    long long left = u_end - u;
    s.ks1 = (int)((K - s.ks0 < left) ? K : s.ks0 + left);
    u += s.ks1 - s.ks0;
    // CTAs whose share touches this tile: first .. last
    long long t0 = (long long)s.tile * K, t1 = t0 + K;
    int first = (int)(((t0 + 1) * G + U - 1) / U) - 1;
    int last = (int)((t1 * G + U - 1) / U) - 1;
    s.part = (int)blockIdx.x - first;
    s.nparts = last - first + 1;
    return true;
  }
};

// The quotient is the approximate one (2 ulp, rounded to bf16 right after): the IEEE division leaves its fast path
// for a numerator of zero, which is what every padded row or column of a tile holds, and a warp then pays the slow
// path for all its lanes (measured: SwiGLU over 255 tokens took 76.7 us, over 256 tokens 63.1).
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

// ---- epilogue of 16 accumulator columns held by one thread (TMEM lane `lane_row` of tile rows a0.., columns c..)
template <int BN, bool DUAL, bool SWAP>
__device__ __forceinline__ void store16(const Params& p, int a0, int b0, int lane_row, int c, const float (&v)[16],
                                        const float (&u)[16]) {
  if (SWAP) {
    // lane = feature, columns = tokens
    const int n = a0 + lane_row;
    if (n >= p.N) return;
    const float bias = (!DUAL && p.bias) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int m = b0 + c + j;
      if (m >= p.M) break;
      const size_t o = (size_t)m * p.ldo + n;
      if (DUAL) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(silu_mul(v[j], u[j]));
      else if (p.epilogue == EPI_RESIDUAL) atomicAdd((float*)p.out + o, v[j] + bias);  // result unused: a fire-and-forget
                                                                                       // add; one thread owns the element
      else if (p.out_f32) ((float*)p.out)[o] = v[j] + bias;
      else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v[j] + bias);
    }
  } else {
    // lane = token, columns = 16 consecutive features
    const int m = a0 + lane_row;
    if (m >= p.M) return;
    const int n = b0 + c;
    if (n >= p.N) return;
    float r[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) r[j] = DUAL ? silu_mul(v[j], u[j]) : v[j];
    const size_t o = (size_t)m * p.ldo + n;
    const bool full = n + 16 <= p.N;
    if (!DUAL && p.bias) {
#pragma unroll
      for (int j = 0; j < 16; ++j) if (n + j < p.N) r[j] += __bfloat162float(p.bias[n + j]);
    }
    if (p.epilogue == EPI_RESIDUAL || p.out_f32) {
      float* dst = (float*)p.out + o;
      const bool vec = full && ((((size_t)dst) & 15) == 0);
      if (vec) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float4 x = make_float4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
          if (p.epilogue == EPI_RESIDUAL) {
            float4 old = *reinterpret_cast<float4*>(dst + 4 * q);
            x.x += old.x; x.y += old.y; x.z += old.z; x.w += old.w;
          }
          *reinterpret_cast<float4*>(dst + 4 * q) = x;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (n + j < p.N) dst[j] = (p.epilogue == EPI_RESIDUAL ? dst[j] : 0.f) + r[j];
      }
    } else {
      __nv_bfloat16* dst = (__nv_bfloat16*)p.out + o;
      const bool vec = full && ((((size_t)dst) & 15) == 0);
      if (vec) {
        uint4 lo, hi;
        __nv_bfloat162 t;
        t = __floats2bfloat162_rn(r[0], r[1]); lo.x = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(r[2], r[3]); lo.y = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(r[4], r[5]); lo.z = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(r[6], r[7]); lo.w = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(r[8], r[9]); hi.x = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(r[10], r[11]); hi.y = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(r[12], r[13]); hi.z = *reinterpret_cast<uint32_t*>(&t);
        t = __floats2bfloat162_rn(r[14], r[15]); hi.w = *reinterpret_cast<uint32_t*>(&t);
        *reinterpret_cast<uint4*>(dst) = lo;
        *reinterpret_cast<uint4*>(dst + 8) = hi;
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) if (n + j < p.N) dst[j] = __float2bfloat16_rn(r[j]);
      }
    }
  }
}

// Many tokens, a whole tile: one epilogue warp's 32 token rows leave in runs of 128 bytes per row (32 32-bit or 64
// bf16 values). A thread writes its row's run into a staging buffer in the 128-byte swizzle of the output's tensor
// map (no bank conflicts), and the copy engine stores the 32 x 128-byte box, or adds it into the 32-bit stream,
// clipped at the matrix's edges. A thread writing its own row straight to global memory instead touches one line
// per lane and instruction: measured, 13 us per tile of the output projection against 26 us of main loop.
template <bool DUAL, int BUFS = 2>
__device__ __forceinline__ void tma_epilogue(const Params& p, const CUtensorMap* tmO, uint32_t acc, int a0, int b0,
                                             int width, bool with_bias, int quarter, int lane, uint8_t* staging,
                                             int& chunk_no, int row_offset = 0) {
  const int y0 = a0 + quarter * 32;
  const int ch = p.out_f32 ? 32 : 64;  // the host cuts column pieces in whole runs
  uint8_t* const my_row = staging + lane * 128;
  const int sw = lane & 7;
#pragma unroll 1
  for (int c = 0; c < width; c += ch) {
    uint8_t* row = my_row + (chunk_no % BUFS) * STAGING_BUF;
    if (lane == 0) bulk_wait_read<BUFS - 1>();  // the copy that last used this buffer has read it
    __syncwarp();
#pragma unroll 1
    for (int h = 0; h < ch; h += 16) {
      float v[16];
      tmem_ld16(acc + c + h, v);
      if (DUAL) {
        float u[16];
        tmem_ld16(acc + 128 + c + h, u);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = silu_mul(v[j], u[j]);
      } else if (p.bias && with_bias) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (b0 + c + h + j < p.N) v[j] += __bfloat162float(p.bias[b0 + c + h + j]);
      }
      if (p.out_f32) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<float4*>(row + ((((h >> 2) + q) ^ sw) << 4)) =
              make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      } else {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint4 w;
          __nv_bfloat162 t;
          t = __floats2bfloat162_rn(v[8 * q], v[8 * q + 1]); w.x = *reinterpret_cast<uint32_t*>(&t);
          t = __floats2bfloat162_rn(v[8 * q + 2], v[8 * q + 3]); w.y = *reinterpret_cast<uint32_t*>(&t);
          t = __floats2bfloat162_rn(v[8 * q + 4], v[8 * q + 5]); w.z = *reinterpret_cast<uint32_t*>(&t);
          t = __floats2bfloat162_rn(v[8 * q + 6], v[8 * q + 7]); w.w = *reinterpret_cast<uint32_t*>(&t);
          *reinterpret_cast<uint4*>(row + ((((h >> 3) + q) ^ sw) << 4)) = w;
        }
      }
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      if (y0 < p.M && b0 + c < p.N) {
        const void* src = staging + (chunk_no % BUFS) * STAGING_BUF;
        if (p.epilogue == EPI_RESIDUAL) tma_reduce_add_2d(tmO, src, b0 + c, y0);
        else tma_store_2d(tmO, src, b0 + c, y0 + row_offset);  // row_offset: the slab of a K slice left unadded
      }
      bulk_commit();
    }
    ++chunk_no;
  }
}

template <int N_THREADS>
__device__ __forceinline__ void epilogue_sync_n() { asm volatile("bar.sync 1, %0;" ::"n"(N_THREADS) : "memory"); }

template <int BN, bool DUAL, bool SWAP, bool TALL = false>
__global__ void __launch_bounds__((Cfg<BN, DUAL, SWAP, TALL>::THREADS), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmO, const Params p) {
  using C = Cfg<BN, DUAL, SWAP, TALL>;
  auto epilogue_sync = [] { epilogue_sync_n<32 * C::EPI_WARPS>(); };
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + C::STAGES * C::STAGE_BYTES;  // 1024-byte aligned: the stages are multiples of 1024 bytes
  uint64_t* full = (uint64_t*)(staging + C::STAGING);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tmem_full = empty + C::STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_slot = (uint32_t*)(tmem_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* last_flag = (int*)(tmem_slot + 2);
  volatile int* seg_ok = (volatile int*)(tmem_slot + 3);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], C::EPI_WARPS);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    *last_flag = 0;
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

  // weights and activations of one stage: which is which depends on the orientation
  // few tokens: every weight is read once per step, so it should not displace what is read again (activations,
  // partial sums, keys and values)
  const uint64_t once = SWAP ? l2_evict_first() : 0;
  // bytes a stage of this segment receives: a column piece of up to 128 weight rows needs one box of them only
  auto stage_tx = [&](const Segment& s) -> uint32_t {
    return C::STAGE_BYTES - ((!SWAP && !DUAL && BN == 256 && s.w <= 128) ? 128 * TILE_K * 2 : 0);
  };
  auto load_weights = [&](uint8_t* st, uint64_t* bar, const Segment& s, int kc) {
    if (SWAP) {
      tma_load_2d_hint(st, &tmA, bar, kc, s.a0, once);
      if (DUAL) tma_load_2d_hint(st + TILE_A * TILE_K * 2, &tmA, bar, kc, p.N + s.a0, once);
    } else {
      tma_load_2d(st + C::A_BYTES, &tmB, bar, kc, s.b0);
      if (BN == 256 && (DUAL || s.w > 128)) tma_load_2d(st + C::A_BYTES + 128 * TILE_K * 2, &tmB, bar, kc, DUAL ? p.N + s.b0 : s.b0 + 128);
    }
  };
  auto load_activations = [&](uint8_t* st, uint64_t* bar, const Segment& s, int kc) {
    if (SWAP) tma_load_2d(st + C::A_BYTES, &tmB, bar, kc, s.b0);
    else {
      tma_load_2d(st, &tmA, bar, kc, s.a0);
      if (TALL) tma_load_2d(st + TILE_A * TILE_K * 2, &tmA, bar, kc, s.a0 + TILE_A);  // rows past M read as zeros
    }
  };

  if ((warp == 0 || warp == C::PROD2_WARP) && lane == 0) {
    // ------------------------------------------------ producers: stages in turn (it mod NPROD)
    const int mine = warp == 0 ? 0 : 1;
    // the first ring of weight tiles is requested before waiting for the predecessor kernel
    {
      SegmentWalk pre(p, C::OUT_COLS);
      Segment s;
      int it = 0;
      const int ahead = C::STAGES;
      while (it < ahead && pre.next(s)) {
        for (int ks = s.ks0; ks < s.ks1 && it < ahead; ++ks, ++it) {
          if (it % NPROD != mine) continue;
          mbar_expect_tx(&full[it], stage_tx(s));
          load_weights(smem + it * C::STAGE_BYTES, &full[it], s, ks * TILE_K);
        }
      }
    }
    pdl_wait();
    SegmentWalk walk(p, C::OUT_COLS);
    Segment s;
    int it = 0;
    bool ok = true;
    while (ok && walk.next(s)) {
      for (int ks = s.ks0; ks < s.ks1; ++ks, ++it) {
        if (it % NPROD != mine) continue;
        const int st = it % C::STAGES;
        uint8_t* sp = smem + st * C::STAGE_BYTES;
        if (it >= C::STAGES) {
          if (!mbar_wait(&empty[st], ((it / C::STAGES) & 1) ^ 1, p.err, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full[st], stage_tx(s));
          load_weights(sp, &full[st], s, ks * TILE_K);
        }
        load_activations(sp, &full[st], s, ks * TILE_K);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------ MMA issuer
    pdl_wait();
    SegmentWalk walk(p, C::OUT_COLS);
    Segment s;
    int it = 0, seg = 0;
    bool ok = true;
    while (ok && walk.next(s)) {
      const int buf = seg % C::ACC_BUFS;
      // a column piece is narrower than a tile (never with SwiGLU, whose tile is 128 gate and 128 up columns)
      const uint32_t idesc = instr_desc((SWAP || DUAL) ? C::MMA_N : s.w);
      if (!mbar_wait(&tmem_empty[buf], ((seg / C::ACC_BUFS) & 1) ^ 1, p.err, abort_flag)) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * C::NCOLS;
      for (int ks = s.ks0; ks < s.ks1; ++ks, ++it) {
        const int st = it % C::STAGES;
        if (!mbar_wait(&full[st], (it / C::STAGES) & 1, p.err, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + st * C::STAGE_BYTES);
        const uint64_t adesc = smem_desc(sa);
        const uint64_t adesc2 = smem_desc(sa + TILE_A * TILE_K * 2);
        const uint64_t bdesc = smem_desc(sa + C::A_BYTES);
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k) {
          const uint32_t accumulate = (ks > s.ks0 || k > 0) ? 1u : 0u;
          const uint64_t koff = (uint64_t)(k * UMMA_K * 2 >> 4);
          umma_bf16(acc, adesc + koff, bdesc + koff, idesc, accumulate);
          if (SWAP && DUAL) umma_bf16(acc + BN, adesc2 + koff, bdesc + koff, idesc, accumulate);
          if (TALL) umma_bf16(acc + BN, adesc2 + koff, bdesc + koff, idesc, accumulate);  // the second row block
        }
        umma_commit(&empty[st]);
      }
      if (ok) umma_commit(&tmem_full[buf]);
      ++seg;
    }
  } else if (warp >= 2 && warp < 2 + C::EPI_WARPS) {
    // ------------------------------------------------ epilogue: four warps per row block, one TMEM lane per thread
    pdl_wait();
    const int quarter = warp & 3;               // the TMEM lanes this warp may read
    const int block = TALL ? (warp - 2) >> 2 : 0;  // which 128-row block of a tall tile
    const int lane_row = quarter * 32 + lane;   // row within the block
    const int eidx = (warp - 2) * 32 + lane;    // 0.. among the epilogue threads
    SegmentWalk walk(p, C::OUT_COLS);
    Segment s;
    int seg = 0, chunk_no = 0;
    while (walk.next(s)) {
      const int buf = seg % C::ACC_BUFS;
      // one thread waits and tells the others, so all leave the loop together (they share named barriers)
      if (eidx == 0) seg_ok[buf] = mbar_wait(&tmem_full[buf], (seg / C::ACC_BUFS) & 1, p.err, abort_flag) ? 1 : 0;
      epilogue_sync();
      if (!seg_ok[buf]) break;
      tc_fence_after();
      const int a0 = s.a0 + block * TILE_A, b0 = s.b0;
      const uint32_t acc = tmem_base + buf * C::NCOLS + block * BN + ((uint32_t)(quarter * 32) << 16);
      if (SWAP && !DUAL && p.epilogue == EPI_PARTIAL) {
        // this K slice's partial sums go out as they are, [slice][token][feature]; whoever reads them adds them up
        float* dst = (float*)p.out + (size_t)s.part * p.M * p.ldo;
        const int n = a0 + lane_row;
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          tmem_ld16(acc + c, v);
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (b0 + c + j < p.M) dst[(size_t)(b0 + c + j) * p.ldo + n] = v[j];
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      } else if (!SWAP && s.nparts == 1 && p.tma_out) {
        tma_epilogue<DUAL, C::STAGING_BUFS>(p, &tmO, acc, a0, b0, s.w, true, quarter, lane,
                                            staging + (warp - 2) * (C::STAGING_BUFS * STAGING_BUF), chunk_no);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      } else if (!SWAP && !DUAL && p.ordered_add) {
        // One even K slice of a tile (every CTA has one, all CTAs are resident), added into the 32-bit stream by
        // the copy engine: the slices of a tile take turns in K order, so the sum does not depend on who finished
        // first, and nothing is parked in a workspace or read back. The turn is the tile's counter.
        if (eidx == 0) {
          int mine = 0;
          const unsigned long long t0 = global_ns();
          unsigned spins = 0;
          while (true) {
            if (*reinterpret_cast<volatile int*>(&p.counters[s.tile]) == s.part) { mine = 1; break; }
            if ((++spins & 63u) == 0) {
              if (*abort_flag) break;
              if (global_ns() - t0 > WAIT_LIMIT_NS) {
                if (p.err) atomicExch(p.err, CUCA_ERR_WAIT_TIMEOUT);
                *abort_flag = 1;
                break;
              }
            }
          }
          *last_flag = mine;
        }
        epilogue_sync();
        const bool mine = *last_flag != 0;
        epilogue_sync();  // everyone has read the flag before it is written again
        if (!mine) break;
        __threadfence();  // the slices before this one have added their sums
        tma_epilogue<false, C::STAGING_BUFS>(p, &tmO, acc, a0, b0, s.w, s.part == 0, quarter, lane,
                                             staging + (warp - 2) * (C::STAGING_BUFS * STAGING_BUF), chunk_no);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&tmem_empty[buf]);
          bulk_wait_all();  // this warp's adds have been performed
        }
        __threadfence();
        epilogue_sync();
        if (eidx == 0) {
          if (s.part == s.nparts - 1) atomicExch(&p.counters[s.tile], 0);  // ready for the next launch
          else atomicAdd(&p.counters[s.tile], 1);
        }
      } else if (s.nparts == 1) {
#pragma unroll 1
        for (int c = 0; c < (SWAP ? C::OUT_COLS : s.w); c += 16) {
          float v[16], u[16];
          tmem_ld16(acc + c, v);
          if (DUAL) tmem_ld16(acc + (SWAP ? BN : 128) + c, u);
          store16<BN, DUAL, SWAP>(p, a0, b0, lane_row, c, v, u);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      } else {
        // a part of a tile: park it in the workspace, [tile][part][column][lane]
        float* ws = p.workspace + ((size_t)s.tile * p.max_parts + s.part) * C::NCOLS * TILE_A;
#pragma unroll 1
        for (int c = 0; c < C::NCOLS; c += 16) {
          float v[16];
          tmem_ld16(acc + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) ws[(size_t)(c + j) * TILE_A + lane_row] = v[j];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);  // the accumulator is free while the parts are added
        __threadfence();
        epilogue_sync();
        if (eidx == 0) *last_flag = (atomicAdd(&p.counters[s.tile], 1) == s.nparts - 1) ? 1 : 0;
        epilogue_sync();
        const bool last = *last_flag != 0;
        epilogue_sync();  // everyone has read the flag before a later segment rewrites it
        if (last) {
          __threadfence();
          const float* base = p.workspace + (size_t)s.tile * p.max_parts * C::NCOLS * TILE_A + lane_row;
#pragma unroll 1
          for (int c = 0; c < C::OUT_COLS; c += 16) {
            float v[16], u[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = u[j] = 0.f;
            // parts in K order: the sum does not depend on who arrived last; two parts' loads in flight at once
            for (int q0 = 0; q0 < s.nparts; q0 += 2) {
              float a[2][16], b[2][16];
#pragma unroll
              for (int qq = 0; qq < 2; ++qq) {
                const bool live = q0 + qq < s.nparts;
                const float* part = base + (size_t)(q0 + qq) * C::NCOLS * TILE_A;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  a[qq][j] = live ? __ldcg(part + (size_t)(c + j) * TILE_A) : 0.f;
                  if (DUAL) b[qq][j] = live ? __ldcg(part + (size_t)((SWAP ? BN : 128) + c + j) * TILE_A) : 0.f;
                }
              }
#pragma unroll
              for (int qq = 0; qq < 2; ++qq)
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  v[j] += a[qq][j];
                  if (DUAL) u[j] += b[qq][j];
                }
            }
            store16<BN, DUAL, SWAP>(p, a0, b0, lane_row, c, v, u);
          }
          if (eidx == 0) p.counters[s.tile] = 0;  // ready for the next launch
        }
      }
      ++seg;
    }
    if (!SWAP && lane == 0) bulk_wait_all();  // this thread's stores have left shared memory and landed
  }
  __syncwarp();
  if (*abort_flag) {
    // let copies in flight land before the shared memory is handed to another CTA
    unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ------------------------------------------------------------------ many tokens: two SMs on one tile
// A pair of CTAs (a cluster of two, on neighbouring SMs) takes a tile of 256 tokens x 256 weight rows. Each CTA
// stages its own 128 token rows and HALF of the tile's weight rows (16 KB + 16 KB per K step instead of 16 + 32), and
// one thread of the first CTA issues `tcgen05.mma.cta_group::2` with M = 256: the tensor cores of both SMs read
// both halves of the weight tile, each SM accumulates its own 128 rows x 256 columns in its own tensor memory.
// Per SM and K step that is 32 KB from L2 for 278 ns of MMAs (the one-SM form needs 48 KB and runs at the pace of
// those loads), in six stages of 32 KB, with two accumulators as before so that a tile's epilogue runs under the
// next tile's main loop. Who signals whom: both CTAs' copies complete on the first CTA's `full` barrier (its
// producer expects the bytes of both); the MMA thread's commits arrive on the `empty` and `tmem_full` barriers of
// both CTAs (`tcgen05.commit ... multicast::cluster`, an arrival, not a load); the epilogue warps of both CTAs
// arrive on the first CTA's `tmem_empty`. No copy is multicast: each CTA fetches what it stages.
struct PairCfg {
  static constexpr int A_BYTES = TILE_A * TILE_K * 2;   // this CTA's 128 token rows of a K step
  static constexpr int B_BYTES = 128 * TILE_K * 2;      // this CTA's half of the 256 weight rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int NCOLS = 256;
  static constexpr int EPI_WARPS = 4;
  static constexpr int PROD2_WARP = 2 + EPI_WARPS;
  static constexpr int THREADS = 32 * (PROD2_WARP + 1);
  static constexpr int STAGING = EPI_WARPS * 2 * STAGING_BUF;
  static constexpr int SMEM = STAGES * STAGE_BYTES + STAGING + 1024 + 512;
};

__device__ __forceinline__ uint32_t pair_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of the first CTA's copy of a shared-memory object of this CTA.
__device__ __forceinline__ uint32_t in_first_cta(const void* p) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(a) : "r"(smem_u32(p)));
  return a;
}
__device__ __forceinline__ void pair_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void pair_tma_load_2d(void* dst, const CUtensorMap* map, uint32_t bar_first, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_first), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void pair_mbar_arrive_first(uint32_t bar_first) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_first) : "memory");
}
__device__ __forceinline__ void pair_tmem_alloc(uint32_t* dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void pair_tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void pair_tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void pair_umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// An arrival on the barrier at this offset in both CTAs of the pair, once the MMAs issued so far are done.
__device__ __forceinline__ void pair_umma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
// M = 256 over the pair (128 rows per CTA), N = 256.
__host__ __device__ constexpr uint32_t pair_instr_desc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <bool DUAL>
__global__ void __launch_bounds__(PairCfg::THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmO, const Params p) {
  using C = PairCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + C::STAGES * C::STAGE_BYTES;
  uint64_t* full = (uint64_t*)(staging + C::STAGING);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tmem_full = empty + C::STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint32_t* tmem_slot = (uint32_t*)(tmem_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* seg_ok = (volatile int*)(tmem_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = pair_rank();
  const bool first = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);   // the first CTA's producer, with the bytes of both CTAs' copies
      mbar_init(&empty[s], 1);  // the MMA thread's commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2 * C::EPI_WARPS);  // one arrival per epilogue warp of either CTA
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    pair_tmem_alloc(tmem_slot, 512);
    pair_tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  pair_sync();  // the other CTA's barriers exist before anything of this CTA signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // unit u: K slice (u % per_tile) of tile (u / per_tile); a tile is 256 token rows from a0 and 256 weight rows
  // (SwiGLU: 128 gate and 128 up) for the output columns from b0. With more than one slice per tile the slices stay
  // unadded: slice k goes to slab k of `out` (EPI_PARTIAL) for the kernel that reads them next.
  const int units = p.tiles * p.per_tile;
  auto tile_a0 = [&](int t) { return (t % p.tiles_a) * 256; };
  auto tile_b0 = [&](int t) { return (t / p.tiles_a) * (DUAL ? 128 : 256); };
  auto ks_first = [&](int u) { return (int)((long long)(u % p.per_tile) * p.ksteps / p.per_tile); };
  auto ks_end = [&](int u) { return (int)((long long)(u % p.per_tile + 1) * p.ksteps / p.per_tile); };
  // this CTA's half of the weight rows: the first CTA's rows become accumulator columns 0..127, the second's 128..255
  auto weight_row = [&](int b0) { return DUAL ? (first ? b0 : p.N + b0) : b0 + (int)rank * 128; };

  if ((warp == 0 || warp == C::PROD2_WARP) && lane == 0) {
    // ------------------------------------------------ producers of this CTA: stages in turn
    const int mine = warp == 0 ? 0 : 1;
    uint32_t full_first[C::STAGES];
#pragma unroll
    for (int s = 0; s < C::STAGES; ++s) full_first[s] = in_first_cta(&full[s]);
    // the first ring of weight tiles is requested before waiting for the predecessor kernel
    {
      int it = 0;
      for (int u = pair; u < units && it < C::STAGES; u += n_pairs)
        for (int ks = ks_first(u); ks < ks_end(u) && it < C::STAGES; ++ks, ++it) {
          if (it % NPROD != mine) continue;
          if (first) mbar_expect_tx(&full[it], 2 * C::STAGE_BYTES);
          pair_tma_load_2d(smem + it * C::STAGE_BYTES + C::A_BYTES, &tmB, full_first[it], ks * TILE_K,
                           weight_row(tile_b0(u / p.per_tile)));
        }
    }
    pdl_wait();
    int it = 0;
    bool ok = true;
    for (int u = pair; ok && u < units; u += n_pairs) {
      const int t = u / p.per_tile;
      const int a0 = tile_a0(t) + (int)rank * TILE_A, wr = weight_row(tile_b0(t));
      for (int ks = ks_first(u); ks < ks_end(u); ++ks, ++it) {
        if (it % NPROD != mine) continue;
        const int st = it % C::STAGES;
        uint8_t* sp = smem + st * C::STAGE_BYTES;
        if (it >= C::STAGES) {
          if (!mbar_wait(&empty[st], ((it / C::STAGES) & 1) ^ 1, p.err, abort_flag)) { ok = false; break; }
          if (first) mbar_expect_tx(&full[st], 2 * C::STAGE_BYTES);
          pair_tma_load_2d(sp + C::A_BYTES, &tmB, full_first[st], ks * TILE_K, wr);
        }
        pair_tma_load_2d(sp, &tmA, full_first[st], ks * TILE_K, a0);  // rows past M read as zeros
      }
    }
  } else if (warp == 1 && lane == 0 && first) {
    // ------------------------------------------------ MMA issuer of the pair
    pdl_wait();
    constexpr uint32_t idesc = pair_instr_desc();
    int it = 0, seg = 0;
    bool ok = true;
    for (int u = pair; ok && u < units; u += n_pairs, ++seg) {
      const int buf = seg & 1;
      if (!mbar_wait(&tmem_empty[buf], ((seg >> 1) & 1) ^ 1, p.err, abort_flag)) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * C::NCOLS;
      const int ks0 = ks_first(u);
      for (int ks = ks0; ks < ks_end(u); ++ks, ++it) {
        const int st = it % C::STAGES;
        if (!mbar_wait(&full[st], (it / C::STAGES) & 1, p.err, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + st * C::STAGE_BYTES);
        const uint64_t adesc = smem_desc(sa), bdesc = smem_desc(sa + C::A_BYTES);
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k) {
          const uint64_t koff = (uint64_t)(k * UMMA_K * 2 >> 4);
          pair_umma_bf16(acc, adesc + koff, bdesc + koff, idesc, (ks > ks0 || k > 0) ? 1u : 0u);
        }
        pair_umma_commit(&empty[st]);
      }
      if (ok) pair_umma_commit(&tmem_full[buf]);
    }
  } else if (warp >= 2 && warp < 2 + C::EPI_WARPS) {
    // ------------------------------------------------ epilogue of this CTA's 128 rows
    pdl_wait();
    const int quarter = warp & 3;
    const int eidx = (warp - 2) * 32 + lane;
    uint32_t empty_first[2] = {in_first_cta(&tmem_empty[0]), in_first_cta(&tmem_empty[1])};
    int seg = 0, chunk_no = 0;
    for (int u = pair; u < units; u += n_pairs, ++seg) {
      const int buf = seg & 1, t = u / p.per_tile;
      if (eidx == 0) seg_ok[buf] = mbar_wait(&tmem_full[buf], (seg >> 1) & 1, p.err, abort_flag) ? 1 : 0;
      epilogue_sync_n<32 * C::EPI_WARPS>();
      if (!seg_ok[buf]) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * C::NCOLS + ((uint32_t)(quarter * 32) << 16);
      tma_epilogue<DUAL, 2>(p, &tmO, acc, tile_a0(t) + (int)rank * TILE_A, tile_b0(t), DUAL ? 128 : 256, true, quarter,
                            lane, staging + (warp - 2) * (2 * STAGING_BUF), chunk_no, (u % p.per_tile) * p.slab_rows);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) pair_mbar_arrive_first(empty_first[buf]);
    }
    if (lane == 0) bulk_wait_all();  // this thread's stores have left shared memory and landed
  }
  __syncwarp();
  if (*abort_flag) {
    // let copies in flight land before the shared memory is handed to another CTA
    unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  pair_sync();  // neither CTA leaves (or frees tensor memory) while the other may still signal it or read its stages
  if (warp == 1) pair_tmem_dealloc(tmem_base, 512);
}

// ------------------------------------------------------------------ host side
}  // namespace
int cuca_device_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

// Most tokens for which a contraction can leave its K slices unadded (cuca_gemm_tc_partial).
CUCA_API int cuca_gemm_tc_partial_max_tokens();

// How many SMs the current device has (the Python side sizes its split choices by it too).
CUCA_API int cuca_sm_count() { return cuca_device_sms(); }

namespace {
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
  int elem_bytes;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && stride == o.stride && box_rows == o.box_rows &&
           elem_bytes == o.elem_bytes;
  }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.stride;
    h = h * 1000003u ^ k.box_rows;
    h = h * 1000003u ^ (size_t)k.elem_bytes;
    return h;
  }
};

}  // namespace

bool cuca_tensor_map_bf16(const void* ptr, uint64_t rows, uint64_t cols, uint64_t stride, uint32_t box_rows,
                          CUtensorMap* out) {
  return cuca_tensor_map_2d(ptr, 2, rows, cols, stride, box_rows, out);
}

bool cuca_tensor_map_2d(const void* ptr, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t stride,
                        uint32_t box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
  static std::mutex mu;
  if (elem_bytes != 2 && elem_bytes != 4) return false;
  MapKey key{ptr, rows, cols, stride, box_rows, elem_bytes};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {stride * (cuuint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

namespace {
template <int BN, bool DUAL, bool SWAP, bool TALL = false>
int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmO, const Params& p, int grid,
              cudaStream_t stream) {
  using C = Cfg<BN, DUAL, SWAP, TALL>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, DUAL, SWAP, TALL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM);
    if (e != cudaSuccess) {
      cuca_set_error("gemm_tc: cannot reserve %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e));
      return 2;
    }
    configured = true;
  }
  cuca_launch(gemm_tc_kernel<BN, DUAL, SWAP, TALL>, dim3(grid), dim3(C::THREADS), C::SMEM, stream, true, tmA, tmB, tmO, p);
  CUCA_CHECK_LAUNCH("gemm_tc");
  return 0;
}

template <bool DUAL>
int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmO, const Params& p, int grid,
                cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::SMEM);
    if (e != cudaSuccess) {
      cuca_set_error("gemm_tc: cannot reserve %d bytes of shared memory: %s", PairCfg::SMEM, cudaGetErrorString(e));
      return 2;
    }
    configured = true;
  }
  // as many pairs as are resident together (a cluster lies within one GPC, so an odd SM there stays idle)
  static int resident_pairs = 0;
  if (!resident_pairs) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (cuca_device_sms() / 2));
    cfg.blockDim = dim3(PairCfg::THREADS);
    cfg.dynamicSmemBytes = PairCfg::SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<DUAL>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = cuca_device_sms() / 2;
    }
    resident_pairs = n;
  }
  if (grid > 2 * resident_pairs) grid = 2 * resident_pairs;
  cudaError_t e = cuca_launch_cluster(gemm_pair_kernel<DUAL>, dim3(grid), dim3(PairCfg::THREADS), PairCfg::SMEM, stream, true, 2,
                                      tmA, tmB, tmO, p);
  if (e != cudaSuccess) {
    cuca_set_error("gemm_tc: launch of a pair kernel failed: %s", cudaGetErrorString(e));
    return 2;
  }
  CUCA_CHECK_LAUNCH("gemm_tc pair");
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

// K slices left unadded (cuca_gemm_tc_partial) over more than 128 tokens come from pairs of CTAs: a tile of 256
// tokens x 256 weight rows stages 32 KB per SM and K step where the one-SM forms stage 48 (and every CTA of the
// weights-as-rows form re-reads all tokens), and whole 32-row boxes of a slice leave through the copy engine.
constexpr int PAIR_PARTIAL_MAX_TOKENS = 512;
// Slices per tile of that form: the count that makes the rounds of (tile, slice) units over the pairs, times a
// unit's K steps plus about eight steps' worth of start and epilogue, the shortest; a step's worth per slice for
// what writing and re-reading it costs. (q/k/v at 512 tokens: 48 tiles as three slices each in two rounds of 22
// K steps, rather than one round of 64 on 48 of the 74 pairs.)
static int pair_partial_slices(int M, int N, int K, int max_slices) {
  const int pairs = cuca_device_sms() / 2;
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256), ksteps = (K + TILE_K - 1) / TILE_K;
  int best = 1;
  long long best_cost = -1;
  for (int n = 1; n <= max_slices && (n == 1 || 2 * n <= ksteps); ++n) {
    const long long rounds = ((long long)tiles * n + pairs - 1) / pairs;
    const long long cost = rounds * ((ksteps + n - 1) / n + 8) + n;
    if (best_cost < 0 || cost < best_cost) { best = n; best_cost = cost; }
  }
  return best;
}
static int sms_pairs() { return cuca_device_sms() / 2; }
static int allow_pair = -1;
static bool pair_partial_takes(int M, int N) {
  if (allow_pair < 0) { const char* e = getenv("CUCA_GEMM_PAIR"); allow_pair = e ? atoi(e) : 1; }
  // rows of the 32-bit output are 16-byte multiples (the copy engine stores them)
  return allow_pair != 0 && M > TILE_A && M <= PAIR_PARTIAL_MAX_TOKENS && N % 4 == 0 && cuca_device_sms() >= 2;
}

// When the two-SM form runs: 1 by the rule in gemm_tc_impl, 0 never, 2 wherever it can (tests and measurements),
// -1 as the environment variable CUCA_GEMM_PAIR says (1 without it).
CUCA_API void cuca_gemm_pair_mode(int mode) { allow_pair = mode; }

// out = epilogue(A[M,K] W[N,K]^T), bf16 operands. workspace/counters: scratch for tiles split along K
// (ws_bytes of 32-bit partials; n_counters zeroed ints, left zeroed). max_splits <= 1: whole tiles only.
static int gemm_tc_impl(const void* A, const void* W, const void* bias, void* out, int out_dtype, int M, int N,
                        int K, int lda, int ldo, int epilogue, void* workspace, size_t ws_bytes, int* counters,
                        int n_counters, int max_splits, int* n_slices_out, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (!cuca_gemm_tc_supported(A, W, M, N, K, lda)) return 1;
  CUCA_REQUIRE(epilogue != EPI_RESIDUAL || out_dtype == CUCA_F32, "gemm_tc: the residual stream is 32-bit");
  CUCA_REQUIRE(epilogue != EPI_SWIGLU || (bias == nullptr && out_dtype == CUCA_BF16), "gemm_tc: SwiGLU writes bf16, no bias");
  const bool dual = epilogue == EPI_SWIGLU;
  CUCA_REQUIRE(epilogue >= 0 && epilogue <= EPI_PARTIAL, "gemm_tc: unknown epilogue %d", epilogue);
  if (epilogue == EPI_PARTIAL && pair_partial_takes(M, N)) {
    CUCA_REQUIRE(out_dtype == CUCA_F32 && bias == nullptr && n_slices_out != nullptr && ((uintptr_t)out & 15) == 0, "gemm_tc: partial sums are 32-bit, without bias, in rows of 16-byte multiples");
    const int per_tile = pair_partial_slices(M, N, K, max_splits);
    const int slab_rows = (M + 31) / 32 * 32;
    CUtensorMap tmA, tmB, tmO;
    CUCA_REQUIRE(cuca_tensor_map_bf16(A, M, K, lda, TILE_A, &tmA), "gemm_tc: activation tensor map failed");
    CUCA_REQUIRE(cuca_tensor_map_bf16(W, N, K, K, 128, &tmB), "gemm_tc: weight tensor map failed");
    CUCA_REQUIRE(cuca_tensor_map_2d(out, 4, (uint64_t)per_tile * slab_rows, N, N, 32, &tmO), "gemm_tc: output tensor map failed");
    Params p;
    p.out = out; p.bias = nullptr; p.workspace = nullptr; p.counters = nullptr; p.err = err;
    p.M = M; p.N = N; p.K = K; p.ldo = N; p.epilogue = EPI_PARTIAL; p.out_f32 = 1;
    p.tile_rows = 2 * TILE_A;
    p.tiles_a = (M + 255) / 256;
    p.tiles = p.tiles_a * ((N + 255) / 256);
    p.ksteps = (K + TILE_K - 1) / TILE_K;
    p.tma_out = 1;
    p.ordered_add = p.skew = p.stream_k = p.pieces = p.piece_w = 0;
    p.per_tile = per_tile; p.max_parts = 1; p.slab_rows = slab_rows;
    *n_slices_out = per_tile;
    const long long units = (long long)p.tiles * per_tile;
    const int pairs = units < sms_pairs() ? (int)units : sms_pairs();
    return launch_pair<false>(tmA, tmB, tmO, p, 2 * pairs, stream);
  }
  const bool swap = M <= (epilogue == EPI_SWIGLU ? SWAP_MAX_TOKENS_SWIGLU : SWAP_MAX_TOKENS);
  const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const uint64_t w_rows = (uint64_t)N * (dual ? 2 : 1);
  CUtensorMap tmA, tmB, tmO;
  int tma_out = 0;
  if (swap) {
    CUCA_REQUIRE(cuca_tensor_map_bf16(W, w_rows, K, K, TILE_A, &tmA), "gemm_tc: weight tensor map failed");
    CUCA_REQUIRE(cuca_tensor_map_bf16(A, M, K, lda, bn, &tmB), "gemm_tc: activation tensor map failed");
  } else {
    CUCA_REQUIRE(cuca_tensor_map_bf16(A, M, K, lda, TILE_A, &tmA), "gemm_tc: activation tensor map failed");
    CUCA_REQUIRE(cuca_tensor_map_bf16(W, w_rows, K, K, 128, &tmB), "gemm_tc: weight tensor map failed");
    // whole tiles leave through the copy engine where the output's rows are 16-byte multiples
    const int esize = out_dtype == CUCA_F32 ? 4 : 2;
    if (((uintptr_t)out & 15) == 0 && ((size_t)ldo * esize) % 16 == 0)
      tma_out = cuca_tensor_map_2d(out, esize, M, N, ldo, 32, &tmO) ? 1 : 0;
  }
  if (!tma_out) tmO = tmA;  // unused
  Params p;
  p.out = out; p.bias = (const __nv_bfloat16*)bias; p.workspace = (float*)workspace; p.counters = counters;
  p.err = err; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.epilogue = epilogue; p.out_f32 = out_dtype == CUCA_F32;
  const int out_cols = swap ? bn : (dual ? 128 : 256);
  const int ncols = swap ? bn * (dual ? 2 : 1) : 256;
  const int sms = cuca_device_sms();
  const int tiles_b = swap ? (M + bn - 1) / bn : (N + out_cols - 1) / out_cols;
  // Many tokens, whole tiles through the copy engine: tiles of 256 tokens (the tall form, see Cfg) where they fill
  // the SMs in fewer rounds. Measured at 2,048 tokens on the Llama-3.1-8B widths, a tall tile takes 1.84 to 1.9
  // times a 128-row tile (three 64 KB stages hold less of a round trip than four of 48 KB, and the epilogue is
  // not hidden), so it pays only where it halves the rounds: output projection 58.3 -> 53.7 us (256 tiles in
  // two rounds -> 128 in one), down 193 -> 171 us; q/k/v (384 -> 192 tiles) and gate/up (1,792 -> 896) stay. From
  // 129 tokens on the same rule holds: gate/up at 256 tokens 70.0 -> 64.0 us, at 192 tokens 85.1 -> 74.8 (224 tiles
  // in two rounds -> 112 in one).
  // CUCA_GEMM_TALL=0 keeps the 128-row form everywhere, =2 takes the tall form wherever it is allowed.
  bool tall = false;
  if (!swap && tma_out && epilogue != EPI_PARTIAL && M > TILE_A) {
    static int allow = -1;
    if (allow < 0) { const char* e = getenv("CUCA_GEMM_TALL"); allow = e ? atoi(e) : 1; }
    const long long t128 = (long long)((M + TILE_A - 1) / TILE_A) * tiles_b;
    const long long t256 = (long long)((M + 2 * TILE_A - 1) / (2 * TILE_A)) * tiles_b;
    const long long rounds128 = (t128 + sms - 1) / sms, rounds256 = (t256 + sms - 1) / sms;
    tall = allow == 2 || (allow == 1 && rounds256 * 19 < rounds128 * 10);
  }
  // The two-SM form (gemm_pair_kernel): CUCA_GEMM_PAIR=0 never, =2 wherever it is allowed.
  bool pair = false;
  if (!swap && tma_out && epilogue != EPI_PARTIAL && M > TILE_A && sms >= 2) {
    if (allow_pair < 0) { const char* e = getenv("CUCA_GEMM_PAIR"); allow_pair = e ? atoi(e) : 1; }
    // Rounds of tiles times what a round costs in each form, in units of a 128 x 256 tile's time (measured on the
    // Llama-3.1-8B widths at 1,024 to 4,096 tokens: a tall tile 1.9 to 2.1, a pair's tile 0.93 to 0.97; with K above
    // 8,192 the pair lost to the tall form by 5 to 7 %, so it counts as 1.02 there).
    const long long t128 = (long long)((M + TILE_A - 1) / TILE_A) * tiles_b;
    const long long t256 = (long long)((M + 2 * TILE_A - 1) / (2 * TILE_A)) * tiles_b;
    const int pairs = sms / 2;
    const double cost128 = (double)((t128 + sms - 1) / sms);
    const double cost_tall = (double)((t256 + sms - 1) / sms) * 1.95;
    const double cost_pair = (double)((t256 + pairs - 1) / pairs) * (K > 8192 ? 1.02 : 0.96);
    pair = allow_pair == 2 || (allow_pair == 1 && t256 >= pairs && cost_pair < cost128 && cost_pair < (tall ? cost_tall : 1e30));
  }
  if (pair) {
    p.tile_rows = 2 * TILE_A;
    p.tiles_a = (M + p.tile_rows - 1) / p.tile_rows;
    p.tiles = p.tiles_a * tiles_b;
    p.ksteps = (K + TILE_K - 1) / TILE_K;
    p.tma_out = 1;
    p.ordered_add = p.skew = p.stream_k = p.pieces = p.piece_w = 0;
    p.per_tile = p.max_parts = 1;
    p.slab_rows = 0;
    const int pairs = p.tiles < sms / 2 ? p.tiles : sms / 2;
    return dual ? launch_pair<true>(tmA, tmB, tmO, p, 2 * pairs, stream) : launch_pair<false>(tmA, tmB, tmO, p, 2 * pairs, stream);
  }
  p.tile_rows = tall ? 2 * TILE_A : TILE_A;
  p.tiles_a = swap ? (N + TILE_A - 1) / TILE_A : (M + p.tile_rows - 1) / p.tile_rows;
  p.tiles = p.tiles_a * tiles_b;
  p.ksteps = (K + TILE_K - 1) / TILE_K;
  const long long units = (long long)p.tiles * p.ksteps;
  int grid = p.tiles < sms ? p.tiles : sms;
  p.tma_out = tma_out;
  p.ordered_add = 0;
  p.skew = 0;
  p.stream_k = 0;
  p.pieces = p.piece_w = 0;
  p.per_tile = 1;
  p.max_parts = 1;
  // Tokens as rows (more than 256 of them), fewer tiles than SMs, K not long: column pieces as narrow as it takes for about one per SM,
  // each over all of K, so nothing is added up afterwards. (Measured at 256 tokens, K = 4096: 31 us against 57 us
  // with K slices; with K = 14336 no gain. A piece's main loop runs at the pace of its loads, 4 stages deep, not
  // of its MMAs, so a piece takes as long as a whole tile: cutting the last round of many tiles this way gains
  // nothing and is not done.)
  bool pieced = false;
  if (tall) {
    // whole tiles in turn, nothing split
  } else if (!swap && !dual && p.tiles < sms && p.ksteps <= 128) {
    const int unit = out_dtype == CUCA_F32 ? 32 : 64;  // whole 128-byte runs of the epilogue
    for (int w = unit; w < out_cols && !pieced; w += unit) {
      const int pieces = p.tiles_a * ((N + w - 1) / w);
      if (pieces > sms) continue;
      if (pieces * 2 < sms || pieces <= p.tiles) break;  // too few even at the narrowest: K is shared out below instead
      pieced = true;
      p.pieces = pieces;
      p.piece_w = w;
      grid = pieces;
    }
  }
  if (pieced || tall) {
  } else if (epilogue == EPI_PARTIAL) {
    CUCA_REQUIRE(swap && out_dtype == CUCA_F32 && bias == nullptr && n_slices_out != nullptr,
                 "gemm_tc: partial sums are for up to %d tokens, 32-bit, without bias", SWAP_MAX_TOKENS);
    int per_tile = sms / p.tiles;
    if (per_tile > max_splits) per_tile = max_splits;
    if (per_tile > p.ksteps / 2) per_tile = p.ksteps / 2;
    if (per_tile < 1) per_tile = 1;
    if (p.tiles > sms) per_tile = 1;
    *n_slices_out = per_tile;
    if (p.tiles <= sms) {
      p.stream_k = 2;
      p.per_tile = per_tile;
      grid = per_tile * p.tiles;
    }
  } else if (workspace && counters && max_splits > 1 && p.tiles < (swap ? 2 * sms : sms) && p.tiles <= n_counters &&
             p.ksteps >= 2 && p.tiles % sms != 0) {  // whole tiles in turn would leave SMs idle
    // If a whole number of CTAs per tile fills most of the GPU, every CTA gets one even K slice of one tile (one
    // accumulator drain each); else the K steps are dealt out evenly across tile borders.
    const int per_tile = sms / p.tiles;
    if (per_tile >= 1 && (long long)per_tile * p.tiles * 4 >= 3LL * sms && p.ksteps >= 2 * per_tile) {
      size_t need = (size_t)p.tiles * per_tile * ncols * TILE_A * sizeof(float);
      if (per_tile == 1) {
        grid = p.tiles;  // one CTA per tile, nothing to add up
      } else if (!swap && tma_out && epilogue == EPI_RESIDUAL) {
        p.stream_k = 2;
        p.per_tile = per_tile;
        p.ordered_add = 1;
        // a turn (adds performed, fence, counter, the next slice's poll) takes about as long as 14 K steps (measured
        // at 256 tokens, K = 14336, four slices: 63.5 us with even slices, 55.3 with 14, 57.3 with 8 or 20)
        const int most = p.ksteps / (per_tile * (per_tile + 1) / 2);  // the first slice keeps at least `skew` steps
        p.skew = 14 < most ? 14 : most;
        grid = per_tile * p.tiles;
      } else if (need <= ws_bytes) {
        p.stream_k = 2;
        p.per_tile = per_tile;
        p.max_parts = per_tile;
        grid = per_tile * p.tiles;
      }
    } else if (!swap && 2 * p.tiles >= sms) {
      // many tokens, tiles for more than half of the SMs: one whole tile per CTA. Dealing the K steps out over all
      // SMs costs more in the last-arriver reduction than the idle SMs do (768 tokens, down projection of the
      // Llama-3.1-8B widths, 96 tiles: 127.6 us dealt out).
      grid = p.tiles;
    } else {
      long long g = units / 2 < sms ? units / 2 : sms;
      long long per = units / g;  // smallest share
      int parts = (int)((p.ksteps + per - 1) / per) + 1;
      size_t need = (size_t)p.tiles * parts * ncols * TILE_A * sizeof(float);
      if (g > p.tiles && need <= ws_bytes) {
        p.stream_k = 1;
        p.max_parts = parts;
        grid = (int)g;
      }
    }
  }
#define GO(BN_)                                                                                       \
  case BN_:                                                                                           \
    return dual ? launch_tc<BN_, true, true>(tmA, tmB, tmO, p, grid, stream)                               \
                : launch_tc<BN_, false, true>(tmA, tmB, tmO, p, grid, stream);
  if (swap) {
    switch (bn) { GO(16) GO(32) GO(64) }
    return bn == 128 ? launch_tc<128, false, true>(tmA, tmB, tmO, p, grid, stream)  // 65..256 tokens, never SwiGLU
                     : launch_tc<256, false, true>(tmA, tmB, tmO, p, grid, stream);
  }
#undef GO
  // column pieces up to 128 wide: stages of 128 weight rows, so that six instead of four fit (a piece's main loop
  // runs at the pace of its loads)
  if (pieced && p.piece_w <= 128) return launch_tc<128, false, false>(tmA, tmB, tmO, p, grid, stream);
  if (tall)
    return dual ? launch_tc<256, true, false, true>(tmA, tmB, tmO, p, grid, stream)
                : launch_tc<256, false, false, true>(tmA, tmB, tmO, p, grid, stream);
  return dual ? launch_tc<256, true, false>(tmA, tmB, tmO, p, grid, stream)
              : launch_tc<256, false, false>(tmA, tmB, tmO, p, grid, stream);
}

CUCA_API int cuca_gemm_tc(const void* A, const void* W, const void* bias, void* out, int out_dtype, int M, int N,
                          int K, int lda, int ldo, int epilogue, void* workspace, size_t ws_bytes, int* counters,
                          int n_counters, int max_splits, int* err, cudaStream_t stream) {
  CUCA_REQUIRE(epilogue != EPI_PARTIAL, "gemm_tc: use cuca_gemm_tc_partial for partial sums");
  return gemm_tc_impl(A, W, bias, out, out_dtype, M, N, K, lda, ldo, epilogue, workspace, ws_bytes, counters,
                      n_counters, max_splits, nullptr, err, stream);
}

CUCA_API int cuca_gemm_tc_partial_max_tokens() { return pair_partial_takes(PAIR_PARTIAL_MAX_TOKENS, 4) ? PAIR_PARTIAL_MAX_TOKENS : SWAP_MAX_TOKENS; }

// Rows of one slice's slab in the output of cuca_gemm_tc_partial for this many tokens (at least M; the two-SM form
// stores whole boxes of 32 rows, so its slabs are padded to a multiple of 32) and N features.
CUCA_API int cuca_gemm_tc_partial_rows(int M, int N) { return pair_partial_takes(M, N) ? (M + 31) / 32 * 32 : M; }

// How many K slices cuca_gemm_tc_partial will write for this shape (the first dimension of its output).
CUCA_API int cuca_gemm_tc_partial_slices(int M, int N, int K, int max_slices) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (pair_partial_takes(M, N)) return pair_partial_slices(M, N, K, max_slices);
  if (M > SWAP_MAX_TOKENS) return 0;
  const int sms = cuca_device_sms();
  const int tiles = (N + TILE_A - 1) / TILE_A, ksteps = (K + TILE_K - 1) / TILE_K;
  int per_tile = sms / tiles;
  if (per_tile > max_slices) per_tile = max_slices;
  if (per_tile > ksteps / 2) per_tile = ksteps / 2;
  if (per_tile < 1 || tiles > sms) per_tile = 1;
  return per_tile;
}

// partial[slice][rows][N] (32-bit) = A[M, K slice] W[N, K slice]^T for up to cuca_gemm_tc_partial_max_tokens()
// tokens, rows = cuca_gemm_tc_partial_rows(M): the K slices of a tile are not added up here (no workspace, no
// counters, no second pass); the kernel that reads the result adds them in slice order. *n_slices gets the number
// of slices written (cuca_gemm_tc_partial_slices of the same shape).
CUCA_API int cuca_gemm_tc_partial(const void* A, const void* W, float* partial, int M, int N, int K, int lda,
                                  int max_slices, int* n_slices, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  return gemm_tc_impl(A, W, nullptr, partial, CUCA_F32, M, N, K, lda, N, EPI_PARTIAL, nullptr, 0, nullptr, 0,
                      max_slices, n_slices, err, stream);
}


// ------------------------------------------------------------------ a wait that runs out (for the tests)
namespace {
__global__ void wait_probe_kernel(unsigned long long limit_ns, int* err, int* report) {
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // two roles, as in the contraction: each waits for a phase that nothing ever completes. The first to run out
  // of time records the error and raises the CTA's abort flag; the other sees the flag and gives up too.
  if (threadIdx.x == 0) report[0] = mbar_wait(&bars[0], 0, err, &abort_flag, limit_ns) ? 1 : 0;
  if (threadIdx.x == 32) report[1] = mbar_wait(&bars[1], 0, err, &abort_flag, 1000ull * limit_ns) ? 1 : 0;
  __syncthreads();
  if (threadIdx.x == 0) report[2] = abort_flag;
}
}  // namespace

// The kernels of this library never wait without a limit: a wait that runs out records CUCA_ERR_WAIT_TIMEOUT in
// the error word, tells the CTA's other roles to give up, and the kernel returns. This entry shows that path on
// its own: two threads wait (for `limit_ns`, and for a thousand times that) on barriers nobody arrives at.
// report[0..1]: whether the waits succeeded (both 0), report[2]: the abort flag (1).
CUCA_API int cuca_wait_probe(unsigned long long limit_ns, int* err, int* report, cudaStream_t stream) {
  CUCA_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ull, "wait_probe: a limit of %llu ns (at most 0.1 s)", limit_ns);
  wait_probe_kernel<<<1, 64, 0, stream>>>(limit_ns, err, report);
  CUCA_CHECK_LAUNCH("wait_probe");
  return 0;
}
