// Paged causal attention for prompt portions on the 5th-generation tensor cores (bfloat16, head size 64 or 128).
//
// A CTA takes up to 128 consecutive rows of one request and one query head and walks the request's keys in
// tiles of 64 positions. Both contractions run as tcgen05.mma with accumulators in tensor memory:
//
//   S[128 rows, 64 keys]   = Q K^T        (Q and K tiles K-major in shared memory, loaded by TMA from the
//                                          q buffer and straight from the pages through the block table)
//   O[128 rows, head size] += P V         (P written by the softmax threads as bf16 into the tensor memory that
//                                          held S: the A operand comes from there; V tiles as loaded, i.e.
//                                          the MN-major B operand)
//
// Warp 0 issues TMA, one thread per query tile issues its MMAs, four warps per query tile own one query row per
// thread (= one TMEM lane): they read S with tcgen05.ld, scale, mask (causal, window), keep the running maximum and sum in
// 32-bit, rescale O in tensor memory, and hand P back.
//
// A kernel that allocates tensor memory gets one CTA per SM, so the overlap of softmax and tensor pipe has to
// happen inside the CTA: it takes the same rows for TWO query heads of one key/value head (when the group size is
// even; else one), with four softmax warps each. Both tiles read the same K and V tiles; while the softmax threads
// of one work on its scores, the tensor pipe runs the other's P V and its next scores.
//
// Every mbarrier wait is bounded; on a timeout the kernel records CUCA_ERR_WAIT_TIMEOUT, all roles stop, TMEM
// is freed and the kernel returns.
#include "tcgen05.cuh"
#include <math.h>
#include <stdlib.h>

namespace {

constexpr int ROWS = 128;     // query rows per tile = TMEM lanes
constexpr int KEYS = 64;      // keys per tile
constexpr int NQ = 2;         // query tiles per CTA (two query heads of one key/value group, same rows)
// Tiles are stored as 64-element halves: [halves][rows][128 B], 128-byte swizzled.
constexpr int Q_HALF = ROWS * 128;               // 16 KB; a Q tile has D / 64 of them
constexpr int KV_HALF = KEYS * 128;              // a K or V tile [keys][D] has D / 64 of them
constexpr int BAR_BYTES = 256;                   // mbarriers, the TMEM address, the abort flag: behind the tiles
constexpr int TMEM_COLS = 512;                   // two S buffers per query tile (4 x 64 columns), O of both (2 x D)
constexpr int NTHREADS = 64 + NQ * 128 + 32;     // warp 0 TMA, warp 1 MMA of query tile 0, four softmax warps per query
                                                 // tile, last warp MMA of query tile 1
// What depends on the head size D (64 or 128).
template <int D>
struct Shape {
  static constexpr int Q_BYTES = (D / 64) * Q_HALF;
  static constexpr int KV_TILE = (D / 64) * KV_HALF;
  static constexpr int KV_STAGES = D == 128 ? 5 : 8;
  static constexpr int TILES_BYTES = NQ * Q_BYTES + KV_STAGES * 2 * KV_TILE;   // 224 KB / 192 KB
  static constexpr int DYN_SMEM = TILES_BYTES + BAR_BYTES + 1024;  // + what aligning the tiles to 1024 bytes may cost
};

struct Params {
  __nv_bfloat16* out;
  int out_stride;
  const int* tables;
  int table_stride;
  const int* positions;
  const int* seq_of_row;
  const int* tile_row0;
  const int* tile_nrows;
  int n_blocks, bs, nh, nkv;
  int heads_per_cta;     // 2: a CTA takes two query heads of one key/value head (even group size); else 1
  int n_tiles;           // tiles of the launch (heaviest first)
  int pair_tiles;        // 1: CTA b takes tile b and then tile n_tiles - 1 - b (a heavy and a light one)
  float scale_log2e;
  int window;
  int* err;
};

// test_wait never suspends the thread (try_wait may, for a time the hardware chooses): for loops that watch
// several barriers at once
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// the same with the A operand in tensor memory: row i in lane i, two bf16 per 32-bit column (K = 16 is 8 columns)
__device__ __forceinline__ void umma_bf16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st32_raw(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {  // ex2.approx: exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// as tmem_ld32 without the wait: several loads can be in flight before one tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major operand tile (the V tile as loaded: one key per 128-byte row of 64 head dimensions): 64 elements
// of N contiguous, the next 64 at `lbo` bytes, 8-key groups `sbo` bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// bf16 x bf16 -> f32, M = 128, N = n; b_mn: the B operand is MN-major
__host__ __device__ constexpr uint32_t instr_desc_b(bool b_mn, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

template <int D>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const Params p) {
  using SH = Shape<D>;
  constexpr int Q_BYTES = SH::Q_BYTES, KV_TILE = SH::KV_TILE, KV_STAGES = SH::KV_STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;                                  // NQ Q tiles
  uint8_t* kv_s = q_s + NQ * Q_BYTES;                   // KV_STAGES x (K tile + V tile)
  uint64_t* bars = (uint64_t*)(kv_s + KV_STAGES * 2 * KV_TILE);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;              // [KV_STAGES]
  uint64_t* kv_empty = kv_full + KV_STAGES;  // [KV_STAGES]
  uint64_t* s_full = kv_empty + KV_STAGES;   // [NQ][2] the scores of an even / odd key tile are in tensor memory
  uint64_t* p_full = s_full + 2 * NQ;        // [NQ] P is in tensor memory and O is rescaled (128 arrivals)
  uint64_t* pv_done = p_full + NQ;           // [NQ] the P V contraction of a tile has finished
  uint32_t* tmem_slot = (uint32_t*)(pv_done + NQ);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  if (smem + SH::TILES_BYTES + BAR_BYTES > smem_raw + SH::DYN_SMEM) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, CUCA_ERR_SMEM_LAYOUT);
    return;
  }
  // This CTA's query tiles: the same rows for `nq` consecutive query heads, which share their key/value head.
  const int nq = p.heads_per_cta;             // 1 or NQ
  const int head0 = blockIdx.y * nq;
  const int kvh = head0 / (p.nh / p.nkv);
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  // One tile, or two in turn: with a causal mask the tiles of a prompt differ in their keys by up to the prompt's
  // length, and the host's list has the heaviest first, so CTA b takes tile b and then tile n - 1 - b: equal work
  // for every CTA and one round of CTAs where the tiles alone would need two (a 2,048-token prompt of the
  // Llama-3.1-8B shape: 256 tiles x head pairs on 148 SMs). Between the two the barriers are set up anew.
  const int second = p.n_tiles - 1 - (int)blockIdx.x;
  const int n_items = (p.pair_tiles && second != (int)blockIdx.x) ? 2 : 1;
  uint32_t tmem_base = 0;
  for (int item = 0; item < n_items; ++item) {
  const int tile = item == 0 ? (int)blockIdx.x : second;
  const int row0 = p.tile_row0[tile], n_rows = p.tile_nrows[tile];
  const int seq = p.seq_of_row[row0];
  const int pos0 = p.positions[row0];
  const int lo_min = (p.window > 0 && pos0 - (p.window - 1) > 0) ? pos0 - (p.window - 1) : 0;
  const int hi = pos0 + n_rows;                       // keys [lo_min, hi) matter
  const int first_tile = lo_min / KEYS;
  const int n_tiles = (hi - 1) / KEYS - first_tile + 1;
  const int* table = p.tables + (size_t)(seq < 0 ? 0 : seq) * p.table_stride;

  if (threadIdx.x == 0) {
    if (item > 0) {
      // every thread has left the first tile (the barrier below it): its barriers are dead and set up again
      for (uint64_t* b = bars; b < (uint64_t*)tmem_slot; ++b)
        asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(b)) : "memory");
    }
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], nq); }  // one commit per query tile
    for (int x = 0; x < NQ; ++x) {
      mbar_init(&s_full[2 * x], 1);
      mbar_init(&s_full[2 * x + 1], 1);
      mbar_init(&p_full[x], 128);
      mbar_init(&pv_done[x], 1);
    }
    if (item == 0) *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  tmem_base = *tmem_slot;
  // query tile x: scores of key tile t in columns [64 (2 x + t % 2), + 64), output in [256 + 128 x, + 128)
  auto tmem_s = [&](int x, int t) { return tmem_base + (uint32_t)((2 * x + (t & 1)) * KEYS); };
  auto tmem_o = [&](int x) { return tmem_base + (uint32_t)(2 * NQ * KEYS + x * D); };

  if (seq < 0) {
    // a tile of padding rows: nothing to do
  } else
  if (warp == 0) {
    // ------------------------------------------------ producer: the Q tiles once, then K and V tiles page by page.
    // Lane 0 issues the copies; the warp reads the block table 32 entries at a time (one coalesced load for
    // several tiles ahead), so no copy waits for a table lookup of its own.
    if (lane == 0) {
      mbar_expect_tx(q_full, nq * Q_BYTES);
      for (int x = 0; x < nq; ++x) {
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_load_2d(q_s + x * Q_BYTES + h * Q_HALF, &tmQ, q_full, (head0 + x) * D + h * 64, row0);
      }
    }
    const int pages = KEYS / p.bs;          // pages per key tile: 1..8
    const int per_batch = 32 / pages;       // key tiles whose table entries one load brings
    int entry = 0;
    for (int j = 0; j < n_tiles; ++j) {
      const int in_batch = j % per_batch;
      if (in_batch == 0) {
        const int tj = j + lane / pages;
        const int kp = (first_tile + tj) * KEYS + (lane % pages) * p.bs;
        entry = (lane < per_batch * pages && tj < n_tiles && kp < hi) ? table[kp / p.bs] : 0;
      }
      const int s = j % KV_STAGES;
      int ok = 1;
      if (lane == 0 && j >= KV_STAGES) ok = mbar_wait(&kv_empty[s], ((j / KV_STAGES) & 1) ^ 1, p.err, abort_flag) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      uint8_t* ks = kv_s + s * 2 * KV_TILE;
      uint8_t* vs = ks + KV_TILE;
      if (lane == 0) mbar_expect_tx(&kv_full[s], 2 * KV_TILE);
      __syncwarp();
      // one copy per lane: a page needs four (keys and values, two 64-wide halves each), a tile has up to 8 pages;
      // a single thread would need about as long to issue them as the tensor pipe needs for the tile
      const int pg = lane >> 2, which = lane & 3;
      int blk = __shfl_sync(0xffffffffu, entry, in_batch * pages + (pg < pages ? pg : 0));
      if (pg < pages && (which & 1) < D / 64) {
        const int kp = (first_tile + j) * KEYS + pg * p.bs;
        if (blk < 0 || blk >= p.n_blocks) {
          // keys before the window may have given their page back; they are masked. Anything else is an error.
          if (kp + p.bs > lo_min && kp < hi && p.err) atomicExch(p.err, CUCA_ERR_BLOCK_RANGE);
          blk = 0;
        }
        const int grow = (blk * p.nkv + kvh) * p.bs;  // row of the page in the pool seen as [rows][D]
        uint8_t* dst = ((which & 2) ? vs : ks) + ((which & 1) ? KV_HALF : 0) + pg * p.bs * 128;  // bs rows of 128 B
        tma_load_2d(dst, (which & 2) ? &tmV : &tmK, &kv_full[s], (which & 1) ? 64 : 0, grow);
      }
    }
  } else if ((warp == 1 || warp == 2 + 4 * NQ) && lane == 0) {
    // ------------------------------------------------ MMA issuers: one thread per query tile
    // Scores run one key tile ahead of the softmax: each query tile has two S buffers, so when its softmax threads
    // hand over P of key tile j, the scores of j + 1 are already there and those of j + 2 are requested behind the
    // P V of j. The two query tiles share the tensor pipe; each has a thread of its own that issues whatever of its
    // tile is ready (keys landed and an S buffer free -> scores; P handed over -> P V). One thread for both spent
    // 3,100 cycles per key tile issuing (24 MMAs, their descriptors, 6 commits, the polls) while the tensor pipe
    // needed 1,400 and the softmax threads waited 1,600 of their 3,000 for scores. A key/value stage goes back to
    // the producer after both tiles' P V of it (an arrival count of two).
    const int x = warp == 1 ? 0 : 1;
    constexpr uint32_t idesc_qk = instr_desc_b(false, KEYS), idesc_pv = instr_desc_b(true, D);
    bool ok = x < nq && mbar_wait(q_full, 0, p.err, abort_flag);
    // descriptors once: a tile's further K steps are constant offsets of its first (the address field counts 16 bytes)
    const uint64_t q_desc = smem_desc(smem_u32(q_s + x * Q_BYTES));
    uint64_t k_desc[KV_STAGES], v_desc[KV_STAGES];
#pragma unroll
    for (int st = 0; st < KV_STAGES; ++st) {
      k_desc[st] = smem_desc(smem_u32(kv_s + st * 2 * KV_TILE));
      v_desc[st] = desc_mnmajor(smem_u32(kv_s + st * 2 * KV_TILE + KV_TILE), KV_HALF, 1024);
    }
    auto stage_desc = [&](const uint64_t (&d)[KV_STAGES], int st) {  // registers, not local memory
      uint64_t r = d[0];
#pragma unroll
      for (int i = 1; i < KV_STAGES; ++i) r = st == i ? d[i] : r;
      return r;
    };
    // The second query tile starts when the first has handed over its first P: from then on one tile's exponents
    // (XU pipe) run while the other's contractions do (tensor pipe), instead of both tiles doing the same thing at
    // the same time and leaving the other pipe idle.
    if (ok && x == 1 && n_tiles > 1) ok = mbar_wait(&p_full[0], 0, p.err, abort_flag);
    int next_sc = 0, next_pv = 0;
    unsigned long long idle_since = 0;
    unsigned spins = 0;
    while (ok && next_pv < n_tiles) {
      bool progressed = false;
      // scores of key tile t need its keys and the S buffer that the softmax of t - 2 has let go
      if (next_sc < n_tiles && next_sc <= next_pv + 1 &&
          mbar_test_wait(&kv_full[next_sc % KV_STAGES], (next_sc / KV_STAGES) & 1)) {
        const int t = next_sc;
        tc_fence_after();
        const uint64_t kd = stage_desc(k_desc, t % KV_STAGES);
        const uint32_t acc = tmem_s(x, t);
        // S_x[t % 2] = Q_x K_t^T: 8 steps of 16 head dimensions, 32 bytes inside a 64-wide half
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(acc, q_desc + (uint64_t)(((k / 4) * Q_HALF + (k % 4) * 32) >> 4),
                    kd + (uint64_t)(((k / 4) * KV_HALF + (k % 4) * 32) >> 4), idesc_qk, k > 0);
        umma_commit(&s_full[2 * x + (t & 1)]);
        ++next_sc;
        progressed = true;
      }
      if (next_pv < next_sc && mbar_test_wait(&p_full[x], next_pv & 1)) {
        // O_x += P_x V_j: the softmax threads of tile x have written P and rescaled O
        const int j = next_pv, st = j % KV_STAGES;
        tc_fence_after();
        const uint64_t vd = stage_desc(v_desc, st);
        const uint32_t acc = tmem_o(x);
#pragma unroll
        for (int k = 0; k < KEYS / 16; ++k) {
          // A = P[rows][keys] in tensor memory, where the scores of this key tile were: 16 keys = 8 columns.
          // B = V[keys][dims] MN-major: 16 keys = two 8-key groups of 1024 bytes; dims 64..127 in the second half.
          umma_bf16_tmem_a(acc, tmem_s(x, j) + k * 8, vd + (uint64_t)((k * 2048) >> 4), idesc_pv, (j > 0 || k > 0));
        }
        umma_commit(&kv_empty[st]);
        umma_commit(&pv_done[x]);
        ++next_pv;
        progressed = true;
      }
      if (progressed) {
        idle_since = 0;
      } else if ((++spins & 63u) == 0) {
        if (*abort_flag) break;
        const unsigned long long now = global_ns();
        if (idle_since == 0) idle_since = now;
        else if (now - idle_since > WAIT_LIMIT_NS) {
          if (p.err) atomicExch(p.err, CUCA_ERR_WAIT_TIMEOUT);
          *abort_flag = 1;
          break;
        }
      }
    }
  } else if (warp >= 2 && warp < 2 + 4 * NQ) {
    // ------------------------------------------------ softmax: one query row per thread, four warps per tile
    const int x = (warp - 2) >> 2;              // which query tile
    const int quarter = warp & 3;               // the TMEM lanes this warp may touch
    const int r = quarter * 32 + lane;
    const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
    const bool row_ok = r < n_rows;
    const int row_pos = pos0 + r;
    const int row_lo = (p.window > 0 && row_pos - (p.window - 1) > 0) ? row_pos - (p.window - 1) : 0;
    float m = -INFINITY, l = 0.f;
    bool ok = x < nq;
    for (int j = 0; ok && j < n_tiles; ++j) {
      // the tcgen05.ld/st below are warp-wide: a warp leaves the loop together or not at all
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[2 * x + (j & 1)], (j >> 1) & 1, p.err, abort_flag))) { ok = false; break; }
      tc_fence_after();
      const int key0 = (first_tile + j) * KEYS;
      const bool whole = key0 >= lo_min && key0 + KEYS - 1 <= pos0 && (p.window <= 0 || key0 >= pos0 + ROWS - 1 - (p.window - 1));
      // pass 1: the whole row of scores in one round trip to tensor memory, then scale, mask, maximum
      constexpr int NC = KEYS / 32;  // groups of 32 scores
      uint32_t raw[NC][32];
#pragma unroll
      for (int c = 0; c < NC; ++c) tmem_ld32_nowait(tmem_s(x, j) + lane_bits + c * 32, raw[c]);
      tmem_ld_wait();
      // the scale is positive, so the maximum is taken over the raw scores and scaled once; the scaling of every
      // score happens inside the exponent's multiply-add
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (whole) {
        // every row of the tile sees every key of the tile: no tests in the loop (most tiles of a long prompt)
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(raw[c][i]));
      } else {
#pragma unroll
        for (int c = 0; c < NC; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kp = key0 + c * 32 + i;
            if (!(row_ok && kp <= row_pos && kp >= row_lo)) raw[c][i] = 0xff800000u;  // -inf
            mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(raw[c][i]));
          }
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2e;
      // The running maximum only moves when the new one exceeds it by more than 8 (in log2 units): values up to
      // 2^8 above the reference are exact enough in 32-bit sums, and O is rescaled far less often.
      float m_new = m;
      if (mx > m + 8.f || m == -INFINITY) m_new = fmaxf(m, mx);
      const float corr = (m_new == -INFINITY || m == m_new) ? 1.f : fast_exp2(m - m_new);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      // pass 2: P = exp2(s - m) as bf16, two keys per 32-bit column, into the first columns of the tensor memory
      // that held this tile's scores (every thread has read its row of them), and the row sum. The tensor core
      // takes P from there as the A operand of P V: no trip through shared memory.
      // (multiply-add and sum on pairs, in packed 32-bit arithmetic: the loop is bound by instruction issue)
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t pw[KEYS / 2];
      const float2 scale2 = make_float2(p.scale_log2e, p.scale_log2e), neg_m2 = make_float2(-m_use, -m_use);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float2 x2 = __ffma2_rn(make_float2(__uint_as_float(raw[c][2 * e]), __uint_as_float(raw[c][2 * e + 1])), scale2, neg_m2);
          const float2 p2 = make_float2(fast_exp2(x2.x), fast_exp2(x2.y));
          sum2[e & 1] = __fadd2_rn(sum2[e & 1], p2);
          __nv_bfloat162 t2 = __floats2bfloat162_rn(p2.x, p2.y);
          pw[c * 16 + e] = *reinterpret_cast<uint32_t*>(&t2);
        }
      }
      static_assert(KEYS == 64, "one 32-column store holds the P row of a 64-key tile");
      tmem_st32_raw(tmem_s(x, j) + lane_bits, pw);
      l = l * corr + (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
      m = m_new;
      // the previous P V of this tile must have finished before O is rescaled (its phase is awaited every time, so
      // that the barrier never runs two phases ahead of its waiters)
      if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(&pv_done[x], (j - 1) & 1, p.err, abort_flag))) { ok = false; break; }
      tc_fence_after();
      // rescale O (not yet written on the first tile).
      // tcgen05.ld/st are warp-wide: the whole warp rescales if any of its rows moved its maximum
      if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          tmem_ld32(tmem_o(x) + lane_bits + c * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= corr;
          tmem_st32(tmem_o(x) + lane_bits + c * 32, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[x]);
    }
    if (ok && __all_sync(0xffffffffu, mbar_wait(&pv_done[x], (n_tiles - 1) & 1, p.err, abort_flag))) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (size_t)(row0 + r) * p.out_stride + (size_t)(head0 + x) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tmem_ld32(tmem_o(x) + lane_bits + c * 32, o);  // warp-wide: every lane reads, only rows of the tile store
        if (row_ok) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 t2 = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
            w[i] = *reinterpret_cast<uint32_t*>(&t2);
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = make_uint4(w[4 * q4], w[4 * q4 + 1], w[4 * q4 + 2], w[4 * q4 + 3]);
        }
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();  // every role is done with this tile: its barriers may be set up anew, tensor memory reused
  if (*abort_flag) break;
  }
  if (*abort_flag) {
    unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ host side
template <int D>
int launch_attn_tc(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const Params& p, int n_tiles,
                   cudaStream_t stream) {
  const int smem = Shape<D>::DYN_SMEM;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    CUCA_REQUIRE(e == cudaSuccess, "attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", smem,
                 cudaGetErrorString(e));
    configured = true;
  }
  const int grid_x = p.pair_tiles ? (n_tiles + 1) / 2 : n_tiles;
  cuca_launch(attn_tc_kernel<D>, dim3(grid_x, p.nh / p.heads_per_cta), dim3(NTHREADS), smem, stream, true, tmQ, tmK, tmV, p);
  CUCA_CHECK_LAUNCH("attention_prefill_tc");
  return 0;
}

}  // namespace

// 1 if the tcgen05 prefill attention takes this shape: head size 64 or 128, pages of 8..64 positions (a power of
// two), rows of the q buffer and the pools 16-byte aligned.
CUCA_API int cuca_attention_tc_supported(int nh, int nkv, int d, int bs, int q_stride, int out_stride, const void* q,
                                         const void* kpool, const void* vpool) {
  if ((d != 64 && d != 128) || nkv <= 0 || nh % nkv != 0) return 0;
  if (bs < 8 || bs > KEYS || (bs & (bs - 1)) != 0) return 0;
  if (q_stride % 8 != 0 || out_stride % 8 != 0) return 0;
  if (((uintptr_t)q & 15) || ((uintptr_t)kpool & 15) || ((uintptr_t)vpool & 15)) return 0;
  return 1;
}

// Two tiles per CTA in the tcgen05 prefill attention: 1 where it makes one round of CTAs out of more, 0 never, 2
// whenever a launch has two tiles (tests), -1 as the environment variable CUCA_ATTN_PAIR_TILES says (1 without it).
static int pair_mode = -1;
CUCA_API void cuca_attention_pair_tiles_mode(int mode) { pair_mode = mode; }

// Prefill form on tcgen05: tile i covers rows tile_row0[i] .. +tile_nrows[i]-1 (at most 128 consecutive rows of
// one request). q: [n_rows_total][q_stride] with the rotated query heads first; out: [..][out_stride].
CUCA_API int cuca_attention_prefill_tc(const void* q, int q_stride, int n_rows_total, void* out, int out_stride,
                                       const void* kpool, const void* vpool, int n_blocks, int bs,
                                       const int* positions, const int* seq_of_row, const int* tables,
                                       int table_stride, const int* tile_row0, const int* tile_nrows, int n_tiles,
                                       int nh, int nkv, int d, float scale, int window, int* err,
                                       cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  CUCA_REQUIRE(cuca_attention_tc_supported(nh, nkv, d, bs, q_stride, out_stride, q, kpool, vpool),
               "attention_prefill_tc: unsupported shape (heads %d/%d, head size %d, page %d)", nh, nkv, d, bs);
  CUCA_REQUIRE(nh <= 65535, "attention_prefill_tc: too many heads");
  CUtensorMap tmQ, tmK, tmV;
  CUCA_REQUIRE(cuca_tensor_map_bf16(q, n_rows_total, (uint64_t)nh * d, q_stride, ROWS, &tmQ), "attention_prefill_tc: q tensor map failed");
  const uint64_t pool_rows = (uint64_t)n_blocks * nkv * bs;
  CUCA_REQUIRE(cuca_tensor_map_bf16(kpool, pool_rows, d, d, bs, &tmK), "attention_prefill_tc: key tensor map failed");
  CUCA_REQUIRE(cuca_tensor_map_bf16(vpool, pool_rows, d, d, bs, &tmV), "attention_prefill_tc: value tensor map failed");
  Params p;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride; p.tables = tables; p.table_stride = table_stride;
  p.positions = positions; p.seq_of_row = seq_of_row; p.tile_row0 = tile_row0; p.tile_nrows = tile_nrows;
  p.n_blocks = n_blocks; p.bs = bs; p.nh = nh; p.nkv = nkv; p.scale_log2e = scale * 1.4426950408889634f;
  p.window = window; p.err = err;
  p.heads_per_cta = ((nh / nkv) % NQ == 0) ? NQ : 1;
  p.n_tiles = n_tiles;
  // Two tiles per CTA, a heavy and a light one, where that makes one round of CTAs out of more than one
  // (CUCA_ATTN_PAIR_TILES=0 never, =2 whenever there are two tiles).
  if (pair_mode < 0) { const char* e = getenv("CUCA_ATTN_PAIR_TILES"); pair_mode = e ? atoi(e) : 1; }
  const int head_ctas = nh / p.heads_per_cta, sms = cuca_device_sms();
  p.pair_tiles = n_tiles >= 2 && (pair_mode == 2 || (pair_mode == 1 && n_tiles * head_ctas > sms &&
                                                     ((n_tiles + 1) / 2) * head_ctas <= sms)) ? 1 : 0;
  return d == 128 ? launch_attn_tc<128>(tmQ, tmK, tmV, p, n_tiles, stream) : launch_attn_tc<64>(tmQ, tmK, tmV, p, n_tiles, stream);
}
