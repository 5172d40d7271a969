// Paged causal grouped-query attention for bfloat16 on tensor cores (mma.sync m16n8k16, 32-bit
// accumulate and softmax), in two forms that share one core:
//
//  * prefill: a CTA takes up to 64 consecutive rows of one request and one query head; its four
//    warps own 16 rows each and walk the request's keys in tiles of 64 absolute positions, from the
//    first key any row may see to the last row's own position;
//  * decode: a CTA takes one row, one key/value head and one chunk of key positions; the 16 MMA rows
//    are the (up to 16) query heads that share the key head, so keys and values are read once per
//    group; the four warps split each tile's keys and merge at the end; chunks of a row are merged
//    in chunk order by the last CTA to arrive (the result does not depend on arrival order).
//
// Key/value tiles come straight from the pages through the request's block table. Two ways in:
//  * 16-byte cp.async copies by all threads into a ring of three tiles whose rows are padded by 16 bytes, so
//    ldmatrix is free of bank conflicts (prefill; decode with head sizes or page sizes the other way refuses);
//  * decode with head sizes 64 and 128 and pages of at least 16 positions: every warp owns the 16-key groups
//    (tile, 16 warp .. 16 warp + 15), each inside one page, and brings them in with TMA (cp.async.bulk.tensor,
//    128-byte swizzle, one thread, mbarrier hand-over) through a ring of its own, so the loop has no block-wide
//    barrier and no per-thread address arithmetic (batch 64: 69 -> 55 us per layer at Llama-3.1-8B sizes).
// Positions outside a row's range (causal, window) are masked after scaling.
#include "tcgen05.cuh"
#include <math.h>
#include <stdlib.h>
#include <string.h>

namespace {

constexpr int TILE = 64;      // keys per shared-memory tile
constexpr int STAGES = 3;     // tiles in the shared-memory ring: two in flight while one is computed
constexpr int NTHREADS = 128;

struct AttnParams {
  const __nv_bfloat16* q;
  int q_stride;
  __nv_bfloat16* out;
  int out_stride;
  const __nv_bfloat16* kpool;
  const __nv_bfloat16* vpool;
  int n_blocks, bs;
  const int* tables;
  int table_stride;
  const int* positions;
  const int* seq_of_row;
  const int* rows;       // decode: row numbers (null: 0..n-1)
  const int* tile_row0;  // prefill: first row of each tile
  const int* tile_nrows; // prefill: rows in each tile (1..64)
  int nh, nkv;
  float scale_log2e;
  int window;
  int chunk;             // decode: key positions per split (multiple of 64); 0: each row divides its own length
  int slots;             // decode, chunk 0: CTAs the GPU holds at once (for the choice of chunks per row)
  float* part;           // decode: [rows][nh][splits][D + 2] partial (acc, m, l)
  int* counters;         // decode: [rows][nkv], zero before and after
  int cluster;           // decode: 1: the chunk CTAs of a (row, key head) pair are one thread-block cluster and merge
                         // their partial results through distributed shared memory (no scratch, no counters)
  int* err;
  // decode with the projection's K slices as input: the kernel adds them, rotates q and k and stores k and v itself
  const float* partial;  // [slices][rows][(nh + 2 nkv) D] 32-bit; row layout q heads, k heads, v heads
  int n_slices;
  size_t slice_stride;   // floats between slices
  const __nv_bfloat16* bias;  // [(nh + 2 nkv) D] or null
  const float* cos_t;    // [table_rows][rot / 2]
  const float* sin_t;
  int table_rows, rot;
  int has_kv;            // 0: the layer reads another layer's pages and has only q
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Thread-block clusters: a barrier over every thread of every CTA of the cluster (release / acquire), the address
// of a shared-memory location in another CTA of the cluster, and a load from there.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float dsmem_ld(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
struct Smem {
  static constexpr int RS = D + 8;  // row stride in elements: 16 bytes of padding
  static constexpr int TILE_ELEMS = TILE * RS;
  static constexpr int BYTES = STAGES * 2 /*k, v*/ * TILE_ELEMS * 2;
  // fused form: the 16 query rows, then the new key and the new value of the row
  static constexpr int Q_ELEMS = 16 * RS;
  static constexpr int FUSED_BYTES = BYTES + (Q_ELEMS + 2 * D) * 2;
  // decode with TMA: every warp has a ring of its own; a stage holds the warp's 16 keys and values as
  // 64-wide halves of 16 rows x 128 bytes, 128-byte swizzled: K half 0, K half 1, ..., V half 0, ...
  static constexpr int HALVES = D / 64;
  static constexpr int SUB_BYTES = 16 * 128;
  static constexpr int WSTAGE_BYTES = 2 * (HALVES > 0 ? HALVES : 1) * SUB_BYTES;
  static constexpr int WSTAGES = 3;
  static constexpr int RING_BYTES = 4 * WSTAGES * WSTAGE_BYTES;
  static constexpr int TMA_BYTES = RING_BYTES + 1024 /*alignment*/ + (Q_ELEMS + 2 * D) * 2;
};

// One warp's state over its 16 MMA rows: thread (g, t) holds rows g and g + 8.
template <int D>
struct WarpState {
  float acc[D / 8][4];
  float m[2], l[2];
};

template <int D, bool DECODE, bool FUSED, bool TMA>
__global__ void __launch_bounds__(NTHREADS)
attn_mma_kernel(const AttnParams p, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
  static_assert(!FUSED || DECODE, "only the decode form takes the projection's K slices");
  static_assert(!TMA || (DECODE && D % 64 == 0), "the TMA form is for decode with head sizes 64 and 128");
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  using S = Smem<D>;
  uint8_t* ring_base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int G = p.nh / p.nkv;
  pdl_trigger();
  // The fused, TMA-fed decode form reads nothing the kernel before it (the q/k/v projection) writes until it adds
  // that projection's slices: the rows' positions and slots were copied before the step's first kernel ran, the
  // page tables were brought up to date before that, and every key it copies was written by an earlier step
  // (the row's own key comes from registers). So its lookups and its first copies go out before the dependency
  // wait and overlap the projection's tail. Every other form waits here.
  constexpr bool EARLY = FUSED && TMA;
  if (!EARLY) pdl_wait();

  // ---------------------------------------------------------------- what this CTA and warp own
  int seq, kvh, range_lo, range_hi;   // keys [range_lo, range_hi) of request `seq`
  int row_token[2], row_head[2], row_pos[2];  // per owned MMA row (g, g + 8): token row, query head, position
  bool row_ok[2];
  int dec_row = 0, P = 0, warp_pmax = 0;
  int n_used = gridDim.x;  // decode: chunks this row really uses
  if (DECODE) {
    dec_row = p.rows ? p.rows[blockIdx.z] : blockIdx.z;
    seq = p.seq_of_row[dec_row];
    if (seq < 0) return;
    P = p.positions[dec_row];
    kvh = blockIdx.y;
    int lo = (p.window > 0 && P - (p.window - 1) > 0) ? P - (p.window - 1) : 0;
    // chunk 0: every row picks how many of the gridDim.x chunks it uses from its own length, so that the tiles
    // of 64 keys on the critical path (rounds of CTAs the GPU needs, times tiles per chunk) are fewest, and
    // spreads its keys evenly over them; the other chunks of the row are empty
    int chunk = p.chunk;
    if (chunk == 0) {
      const int tiles = (P + TILE) / TILE;
      const int pairs = (int)(gridDim.y * gridDim.z);
      const int nmax = min((int)gridDim.x, tiles);
      int best = 1, best_cost = 0x7fffffff;
      for (int n = 1; n <= nmax; ++n) {
        int rounds = (pairs * n + p.slots - 1) / p.slots;
        // a CTA costs about three tiles' time before and after its own tiles; the merge a little more
        int cost = rounds * ((tiles + n - 1) / n + 3) * 8 + (n > 1 ? 2 : 0);
        if (cost < best_cost) { best_cost = cost; best = n; }
      }
      n_used = best;
      chunk = ((tiles + best - 1) / best) * TILE;
    }
    if ((int)blockIdx.x >= n_used) {
      // a chunk this row does not use: in a cluster it still meets the others at their two barriers (it has
      // nothing to hand over and nobody reads its shared memory)
      if (p.cluster && n_used > 1) {
        cluster_sync_all();
        cluster_sync_all();
      }
      return;
    }
    range_lo = max(lo, (int)blockIdx.x * chunk);
    range_hi = min(P + 1, ((int)blockIdx.x + 1) * chunk);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int item = g + 8 * h;
      row_ok[h] = item < G;
      row_token[h] = dec_row;
      row_head[h] = kvh * G + item;
      row_pos[h] = P;
    }
  } else {
    const int tile = blockIdx.x;
    const int row0 = p.tile_row0[tile], n = p.tile_nrows[tile];
    seq = p.seq_of_row[row0];
    if (seq < 0) return;
    const int pos0 = p.positions[row0];
    const int head = blockIdx.y;
    kvh = head / G;
    range_lo = (p.window > 0 && pos0 - (p.window - 1) > 0) ? pos0 - (p.window - 1) : 0;
    range_hi = pos0 + n;
    warp_pmax = pos0 + warp * 16 + 15;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int i = warp * 16 + g + 8 * h;
      row_ok[h] = i < n;
      row_token[h] = row0 + i;
      row_head[h] = head;
      row_pos[h] = pos0 + i;
    }
  }
  const int* table = p.tables + (size_t)seq * p.table_stride;

  // ---------------------------------------------------------------- query fragments (A operand), from global
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t lo = 0, hi = 0;
      if (!FUSED && row_ok[h]) {
        const __nv_bfloat16* qp = p.q + (size_t)row_token[h] * p.q_stride + (size_t)row_head[h] * D + ks * 16 + 2 * t;
        lo = *reinterpret_cast<const uint32_t*>(qp);
        hi = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
      qf[ks][h] = lo;       // a0 (row g) / a1 (row g + 8): k = 2t, 2t + 1
      qf[ks][2 + h] = hi;   // a2 / a3: k = 2t + 8, 2t + 9
    }
  }

  WarpState<D> st;
#pragma unroll
  for (int j = 0; j < D / 8; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) st.acc[j][c] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;

  // ---------------------------------------------------------------- tile loop
  const int first_tile = range_lo < range_hi ? (range_lo / TILE) : 0;
  const int n_tiles = range_lo < range_hi ? ((range_hi - 1) / TILE - first_tile + 1) : 0;

  // Row offsets of a tile's 64 keys in the pools (-1: masked or without a page), one tile ahead of the copies:
  // the page-table lookups of tile i + 2 are in flight while tile i is computed, so no copy waits on one.
  __shared__ long long s_rowoff[STAGES][TILE];
  const int bs_shift = __ffs(p.bs) - 1, bs_mask = p.bs - 1;
  // fused form: the CTA whose keys include the row's own position makes that key and value itself
  const bool owner = FUSED && p.has_kv && P >= range_lo && P < range_hi;
  auto row_offset = [&](int tile_index) -> long long {
    int kp = (first_tile + tile_index) * TILE + (int)threadIdx.x;
    if (kp < range_lo || kp >= range_hi) return -1;
    if (owner && kp == P) return -1;  // comes from registers, not from the page
    int blk = table[kp >> bs_shift];
    if (blk < 0 || blk >= p.n_blocks) {
      if (p.err) atomicExch(p.err, CUCA_ERR_BLOCK_RANGE);
      return -1;
    }
    return ((((long long)blk * p.nkv + kvh) << bs_shift) + (kp & bs_mask)) * D;
  };
  auto load_tile = [&](int stage, int tile_index) {
    __nv_bfloat16* ks = smem + (size_t)stage * 2 * S::TILE_ELEMS;
    __nv_bfloat16* vs = ks + S::TILE_ELEMS;
    const long long* ro = s_rowoff[tile_index % STAGES];
    constexpr int CH = D / 8;  // 16-byte chunks per row
#pragma unroll
    for (int idx = threadIdx.x; idx < TILE * CH; idx += NTHREADS) {
      int key = idx / CH, ch = idx % CH;
      long long off = ro[key];
      bool valid = off >= 0;
      size_t o = valid ? (size_t)off + ch * 8 : 0;
      cp_async16(smem_u32(ks + key * S::RS + ch * 8), p.kpool + o, valid);
      cp_async16(smem_u32(vs + key * S::RS + ch * 8), p.vpool + o, valid);
    }
  };
  // ---- TMA form: this warp's 16-key groups are (tile ti, keys 16 warp .. 16 warp + 15) for ti in [ti_lo, ti_hi)
  __shared__ __align__(8) uint64_t w_full[4][S::WSTAGES];
  __shared__ int w_abort;
  int ti_lo = 0, n_mine = 0, next_page = -1;
  uint8_t* ring = ring_base + (size_t)warp * S::WSTAGES * S::WSTAGE_BYTES;
  auto group_kp0 = [&](int j) { return (first_tile + ti_lo + j) * TILE + warp * 16; };
  auto page_of = [&](int j) { return table[group_kp0(j) >> bs_shift]; };
  auto issue_group = [&](int j, int page) {  // the whole warp: one copy per lane (keys and values, 64-wide halves)
    const int kp0 = group_kp0(j);
    if (page < 0 || page >= p.n_blocks) {
      if (lane == 0 && p.err) atomicExch(p.err, CUCA_ERR_BLOCK_RANGE);
      page = 0;  // any readable page: these keys are masked or the step is lost anyway
    }
    const int row = ((page * p.nkv + kvh) << bs_shift) + (kp0 & bs_mask);
    const int st = j % S::WSTAGES;
    uint8_t* dst = ring + (size_t)st * S::WSTAGE_BYTES;
    if (lane == 0) mbar_expect_tx(&w_full[warp][st], S::WSTAGE_BYTES);
    __syncwarp();
    if (lane < 2 * S::HALVES) {
      const int h = lane % S::HALVES;
      const bool values = lane >= S::HALVES;
      tma_load_2d(dst + lane * S::SUB_BYTES, values ? &tmV : &tmK, &w_full[warp][st], 64 * h, row);
    }
  };
  // ---- fused form, whole heads rotated, 16-byte rows: a thread's work is four consecutive columns of each half of
  // a head (or of v) over all slices. The loads of its first item (up to four slices, cosines and sines) are asked
  // for here, before the ring is set up, so that the page-table lookups below and these round trips overlap; they
  // are used further down. (One value at a time, as the general form below does it, the prologue took 6 us of the
  // kernel's 20 at batch 8.)
  const int f_half = FUSED ? p.rot / 2 : 0;
  const size_t f_width = FUSED ? (size_t)(p.nh + (p.has_kv ? 2 * p.nkv : 0)) * D : 0;
  const float* f_row = FUSED ? p.partial + (size_t)dec_row * f_width : nullptr;
  const bool f_in_table = FUSED && P >= 0 && P < p.table_rows;
  const bool f_vec = FUSED && p.rot == D && D % 8 == 0 && ((p.slice_stride | f_width) & 3) == 0 &&
                     (((uintptr_t)p.partial | (uintptr_t)p.cos_t | (uintptr_t)p.sin_t) & 15) == 0;
  const int f_hq = f_half / 4;                                   // items per rotated head
  const int f_rope_items = (G + (owner ? 1 : 0)) * f_hq;
  const int f_items = f_rope_items + (owner ? D / 4 : 0);       // then the row's own value
  // columns of item `it`: ca (and ca + half for a rotated head); head index hh (G: the key), offset inside the head
  auto f_item = [&](int it, int& ca, int& hh, int& off) {
    if (it < f_rope_items) {
      hh = it / f_hq;
      off = (it - hh * f_hq) * 4;
      ca = (hh < G ? (kvh * G + hh) * D : (p.nh + kvh) * D) + off;
    } else {
      hh = -1;
      off = (it - f_rope_items) * 4;
      ca = (p.nh + p.nkv + kvh) * D + off;
    }
  };
  float4 pre_a[4], pre_b[4], pre_c = make_float4(1.f, 1.f, 1.f, 1.f), pre_s = make_float4(0.f, 0.f, 0.f, 0.f);
  auto preload = [&]() {
  if (FUSED && f_vec && (int)threadIdx.x < f_items) {
    int ca, hh, off;
    f_item(threadIdx.x, ca, hh, off);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      pre_a[u] = pre_b[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (u < p.n_slices) {
        pre_a[u] = __ldcg(reinterpret_cast<const float4*>(f_row + (size_t)u * p.slice_stride + ca));
        if (hh >= 0) pre_b[u] = __ldcg(reinterpret_cast<const float4*>(f_row + (size_t)u * p.slice_stride + ca + f_half));
      }
    }
    if (hh >= 0 && f_in_table) {
      pre_c = *reinterpret_cast<const float4*>(p.cos_t + (size_t)P * f_half + off);
      pre_s = *reinterpret_cast<const float4*>(p.sin_t + (size_t)P * f_half + off);
    }
  }
  };
  if (!EARLY) preload();

  if (TMA) {
    if (threadIdx.x == 0) w_abort = 0;
    if (lane == 0) {
#pragma unroll
      for (int st = 0; st < S::WSTAGES; ++st) mbar_init(&w_full[warp][st], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // groups with a key in range: a run of consecutive tiles
    int lo = n_tiles, hi = 0;
    for (int ti = 0; ti < n_tiles; ++ti) {
      const int kp0 = (first_tile + ti) * TILE + warp * 16;
      if (kp0 < range_hi && kp0 + 16 > range_lo) { lo = min(lo, ti); hi = ti + 1; }
    }
    ti_lo = lo;
    n_mine = hi > lo ? hi - lo : 0;
    __syncthreads();  // barriers and the abort flag are set up
    {
      int pg[S::WSTAGES];
#pragma unroll
      for (int j = 0; j < S::WSTAGES; ++j) {
        pg[j] = (lane == 0 && j < n_mine) ? page_of(j) : -1;
        pg[j] = __shfl_sync(0xffffffffu, pg[j], 0);
      }
#pragma unroll
      for (int j = 0; j < S::WSTAGES - 1; ++j)
        if (j < n_mine) issue_group(j, pg[j]);
      next_page = pg[S::WSTAGES - 1];
    }
  } else {
    if (threadIdx.x < TILE) {
#pragma unroll
      for (int i = 0; i < STAGES; ++i)
        if (i < n_tiles) s_rowoff[i][threadIdx.x] = row_offset(i);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
      if (i < n_tiles) load_tile(i, i);
      cp_async_commit();
    }
  }

  if (EARLY) {
    pdl_wait();  // from here on the projection's slices are read
    preload();
  }
  // ---------------------------------------------------------------- fused form: q (and k, v) from the K slices
  __nv_bfloat16* q_s = TMA ? reinterpret_cast<__nv_bfloat16*>(ring_base + S::RING_BYTES)
                           : smem + (size_t)STAGES * 2 * S::TILE_ELEMS;  // [16][RS]: the group's rotated query heads
  __nv_bfloat16* k_new = q_s + S::Q_ELEMS;                          // [D] rotated key of the row's own position
  __nv_bfloat16* v_new = k_new + D;                                 // [D] its value
  if (FUSED) {
    const size_t width = (size_t)(p.nh + (p.has_kv ? 2 * p.nkv : 0)) * D;
    const float* prow = p.partial + (size_t)dec_row * width;
    auto value = [&](int col) -> float {
      float v = p.bias ? __bfloat162float(p.bias[col]) : 0.f;
      for (int k0 = 0; k0 < p.n_slices; k0 += 4) {  // four slices' loads in flight at once, added in slice order
        float x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) x[u] = k0 + u < p.n_slices ? __ldcg(prow + (size_t)(k0 + u) * p.slice_stride + col) : 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) v += x[u];
      }
      return v;
    };
    const int half = p.rot / 2;
    const bool in_table = P >= 0 && P < p.table_rows;
    if (!in_table && half > 0 && threadIdx.x == 0 && p.err) atomicExch(p.err, CUCA_ERR_TOKEN_RANGE);
    if (f_vec) {
      auto add4 = [](float4& x, const float4 y) { x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w; };
      auto put4 = [](__nv_bfloat16* dst, float a, float b, float c, float d) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(a, b), pack_bf16(c, d));
      };
      for (int it = threadIdx.x; it < f_items; it += NTHREADS) {
        int ca, hh, off;
        f_item(it, ca, hh, off);
        const bool first = it == (int)threadIdx.x;
        auto bias4 = [&](int col) {
          return p.bias ? make_float4(__bfloat162float(p.bias[col]), __bfloat162float(p.bias[col + 1]),
                                      __bfloat162float(p.bias[col + 2]), __bfloat162float(p.bias[col + 3]))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
        };
        float4 a = bias4(ca), b = hh >= 0 ? bias4(ca + f_half) : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k0 = 0; k0 < p.n_slices; k0 += 4) {  // four slices' loads in flight at once, added in slice order
          float4 xa[4], xb[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            xa[u] = xb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (first && k0 == 0) {
              xa[u] = pre_a[u];
              xb[u] = pre_b[u];
            } else if (k0 + u < p.n_slices) {
              xa[u] = __ldcg(reinterpret_cast<const float4*>(f_row + (size_t)(k0 + u) * p.slice_stride + ca));
              if (hh >= 0) xb[u] = __ldcg(reinterpret_cast<const float4*>(f_row + (size_t)(k0 + u) * p.slice_stride + ca + f_half));
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) { add4(a, xa[u]); add4(b, xb[u]); }
        }
        if (hh < 0) {
          put4(v_new + off, a.x, a.y, a.z, a.w);
          continue;
        }
        float4 c = pre_c, sn = pre_s;
        if (!first) {
          c = in_table ? *reinterpret_cast<const float4*>(p.cos_t + (size_t)P * half + off) : make_float4(1.f, 1.f, 1.f, 1.f);
          sn = in_table ? *reinterpret_cast<const float4*>(p.sin_t + (size_t)P * half + off) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        __nv_bfloat16* dst = (hh < G ? q_s + hh * S::RS : k_new) + off;
        put4(dst, a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y, a.z * c.z - b.z * sn.z, a.w * c.w - b.w * sn.w);
        put4(dst + half, a.x * sn.x + b.x * c.x, a.y * sn.y + b.y * c.y, a.z * sn.z + b.z * c.z, a.w * sn.w + b.w * c.w);
      }
    }
    // per head: `half` rotated pairs (i, i + half), then the values beyond the rotary part as they are
    const int units = D - half;
    const int heads_here = f_vec ? 0 : G + (owner ? 1 : 0);
    for (int idx = threadIdx.x; idx < heads_here * units; idx += NTHREADS) {
      const int hh = idx / units, u = idx % units;
      const int col0 = hh < G ? (kvh * G + hh) * D : (p.nh + kvh) * D;
      __nv_bfloat16* dst = hh < G ? q_s + hh * S::RS : k_new;
      if (u < half) {
        const float c = in_table ? p.cos_t[(size_t)P * half + u] : 1.f;
        const float sn = in_table ? p.sin_t[(size_t)P * half + u] : 0.f;
        const float a = value(col0 + u), b = value(col0 + u + half);
        dst[u] = __float2bfloat16_rn(a * c - b * sn);
        dst[u + half] = __float2bfloat16_rn(a * sn + b * c);
      } else {
        dst[u + half] = __float2bfloat16_rn(value(col0 + u + half));
      }
    }
    if (owner && !f_vec)
      for (int i = threadIdx.x; i < D; i += NTHREADS)
        v_new[i] = __float2bfloat16_rn(value((p.nh + p.nkv + kvh) * D + i));
    for (int idx = threadIdx.x; idx < (16 - G) * D; idx += NTHREADS)
      q_s[(G + idx / D) * S::RS + idx % D] = __float2bfloat16_rn(0.f);
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_bfloat16* qp = q_s + (g + 8 * h) * S::RS + ks * 16 + 2 * t;
        qf[ks][h] = *reinterpret_cast<const uint32_t*>(qp);
        qf[ks][2 + h] = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
    if (owner) {
      // the page keeps the new key and value for the steps to come
      const int blk = table[P >> bs_shift];
      if (blk < 0 || blk >= p.n_blocks) {
        if (threadIdx.x == 0 && p.err) atomicExch(p.err, CUCA_ERR_BLOCK_RANGE);
      } else {
        const size_t off = ((((size_t)blk * p.nkv + kvh) << bs_shift) + (P & bs_mask)) * D;
        for (int i = threadIdx.x; i < 2 * (D / 8); i += NTHREADS) {
          const int which = i / (D / 8), ch = i % (D / 8);
          __nv_bfloat16* pool = const_cast<__nv_bfloat16*>(which ? p.vpool : p.kpool);
          *reinterpret_cast<uint4*>(pool + off + ch * 8) = *reinterpret_cast<const uint4*>((which ? v_new : k_new) + ch * 8);
        }
      }
    }
  }

  // decode: a warp owns 16 keys of each tile and updates its softmax per 16 keys; prefill: every warp takes all
  // 64 keys of the tile in one softmax update
  constexpr int SUBS = DECODE ? 1 : TILE / 16;   // 16-key groups per update
  constexpr int NT = 2 * SUBS;                    // 8-key n-tiles per update
  // One update with the keys [kp0, kp0 + 16 SUBS): kaddr / vaddr give the shared-memory address of (key, dim),
  // `key` counted from key0 within what they address.
  auto update = [&](auto kaddr, auto vaddr, const int kp0, const int key0) {
    // ---- S = Q K^T
    float s[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[nt][c] = 0.f;
    // K steps outermost: consecutive MMAs go to different accumulators, so none waits for the one before it
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int sub = 0; sub < SUBS; ++sub) {
        uint32_t b[4];
        int mat = lane >> 3, r = lane & 7;
        int key = (key0 / 16 + sub) * 16 + (mat >> 1) * 8 + r;
        int dim = kk * 16 + (mat & 1) * 8;
        ldsm_x4(b, kaddr(key, dim));
        mma_bf16(s[2 * sub], qf[kk], b[0], b[1]);
        mma_bf16(s[2 * sub + 1], qf[kk], b[2], b[3]);
      }
    }
    // ---- scale, mask, online softmax (per row: g and g + 8). Tiles that every row of the warp sees whole
    // (the bulk of a long prompt) skip the per-key tests.
    bool whole = !DECODE && kp0 >= range_lo && kp0 + 16 * SUBS <= range_hi && kp0 + 16 * SUBS - 1 <= warp_pmax - 15 &&
                 (p.window <= 0 || kp0 >= warp_pmax - (p.window - 1));
    uint32_t pa[SUBS][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float mx = -INFINITY;
      if (whole) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float v = s[nt][2 * h + e] * p.scale_log2e;
            s[nt][2 * h + e] = v;
            mx = fmaxf(mx, v);
          }
      } else {
        int lo_row = (p.window > 0 && row_pos[h] - (p.window - 1) > 0) ? row_pos[h] - (p.window - 1) : 0;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            int kp = kp0 + nt * 8 + 2 * t + e;
            bool ok = row_ok[h] && kp <= row_pos[h] && kp >= lo_row && kp >= range_lo && kp < range_hi;
            float v = ok ? s[nt][2 * h + e] * p.scale_log2e : -INFINITY;
            s[nt][2 * h + e] = v;
            mx = fmaxf(mx, v);
          }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      float m_new = fmaxf(st.m[h], mx);
      float corr = (m_new == -INFINITY) ? 1.f : exp2f(st.m[h] - m_new);
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float v0 = s[nt][2 * h], v1 = s[nt][2 * h + 1];
        float p0 = (v0 == -INFINITY) ? 0.f : exp2f(v0 - m_new);
        float p1 = (v1 == -INFINITY) ? 0.f : exp2f(v1 - m_new);
        sum += p0 + p1;
        // the accumulator layout of S is the A-operand layout of P: n-tile 2 sub is k 0..7, 2 sub + 1 is k 8..15
        pa[nt >> 1][(nt & 1) * 2 + h] = pack_bf16(p0, p1);
      }
      st.l[h] = st.l[h] * corr + sum;
      st.m[h] = m_new;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        st.acc[j][2 * h] *= corr;
        st.acc[j][2 * h + 1] *= corr;
      }
    }
    // ---- O += P V: P is the A operand (16 rows x 16 keys per step), V tiles are read transposed
#pragma unroll
    for (int sub = 0; sub < SUBS; ++sub) {
#pragma unroll
      for (int j = 0; j < D / 8; j += 2) {
        uint32_t b[4];
        int mat = lane >> 3, r = lane & 7;
        int key = (key0 / 16 + sub) * 16 + (mat & 1) * 8 + r;
        int dim = j * 8 + (mat >> 1) * 8;
        ldsm_x4_trans(b, vaddr(key, dim));
        mma_bf16(st.acc[j], pa[sub], b[0], b[1]);
        mma_bf16(st.acc[j + 1], pa[sub], b[2], b[3]);
      }
    }
  };

  if (TMA) {
    // every warp walks its own groups through its own ring: no block-wide barrier in the loop
    bool ok = true;
    for (int i = 0; i < n_mine && ok; ++i) {
      {
        // group i + WSTAGES - 1 goes into the stage that group i - 1 left; the page of the one after is looked up now
        // (by lane 0, which hands it to the warp one round later)
        const int j = i + S::WSTAGES - 1;
        const int page_j = __shfl_sync(0xffffffffu, next_page, 0);
        if (lane == 0 && j + 1 < n_mine) next_page = page_of(j + 1);
        if (j < n_mine) issue_group(j, page_j);
      }
      const int st_i = i % S::WSTAGES;
      ok = mbar_wait(&w_full[warp][st_i], (i / S::WSTAGES) & 1, p.err, &w_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t kbase = smem_u32(ring + (size_t)st_i * S::WSTAGE_BYTES);
      const uint32_t vbase = kbase + S::HALVES * S::SUB_BYTES;
      // (key, dim) in a swizzled half: row `key` of 128 bytes, 16-byte chunk (dim % 64) / 8 XOR (key % 8)
      auto sw = [](uint32_t base, int key, int dim) {
        return base + (uint32_t)((dim >> 6) * S::SUB_BYTES + key * 128 + ((((dim & 63) >> 3) ^ (key & 7)) << 4));
      };
      const int kp0 = group_kp0(i);
      if (owner && P >= kp0 && P < kp0 + 16) {
        // the row's own key and value take their place among the warp's keys (the page's row is stale)
        const int key = P - kp0;
        for (int c = lane; c < 2 * (D / 8); c += 32) {
          const int which = c / (D / 8), ch = c % (D / 8);
          const uint4 val = *reinterpret_cast<const uint4*>((which ? v_new : k_new) + ch * 8);
          const uint32_t dst = sw(which ? vbase : kbase, key, ch * 8);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w) : "memory");
        }
        __syncwarp();
      }
      update([&](int key, int dim) { return sw(kbase, key, dim); }, [&](int key, int dim) { return sw(vbase, key, dim); },
             kp0, 0);
      __syncwarp();  // every lane has read the stage before lane 0 asks for the next group into it
    }
    if (w_abort) {
      // copies in flight land before the shared memory is used again
      unsigned long long t0 = global_ns();
      while (global_ns() - t0 < 2000000ull) { }
    }
  } else {
    for (int ti = 0; ti < n_tiles; ++ti) {
      const int stage = ti % STAGES;
      if (ti + STAGES - 1 < n_tiles) load_tile((ti + STAGES - 1) % STAGES, ti + STAGES - 1);
      cp_async_commit();
      cp_async_wait<STAGES - 1>();
      __syncthreads();
      long long next_off = -1;
      const bool look_ahead = threadIdx.x < TILE && ti + STAGES < n_tiles;
      if (look_ahead) next_off = row_offset(ti + STAGES);
      const int start = (first_tile + ti) * TILE;
      const __nv_bfloat16* ks = smem + (size_t)stage * 2 * S::TILE_ELEMS;
      const __nv_bfloat16* vs = ks + S::TILE_ELEMS;
      if (owner && P >= start && P < start + TILE) {
        // the row's own key and value take their place in the tile (the copy left zeros there)
        const int key = P - start;
        for (int i = threadIdx.x; i < 2 * (D / 8); i += NTHREADS) {
          const int which = i / (D / 8), ch = i % (D / 8);
          __nv_bfloat16* dst = const_cast<__nv_bfloat16*>(which ? vs : ks) + key * S::RS + ch * 8;
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>((which ? v_new : k_new) + ch * 8);
        }
        __syncthreads();
      }
      const int sub0 = DECODE ? warp : 0;
      const int kp0 = start + sub0 * 16;              // first key of this update
      bool active = kp0 < range_hi && kp0 + 16 * SUBS > range_lo;
      if (!DECODE && kp0 > warp_pmax) active = false;  // every row of this warp lies before these keys (causal)
      if (active)
        update([&](int key, int dim) { return smem_u32(ks + key * S::RS + dim); },
               [&](int key, int dim) { return smem_u32(vs + key * S::RS + dim); }, kp0, sub0 * 16);
      if (look_ahead) s_rowoff[ti % STAGES][threadIdx.x] = next_off;  // this slot was last read to request tile ti
      __syncthreads();  // the stage is overwritten by the load issued in the next iteration
    }
    cp_async_wait<0>();
  }
  // row sums live spread over the four threads of a quad
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
  }

  if (!DECODE) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (!row_ok[h]) continue;
      float inv = st.l[h] > 0.f ? 1.f / st.l[h] : 0.f;
      __nv_bfloat16* o = p.out + (size_t)row_token[h] * p.out_stride + (size_t)row_head[h] * D;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        uint32_t v = pack_bf16(st.acc[j][2 * h] * inv, st.acc[j][2 * h + 1] * inv);
        *reinterpret_cast<uint32_t*>(o + j * 8 + 2 * t) = v;
      }
    }
    return;
  }

  // ---------------------------------------------------------------- decode: merge the four warps, then the chunks
  __syncthreads();
  float* fs = reinterpret_cast<float*>(smem_raw);   // [4 warps][16 rows][D + 2]
  constexpr int FR = D + 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    int rowi = g + 8 * h;
    float* dst = fs + ((size_t)warp * 16 + rowi) * FR;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      dst[j * 8 + 2 * t] = st.acc[j][2 * h];
      dst[j * 8 + 2 * t + 1] = st.acc[j][2 * h + 1];
    }
    if (t == 0) {
      dst[D] = st.m[h];
      dst[D + 1] = st.l[h];
    }
  }
  __syncthreads();
  const int n_splits = gridDim.x;  // layout of the scratch; the row uses the first n_used of them
  const bool by_cluster = p.cluster && n_used > 1;
  // scratch and counters are indexed by the ordinal of the decode row in this launch
  float* part_row = by_cluster ? nullptr : p.part + ((size_t)blockIdx.z * p.nh + (size_t)kvh * G) * n_splits * FR;
  float* cpart = fs + (size_t)4 * 16 * FR;  // cluster form: this CTA's [G][D + 2] (acc, m, l), read by the cluster's first CTA
  for (int idx = threadIdx.x; idx < G * D; idx += NTHREADS) {
    int item = idx / D, dim = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, fs[((size_t)w * 16 + item) * FR + D]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* src = fs + ((size_t)w * 16 + item) * FR;
      float f = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - M);
      L += src[D + 1] * f;
      O += src[dim] * f;
    }
    if (n_used == 1) {
      p.out[(size_t)dec_row * p.out_stride + (size_t)(kvh * G + item) * D + dim] =
          __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    } else {
      float* dst = by_cluster ? cpart + (size_t)item * FR : part_row + ((size_t)item * n_splits + blockIdx.x) * FR;
      dst[dim] = O;
      if (dim == 0) { dst[D] = M; dst[D + 1] = L; }
    }
  }
  if (n_used == 1) return;
  constexpr int MAXS = 32;
  __shared__ float s_m[16][MAXS], s_f[16][MAXS], s_inv[16];
  if (by_cluster) {
    // Every chunk CTA of the row has its partial result in its own shared memory; after the cluster's barrier the
    // first CTA reads them from there and merges in chunk order, and a second barrier keeps the others' shared
    // memory alive until it has. No trip through global memory, no counter, no last arriver.
    cluster_sync_all();
    if (cluster_rank() == 0) {
      const uint32_t mine = smem_u32(cpart);
      for (int qd = threadIdx.x; qd < G * MAXS; qd += NTHREADS) {
        const int item = qd / MAXS, sidx = qd % MAXS;
        float ms = -INFINITY, ls = 0.f;
        if (sidx < n_used) {
          const uint32_t src = dsmem_addr(mine + (uint32_t)((item * FR + D) * sizeof(float)), (uint32_t)sidx);
          ms = dsmem_ld(src);
          ls = dsmem_ld(src + 4);
        }
        s_m[item][sidx] = ms;
        s_f[item][sidx] = ls;
      }
      __syncthreads();
      if (threadIdx.x < G) {
        const int item = threadIdx.x;
        float M = -INFINITY;
        for (int sidx = 0; sidx < n_used; ++sidx) M = fmaxf(M, s_m[item][sidx]);
        float L = 0.f;
        for (int sidx = 0; sidx < n_used; ++sidx) {
          const float f = (s_m[item][sidx] == -INFINITY) ? 0.f : exp2f(s_m[item][sidx] - M);
          L += s_f[item][sidx] * f;
          s_f[item][sidx] = f;
        }
        s_inv[item] = L > 0.f ? 1.f / L : 0.f;
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < G * D; idx += NTHREADS) {
        const int item = idx / D, dim = idx % D;
        const uint32_t at = mine + (uint32_t)((item * FR + dim) * sizeof(float));
        float v[8];
#pragma unroll
        for (int sidx = 0; sidx < 8; ++sidx) v[sidx] = sidx < n_used ? dsmem_ld(dsmem_addr(at, (uint32_t)sidx)) : 0.f;
        float O = 0.f;
#pragma unroll
        for (int sidx = 0; sidx < 8; ++sidx) O += v[sidx] * (sidx < n_used ? s_f[item][sidx] : 0.f);
        p.out[(size_t)dec_row * p.out_stride + (size_t)(kvh * G + item) * D + dim] = __float2bfloat16_rn(O * s_inv[item]);
      }
    }
    cluster_sync_all();
    return;
  }
  __threadfence();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) {
    int arrived = atomicAdd(&p.counters[blockIdx.z * p.nkv + kvh], 1);
    last = arrived == n_used - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // Merge the chunks in chunk order. All loads of a phase are independent and issued together, so the merge
  // costs a few memory round trips, not one per chunk.
  // Up to four output elements per thread and eight chunks (the common case): their partial sums are asked for
  // now, together with the maxima and sums below, so that the merge pays one trip to memory, not two.
  constexpr int PE = 4, PS = 8;
  const bool pre = G * D <= PE * NTHREADS && n_used <= PS;
  float v0[PE][PS];
#pragma unroll
  for (int e = 0; e < PE; ++e) {
    const int idx = threadIdx.x + e * NTHREADS;
    const float* src0 = part_row + (size_t)(idx / D) * n_splits * FR + idx % D;
#pragma unroll
    for (int sidx = 0; sidx < PS; ++sidx)
      v0[e][sidx] = (pre && idx < G * D && sidx < n_used) ? __ldcg(src0 + (size_t)sidx * FR) : 0.f;
  }
  for (int qd = threadIdx.x; qd < G * MAXS; qd += NTHREADS) {
    int item = qd / MAXS, sidx = qd % MAXS;
    float ms = -INFINITY, ls = 0.f;
    if (sidx < n_used) {
      const float* src = part_row + ((size_t)item * n_splits + sidx) * FR;
      ms = __ldcg(src + D);
      ls = __ldcg(src + D + 1);
    }
    s_m[item][sidx] = ms;
    s_f[item][sidx] = ls;
  }
  __syncthreads();
  if (threadIdx.x < G) {
    int item = threadIdx.x;
    float M = -INFINITY;
    for (int sidx = 0; sidx < n_used; ++sidx) M = fmaxf(M, s_m[item][sidx]);
    float L = 0.f;
    for (int sidx = 0; sidx < n_used; ++sidx) {  // chunk order: independent of which CTA came last
      float f = (s_m[item][sidx] == -INFINITY) ? 0.f : exp2f(s_m[item][sidx] - M);
      L += s_f[item][sidx] * f;
      s_f[item][sidx] = f;
    }
    s_inv[item] = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  if (pre) {
#pragma unroll
    for (int e = 0; e < PE; ++e) {
      const int idx = threadIdx.x + e * NTHREADS;
      if (idx >= G * D) break;
      const int item = idx / D, dim = idx % D;
      float O = 0.f;
#pragma unroll
      for (int sidx = 0; sidx < PS; ++sidx) O += v0[e][sidx] * s_f[item][sidx];  // chunks past n_used: 0 x 0
      p.out[(size_t)dec_row * p.out_stride + (size_t)(kvh * G + item) * D + dim] = __float2bfloat16_rn(O * s_inv[item]);
    }
  } else {
    for (int idx = threadIdx.x; idx < G * D; idx += NTHREADS) {
      int item = idx / D, dim = idx % D;
      const float* src0 = part_row + (size_t)item * n_splits * FR + dim;
      float v[MAXS];
#pragma unroll
      for (int sidx = 0; sidx < MAXS; ++sidx) v[sidx] = sidx < n_used ? __ldcg(src0 + (size_t)sidx * FR) : 0.f;
      float O = 0.f;
#pragma unroll
      for (int sidx = 0; sidx < MAXS; ++sidx) O += v[sidx] * s_f[item][sidx];
      p.out[(size_t)dec_row * p.out_stride + (size_t)(kvh * G + item) * D + dim] = __float2bfloat16_rn(O * s_inv[item]);
    }
  }
  if (threadIdx.x == 0) p.counters[blockIdx.z * p.nkv + kvh] = 0;
}

template <int D, bool DECODE, bool FUSED, bool TMA>
int launch(const AttnParams& p, const CUtensorMap& tmK, const CUtensorMap& tmV, dim3 grid, cudaStream_t stream) {
  int smem = TMA ? Smem<D>::TMA_BYTES : FUSED ? Smem<D>::FUSED_BYTES : Smem<D>::BYTES;
  if (DECODE) {
    int need = 5 * 16 * (D + 2) * (int)sizeof(float) + (TMA ? 1024 : 0);  // four warps' results, then the CTA's
    if (need > smem) smem = need;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<D, DECODE, FUSED, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      cuca_set_error("attention: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return 2;
    }
    configured = true;
  }
  if (DECODE && p.cluster)
    cuca_launch_cluster(attn_mma_kernel<D, DECODE, FUSED, TMA>, grid, dim3(NTHREADS), smem, stream, true, grid.x, p, tmK, tmV);
  else
    cuca_launch(attn_mma_kernel<D, DECODE, FUSED, TMA>, grid, dim3(NTHREADS), smem, stream, true, p, tmK, tmV);
  CUCA_CHECK_LAUNCH("attention_mma");
  return 0;
}

// tma: key/value groups by TMA (decode, head sizes 64 and 128, pages of at least 16 positions)
template <bool DECODE, bool FUSED = false>
int dispatch(int d, const AttnParams& p, dim3 grid, cudaStream_t stream, bool tma = false) {
  CUtensorMap tmK, tmV;
  memset(&tmK, 0, sizeof(tmK));
  memset(&tmV, 0, sizeof(tmV));
  if (DECODE && tma) {
    const uint64_t rows = (uint64_t)p.n_blocks * p.nkv * p.bs;
    if (!cuca_tensor_map_bf16(p.kpool, rows, d, d, 16, &tmK) || !cuca_tensor_map_bf16(p.vpool, rows, d, d, 16, &tmV))
      tma = false;
  }
  if constexpr (DECODE) {
    if (tma && d == 64) return launch<64, true, FUSED, true>(p, tmK, tmV, grid, stream);
    if (tma && d == 128) return launch<128, true, FUSED, true>(p, tmK, tmV, grid, stream);
  }
  switch (d) {
    case 16: return launch<16, DECODE, FUSED, false>(p, tmK, tmV, grid, stream);
    case 32: return launch<32, DECODE, FUSED, false>(p, tmK, tmV, grid, stream);
    case 48: return launch<48, DECODE, FUSED, false>(p, tmK, tmV, grid, stream);
    case 64: return launch<64, DECODE, FUSED, false>(p, tmK, tmV, grid, stream);
    case 80: return launch<80, DECODE, FUSED, false>(p, tmK, tmV, grid, stream);
    case 96: return launch<96, DECODE, FUSED, false>(p, tmK, tmV, grid, stream);
    case 112: return launch<112, DECODE, FUSED, false>(p, tmK, tmV, grid, stream);
    case 128: return launch<128, DECODE, FUSED, false>(p, tmK, tmV, grid, stream);
  }
  cuca_set_error("attention_mma: head size %d is not one of 16, 32, ..., 128", d);
  return 1;
}

}  // namespace

// 1 if the tensor-core attention kernels take this shape (bf16 only).
CUCA_API int cuca_attention_mma_supported(int nh, int nkv, int d, int q_stride, int out_stride) {
  if (d % 16 != 0 || d < 16 || d > 128) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 16) return 0;
  if (q_stride % 2 != 0 || out_stride % 2 != 0) return 0;
  return 1;
}

// Floats of scratch the decode form needs for `n_rows` rows split into `n_splits` chunks.
CUCA_API size_t cuca_attention_decode_scratch(int n_rows, int nh, int d, int n_splits) {
  return (size_t)n_rows * nh * n_splits * (d + 2);
}

namespace {
// What the fused form adds to the decode form's arguments.
struct FusedInput {
  const float* partial;
  int n_slices;
  size_t slice_stride;
  const void* bias;
  const float* cos_t;
  const float* sin_t;
  int table_rows, rot, has_kv;
};

int attention_decode_impl(const void* q, int q_stride, const FusedInput* fused, void* out, int out_stride,
                          const void* kpool, const void* vpool, int n_blocks, int bs, const int* positions,
                          const int* seq_of_row, const int* tables, int table_stride, const int* rows, int n_rows,
                          int nh, int nkv, int d, float scale, int window, int chunk, int n_splits, float* part,
                          int* counters, int* err, cudaStream_t stream) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int smem_cta = STAGES * 2 * TILE * (d + 8) * 2 + 2048;
  int per_sm = (227 * 1024) / smem_cta;
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 8) per_sm = 8;
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(cuca_attention_mma_supported(nh, nkv, d, q_stride, out_stride), "attention_decode: unsupported shape "
               "(heads %d/%d, head size %d)", nh, nkv, d);
  CUCA_REQUIRE(chunk >= 0 && chunk % TILE == 0 && n_splits >= 1 && n_splits <= 32, "attention_decode: bad chunking (at most 32 chunks)");
  CUCA_REQUIRE(bs > 0 && (bs & (bs - 1)) == 0, "attention_decode: %d positions per page is no power of two", bs);
  // Without scratch the chunk CTAs of a row form a thread-block cluster (up to eight, the portable size) and merge
  // through distributed shared memory.
  const bool by_cluster = n_splits > 1 && !(part && counters);
  CUCA_REQUIRE(!by_cluster || n_splits <= 8, "attention_decode: %d key chunks need scratch (a cluster merges up to 8)", n_splits);
  CUCA_REQUIRE(n_rows <= 65535, "attention_decode: too many rows");
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.kpool = (const __nv_bfloat16*)kpool; p.vpool = (const __nv_bfloat16*)vpool; p.n_blocks = n_blocks; p.bs = bs;
  p.tables = tables; p.table_stride = table_stride; p.positions = positions; p.seq_of_row = seq_of_row;
  p.rows = rows; p.tile_row0 = nullptr; p.tile_nrows = nullptr; p.nh = nh; p.nkv = nkv;
  p.scale_log2e = scale * 1.4426950408889634f; p.window = window; p.chunk = chunk; p.part = part;
  p.counters = counters; p.err = err; p.slots = sms * per_sm;
  p.cluster = by_cluster ? 1 : 0;
  p.partial = nullptr; p.n_slices = 0; p.slice_stride = 0; p.bias = nullptr; p.cos_t = p.sin_t = nullptr;
  p.table_rows = 0; p.rot = 0; p.has_kv = 0;
  static int env_tma = -1;
  if (env_tma < 0) { const char* e = getenv("CUCA_ATTN_TMA"); env_tma = e ? atoi(e) : 1; }
  // key/value groups of 16 positions by TMA: a group must lie in one page
  const bool tma = env_tma && d % 64 == 0 && bs >= 16 && ((uintptr_t)kpool & 15) == 0 && ((uintptr_t)vpool & 15) == 0;
  if (!fused) return dispatch<true, false>(d, p, dim3(n_splits, nkv, n_rows), stream, tma);
  CUCA_REQUIRE(fused->partial && fused->n_slices >= 1, "attention_decode_fused: no projection slices");
  CUCA_REQUIRE(fused->rot >= 0 && fused->rot <= d && fused->rot % 2 == 0,
               "attention_decode_fused: rotary size %d does not fit head size %d", fused->rot, d);
  CUCA_REQUIRE(fused->rot == 0 || (fused->cos_t && fused->sin_t), "attention_decode_fused: no rotation tables");
  CUCA_REQUIRE(d % 8 == 0 && ((uintptr_t)kpool & 15) == 0 && ((uintptr_t)vpool & 15) == 0,
               "attention_decode_fused: pages must be 16-byte aligned");
  p.partial = fused->partial; p.n_slices = fused->n_slices; p.slice_stride = fused->slice_stride;
  p.bias = (const __nv_bfloat16*)fused->bias; p.cos_t = fused->cos_t; p.sin_t = fused->sin_t;
  p.table_rows = fused->table_rows; p.rot = fused->rot; p.has_kv = fused->has_kv;
  return dispatch<true, true>(d, p, dim3(n_splits, nkv, n_rows), stream, tma);
}
}  // namespace

// Decode form: one query row per entry of `rows` (null: rows 0..n_rows-1), keys split in chunks of `chunk`
// positions (a multiple of 64), `n_splits` chunks cover every row's keys (n_splits * chunk > largest position).
// chunk = 0: each row divides its own keys evenly over the n_splits chunks, whatever its length.
CUCA_API int cuca_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* kpool,
                                   const void* vpool, int n_blocks, int bs, const int* positions,
                                   const int* seq_of_row, const int* tables, int table_stride, const int* rows,
                                   int n_rows, int nh, int nkv, int d, float scale, int window, int chunk,
                                   int n_splits, float* part, int* counters, int* err, cudaStream_t stream) {
  return attention_decode_impl(q, q_stride, nullptr, out, out_stride, kpool, vpool, n_blocks, bs, positions,
                               seq_of_row, tables, table_stride, rows, n_rows, nh, nkv, d, scale, window, chunk,
                               n_splits, part, counters, err, stream);
}

// The decode form fed by the unadded K slices of the stacked q/k/v projection, partial[slice][row][(nh + 2 nkv) d]
// (has_kv = 0: [nh d], a layer that reads another layer's pages): every CTA adds the slices of its group's query
// heads in slice order (plus bias) and rotates them (pairs (i, i + rot/2) by the tables' row of the position);
// the CTA whose keys include the row's own position does the same for that key, takes the value, stores both
// in the page and uses them from shared memory. One launch instead of rotate-and-store plus attention.
CUCA_API int cuca_attention_decode_fused(const float* partial, int n_slices, size_t slice_stride, const void* bias,
                                         const float* cos_t, const float* sin_t, int table_rows, int rot, int has_kv,
                                         void* out, int out_stride, void* kpool, void* vpool, int n_blocks, int bs,
                                         const int* positions, const int* seq_of_row, const int* tables,
                                         int table_stride, const int* rows, int n_rows, int nh, int nkv, int d,
                                         float scale, int window, int chunk, int n_splits, float* part, int* counters,
                                         int* err, cudaStream_t stream) {
  FusedInput f{partial, n_slices, slice_stride, bias, cos_t, sin_t, table_rows, rot, has_kv};
  return attention_decode_impl(nullptr, 2, &f, out, out_stride, kpool, vpool, n_blocks, bs, positions, seq_of_row,
                               tables, table_stride, rows, n_rows, nh, nkv, d, scale, window, chunk, n_splits, part,
                               counters, err, stream);
}

// Prefill form: tile i covers rows tile_row0[i] .. +tile_nrows[i]-1 (at most 64 consecutive rows of one request).
CUCA_API int cuca_attention_prefill(const void* q, int q_stride, void* out, int out_stride, const void* kpool,
                                    const void* vpool, int n_blocks, int bs, const int* positions,
                                    const int* seq_of_row, const int* tables, int table_stride,
                                    const int* tile_row0, const int* tile_nrows, int n_tiles, int nh, int nkv, int d,
                                    float scale, int window, int* err, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  CUCA_REQUIRE(cuca_attention_mma_supported(nh, nkv, d, q_stride, out_stride), "attention_prefill: unsupported "
               "shape (heads %d/%d, head size %d)", nh, nkv, d);
  CUCA_REQUIRE(nh <= 65535, "attention_prefill: too many heads");
  CUCA_REQUIRE(bs > 0 && (bs & (bs - 1)) == 0, "attention_prefill: %d positions per page is no power of two", bs);
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.kpool = (const __nv_bfloat16*)kpool; p.vpool = (const __nv_bfloat16*)vpool; p.n_blocks = n_blocks; p.bs = bs;
  p.tables = tables; p.table_stride = table_stride; p.positions = positions; p.seq_of_row = seq_of_row;
  p.rows = nullptr; p.tile_row0 = tile_row0; p.tile_nrows = tile_nrows; p.nh = nh; p.nkv = nkv;
  p.scale_log2e = scale * 1.4426950408889634f; p.window = window; p.chunk = 0; p.part = nullptr;
  p.counters = nullptr; p.err = err; p.slots = 1; p.cluster = 0;
  p.partial = nullptr; p.n_slices = 0; p.slice_stride = 0; p.bias = nullptr; p.cos_t = p.sin_t = nullptr;
  p.table_rows = 0; p.rot = 0; p.has_kv = 0;
  return dispatch<false, false>(d, p, dim3(n_tiles, nh), stream);
}

// ---------------------------------------------------------------------------------------------------------
// The allocation-free variant (see no_alloc.h): the same decode kernel, its scratch in the library's image.
// ---------------------------------------------------------------------------------------------------------
#include "no_alloc.h"
#include <mutex>

// Counters first (they are the part that must start at zero), partials behind them. In host code this name is
// only a handle for cudaGetSymbolAddress; it is not a device address and must never be handed to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CUCA_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
void* g_noalloc_addr[NOALLOC_MAX_DEVICES];
bool g_noalloc_ready[NOALLOC_MAX_DEVICES];
std::mutex g_noalloc_mu;

// Device address of the scratch array on the current device; looked up once per device.
int noalloc_scratch(void** addr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
    cuca_set_error("attention_decode_noalloc: no usable current device (%s)", cudaGetErrorString(e));
    return 2;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ready[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cuca_set_error("attention_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                     cudaGetErrorString(e));
      return 2;
    }
    g_noalloc_addr[dev] = p;
    g_noalloc_ready[dev] = true;
  }
  *addr = g_noalloc_addr[dev];
  return 0;
}
}  // namespace

CUCA_API int cuca_attention_decode_noalloc(const void* q, int q_stride, void* out, int out_stride, const void* kpool,
                                           const void* vpool, int n_blocks, int bs, const int* positions,
                                           const int* seq_of_row, const int* tables, int table_stride,
                                           const int* rows, int n_rows, int nh, int nkv, int d, float scale,
                                           int window, int chunk, int n_splits, int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(n_rows > 0 && nh > 0 && nkv > 0 && d > 0 && n_splits >= 1, "attention_decode_noalloc: bad sizes");
  const size_t part_floats = cuca_attention_decode_scratch(n_rows, nh, d, n_splits);
  const size_t counters = (size_t)n_rows * nkv;
  CUCA_REQUIRE(part_floats <= CUCA_NOALLOC_PART_FLOATS && counters <= CUCA_NOALLOC_COUNTERS,
               "attention_decode_noalloc: %d rows x %d heads x %d chunks x head size %d needs %zu scratch floats and "
               "%zu counters; the built-in scratch holds %u floats and %u counters. Use fewer chunks or rows, or "
               "cuca_attention_decode with a buffer of your own",
               n_rows, nh, n_splits, d, part_floats, counters, CUCA_NOALLOC_PART_FLOATS, CUCA_NOALLOC_COUNTERS);
  void* base = nullptr;
  int rc = noalloc_scratch(&base);
  if (rc) return rc;
  int* cnt = reinterpret_cast<int*>(base);
  float* part = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + CUCA_NOALLOC_COUNTERS * 4u);
  // the array keeps the last call's contents: the counters this call uses must start at zero
  cudaError_t e = cudaMemsetAsync(cnt, 0, counters * sizeof(int), stream);
  if (e != cudaSuccess) {
    cuca_set_error("attention_decode_noalloc: clearing the counters failed: %s", cudaGetErrorString(e));
    return 2;
  }
  return cuca_attention_decode(q, q_stride, out, out_stride, kpool, vpool, n_blocks, bs, positions, seq_of_row,
                               tables, table_stride, rows, n_rows, nh, nkv, d, scale, window, chunk, n_splits, part,
                               cnt, err, stream);
}
