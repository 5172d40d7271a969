// How a step's rows are handed to the attention kernels, made on the device from the per-request description of
// the step (first row, token count, cached positions): requests that bring one token become rows of the split-key
// decode form; longer portions are cut into tiles of consecutive rows for a prefill form, heaviest tile (latest
// positions, most keys) first so that the long tiles do not start last. The tile heights are the kernels' own
// (`cuca_attention_tile_rows`); nothing outside the attention part and this library knows them.
#include "common.cuh"

namespace {
constexpr int PLAN_THREADS = 1024;
constexpr int SORT_MAX = 2048;  // tiles ranked in shared memory; beyond that they keep the requests' order

__global__ void attention_plan_kernel(const int* __restrict__ req_row0, const int* __restrict__ req_count,
                                      const int* __restrict__ req_start, int n_req, int tile_rows,
                                      int* __restrict__ decode_rows, int n_decode, int* __restrict__ tile_row0,
                                      int* __restrict__ tile_nrows, int n_tiles) {
  pdl_trigger();
  pdl_wait();
  __shared__ int s_row0[SORT_MAX], s_n[SORT_MAX], s_pos[SORT_MAX];
  __shared__ int s_carry[2];
  const int tid = threadIdx.x;
  if (tid == 0) s_carry[0] = s_carry[1] = 0;
  __syncthreads();
  const bool sort = n_tiles <= SORT_MAX;
  // requests in blocks of PLAN_THREADS; within a block an exclusive scan of (single rows, tiles) by warp shuffles
  __shared__ int s_warp[2][32];
  for (int base = 0; base < n_req; base += PLAN_THREADS) {
    const int i = base + tid;
    const int cnt = i < n_req ? req_count[i] : 0;
    const int one = cnt == 1 ? 1 : 0;
    const int tiles = cnt > 1 ? (cnt + tile_rows - 1) / tile_rows : 0;
    int a = one, b = tiles;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int ua = __shfl_up_sync(0xffffffffu, a, o), ub = __shfl_up_sync(0xffffffffu, b, o);
      if ((tid & 31) >= o) { a += ua; b += ub; }
    }
    if ((tid & 31) == 31) { s_warp[0][tid >> 5] = a; s_warp[1][tid >> 5] = b; }
    __syncthreads();
    int wa = 0, wb = 0;
    for (int w = 0; w < (tid >> 5); ++w) { wa += s_warp[0][w]; wb += s_warp[1][w]; }
    const int d0 = s_carry[0] + wa + a - one, t0 = s_carry[1] + wb + b - tiles;
    if (one && d0 < n_decode && decode_rows) decode_rows[d0] = req_row0[i];
    for (int k = 0; k < tiles; ++k) {
      const int t = t0 + k;
      if (t >= n_tiles) break;
      const int off = k * tile_rows;
      const int r0 = req_row0[i] + off, n = min(tile_rows, cnt - off), pos = req_start[i] + off;
      if (sort) { s_row0[t] = r0; s_n[t] = n; s_pos[t] = pos; }
      else { tile_row0[t] = r0; tile_nrows[t] = n; }
    }
    __syncthreads();
    if (tid == PLAN_THREADS - 1) { s_carry[0] += wa + a; s_carry[1] += wb + b; }
    __syncthreads();
  }
  if (!sort) return;
  for (int t = tid; t < n_tiles; t += PLAN_THREADS) {
    const int pos = s_pos[t];
    int rank = 0;
    for (int j = 0; j < n_tiles; ++j) rank += (s_pos[j] > pos || (s_pos[j] == pos && j < t)) ? 1 : 0;
    tile_row0[rank] = s_row0[t];
    tile_nrows[rank] = s_n[t];
  }
}
}  // namespace

// Rows per tile of the prefill forms: which 0 = the `mma.sync` form, 1 = the tcgen05 form.
CUCA_API int cuca_attention_tile_rows(int which) { return which == 1 ? 128 : 64; }

// From (first row, token count, cached positions) of each of `n_req` requests: decode_rows[n_decode] = rows of the
// requests that bring one token, in request order (may be null when n_decode is 0 or every row is one);
// tile_row0/tile_nrows[n_tiles] = the longer portions in tiles of up to `tile_rows` rows, heaviest first.
// n_decode and n_tiles are the caller's counts (from the same per-request counts, on the host).
CUCA_API int cuca_attention_plan(const int* req_row0, const int* req_count, const int* req_start, int n_req,
                                 int tile_rows, int* decode_rows, int n_decode, int* tile_row0, int* tile_nrows,
                                 int n_tiles, cudaStream_t stream) {
  if (n_req == 0 || (n_tiles == 0 && (n_decode == 0 || !decode_rows))) return 0;
  CUCA_REQUIRE(tile_rows > 0, "attention_plan: tiles of %d rows", tile_rows);
  CUCA_REQUIRE(n_tiles == 0 || (tile_row0 && tile_nrows), "attention_plan: no room for the tiles");
  cuca_launch(attention_plan_kernel, dim3(1), dim3(PLAN_THREADS), 0, stream, true, req_row0, req_count, req_start,
              n_req, tile_rows, decode_rows, n_decode, tile_row0, tile_nrows, n_tiles);
  CUCA_CHECK_LAUNCH("attention_plan");
  return 0;
}
