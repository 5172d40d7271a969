// Token selection on the device, one block of 1024 threads per row, in the
// reference's order (src/provider/local/sampler.rs:159-331): temperature <= 0
// takes the first maximum; otherwise logits are divided by the temperature,
// cut to the top_k best by (logit descending, id ascending), soft-maxed, cut to
// the shortest most-likely-first prefix whose mass reaches top_p, and one token
// is drawn with target = u * total, first cumulative sum above the target, u
// from the request's own SplitMix64 state ((next_u64 >> 40) / 2^24).
//
// Up to 1024 ranked candidates are selected by a radix select on an order-
// preserving key, sorted in shared memory, and summed by one thread in sorted
// order, which reproduces the reference's 32-bit arithmetic step by step. Wider
// cuts (top_k above 1024, or a nucleus that needs more than 1024 candidates of
// a flat distribution) sort the whole vocabulary in a scratch row of global
// memory and use parallel prefix sums; without top_k and top_p the draw walks
// the vocabulary in id order, as the reference does.
#include "common.cuh"

namespace {

constexpr int NT = 1024;
constexpr int SMEM_CAND = 1024;

__device__ __forceinline__ unsigned ordered_key(float v) {
  // larger float -> larger key; NaN and infinities are never candidates, they map to 0
  if (!(fabsf(v) <= 3.402823466e38f)) return 0u;
  unsigned u = __float_as_uint(v);
  unsigned k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return k == 0u ? 1u : k;
}
__device__ __forceinline__ float key_value(unsigned k) {
  unsigned u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(u);
}
__device__ __forceinline__ unsigned long long composite(unsigned key, unsigned id) {
  return ((unsigned long long)key << 32) | (unsigned long long)(0xFFFFFFFFu - id);
}

struct Shared {
  unsigned long long cand[SMEM_CAND];
  float prob[SMEM_CAND];
  float fscan[NT];
  int iscan[NT];
  unsigned hist[256];
  unsigned long long red64[32];
  float redf[32];
  int misc[8];
  float fmisc[4];
};

__device__ float block_max(float v, Shared& sh) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) sh.redf[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh.redf[0];
  for (int i = 1; i < NT / 32; ++i) r = fmaxf(r, sh.redf[i]);
  __syncthreads();
  return r;
}
__device__ float block_sum(float v, Shared& sh) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sh.redf[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < NT / 32; ++i) r += sh.redf[i];
  __syncthreads();
  return r;
}
// inclusive scan of one float per thread; returns this thread's inclusive prefix, total in *total
__device__ float block_scan_f(float v, Shared& sh, float* total) {
  sh.fscan[threadIdx.x] = v;
  __syncthreads();
  for (int off = 1; off < NT; off <<= 1) {
    float add = threadIdx.x >= off ? sh.fscan[threadIdx.x - off] : 0.f;
    __syncthreads();
    sh.fscan[threadIdx.x] += add;
    __syncthreads();
  }
  float r = sh.fscan[threadIdx.x];
  *total = sh.fscan[NT - 1];
  __syncthreads();
  return r;
}
__device__ int block_scan_i(int v, Shared& sh, int* total) {
  sh.iscan[threadIdx.x] = v;
  __syncthreads();
  for (int off = 1; off < NT; off <<= 1) {
    int add = threadIdx.x >= off ? sh.iscan[threadIdx.x - off] : 0;
    __syncthreads();
    sh.iscan[threadIdx.x] += add;
    __syncthreads();
  }
  int r = sh.iscan[threadIdx.x];
  *total = sh.iscan[NT - 1];
  __syncthreads();
  return r;
}

// The largest (value, then lowest id) of row[lo..hi) as one 64-bit word: key of the value above 0xFFFFFFFF - id.
__device__ unsigned long long block_argmax_word(const float* row, int lo, int hi, Shared& sh) {
  unsigned long long best = 0ull;
  for (int i = lo + threadIdx.x; i < hi; i += NT) {
    float v = row[i];
    unsigned k = (v != v) ? 0u : ((__float_as_uint(v) & 0x80000000u) ? ~__float_as_uint(v) : (__float_as_uint(v) | 0x80000000u));
    unsigned long long c = composite(k, (unsigned)i);
    best = c > best ? c : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) sh.red64[threadIdx.x >> 5] = best;
  __syncthreads();
  best = sh.red64[0];
  for (int i = 1; i < NT / 32; ++i) best = sh.red64[i] > best ? sh.red64[i] : best;
  __syncthreads();
  return best;
}
__device__ __forceinline__ int argmax_id(unsigned long long best) {
  unsigned key = (unsigned)(best >> 32);
  // nothing above -inf: id 0, as the reference's greedy()
  if (key <= 0x007FFFFFu) return 0;  // key of -inf is ~0xFF800000 = 0x007FFFFF
  return (int)(0xFFFFFFFFu - (unsigned)(best & 0xFFFFFFFFull));
}
__device__ int block_argmax(const float* row, int V, Shared& sh) { return argmax_id(block_argmax_word(row, 0, V, sh)); }

// The m best candidates by (key desc, id asc) into sh.cand[0..m) sorted; m <= SMEM_CAND, m <= n_finite.
__device__ void select_sorted(const float* row, int V, float temp, int m, Shared& sh) {
  // radix select of the m-th largest key
  unsigned prefix = 0, mask = 0;
  int remaining = m;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += NT) sh.hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += NT) {
      unsigned k = ordered_key(row[i] / temp);
      if (k != 0u && (k & mask) == prefix) atomicAdd(&sh.hist[(k >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0, b = 255;
      for (; b > 0; --b) {
        if (acc + (int)sh.hist[b] >= remaining) break;
        acc += (int)sh.hist[b];
      }
      sh.misc[0] = b;
      sh.misc[1] = remaining - acc;
    }
    __syncthreads();
    prefix |= (unsigned)sh.misc[0] << shift;
    mask |= 255u << shift;
    remaining = sh.misc[1];
    __syncthreads();
  }
  const unsigned kth = prefix;   // key of the m-th best
  const int ties_wanted = remaining;  // how many of the candidates equal to kth make the cut (lowest ids first)
  if (threadIdx.x == 0) sh.misc[2] = 0;
  __syncthreads();
  // contiguous id chunks so that ties are taken in id order
  const int chunk = (V + NT - 1) / NT;
  const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
  int my_ties = 0;
  for (int i = lo; i < hi; ++i) {
    unsigned k = ordered_key(row[i] / temp);
    if (k > kth) {
      int slot = atomicAdd(&sh.misc[2], 1);
      sh.cand[slot] = composite(k, (unsigned)i);
    } else if (k == kth && k != 0u) {
      ++my_ties;
    }
  }
  int total_ties;
  int incl = block_scan_i(my_ties, sh, &total_ties);
  int rank = incl - my_ties;
  const int n_gt = sh.misc[2];
  for (int i = lo; i < hi && rank < ties_wanted; ++i) {
    unsigned k = ordered_key(row[i] / temp);
    if (k == kth && k != 0u) {
      sh.cand[n_gt + rank] = composite(k, (unsigned)i);
      ++rank;
    }
  }
  __syncthreads();
  // pad to a power of two and sort descending (bitonic)
  int n2 = 1;
  while (n2 < m) n2 <<= 1;
  for (int i = m + threadIdx.x; i < n2; i += NT) sh.cand[i] = 0ull;
  __syncthreads();
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      int i = threadIdx.x;
      if (i < n2) {
        int j = i ^ stride;
        if (j > i) {
          bool desc = (i & size) == 0;
          unsigned long long a = sh.cand[i], b = sh.cand[j];
          if ((a < b) == desc) { sh.cand[i] = b; sh.cand[j] = a; }
        }
      }
      __syncthreads();
    }
  }
}

__device__ __forceinline__ float next_uniform(unsigned long long* state) {
  unsigned long long s = *state + 0x9E3779B97F4A7C15ull;
  *state = s;
  unsigned long long z = s;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) / 16777216.0f;
}

// Thread 0: probabilities of sh.cand[0..m) relative to `denom` (0: their own sum), top-p cut, draw.
// Sequential 32-bit sums in sorted order, as the reference computes them.
__device__ int finish_sorted_smem(int m, float max_v, float denom, float top_p, unsigned long long* rng, Shared& sh) {
  for (int i = threadIdx.x; i < m; i += NT) sh.prob[i] = expf(key_value((unsigned)(sh.cand[i] >> 32)) - max_v);
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = denom;
    if (sum <= 0.f) {
      sum = 0.f;
      for (int i = 0; i < m; ++i) sum += sh.prob[i];
    }
    int kept = 0;  // candidates with probability above zero stay, in order
    float cumulative = 0.f;
    int keep = -1;
    for (int i = 0; i < m; ++i) {
      float p = sh.prob[i] / sum;
      if (!(p > 0.f)) continue;
      sh.prob[kept] = p;
      sh.cand[kept] = sh.cand[i];
      ++kept;
      cumulative += p;
      if (keep < 0 && cumulative >= top_p) { keep = kept; break; }
    }
    if (keep < 0) keep = kept;
    int result = -1;
    if (keep > 0) {
      float total = 0.f;
      for (int i = 0; i < keep; ++i) total += sh.prob[i];
      float target = next_uniform(rng) * total;
      float acc = 0.f;
      result = (int)(0xFFFFFFFFu - (unsigned)(sh.cand[keep - 1] & 0xFFFFFFFFull));
      for (int i = 0; i < keep; ++i) {
        acc += sh.prob[i];
        if (target < acc) { result = (int)(0xFFFFFFFFu - (unsigned)(sh.cand[i] & 0xFFFFFFFFull)); break; }
      }
    }
    sh.misc[3] = result;
  }
  __syncthreads();
  int r = sh.misc[3];
  __syncthreads();
  return r;
}

// First index i in [0, n) whose inclusive prefix sum of f(i) satisfies (ge ? >= : >) threshold; n if none.
// Every thread owns a contiguous chunk; *total gets the sum of all f(i).
template <typename F>
__device__ int prefix_find(F f, int n, float threshold, bool ge, Shared& sh, float* total) {
  const int chunk = (n + NT - 1) / NT;
  const int lo = min(n, threadIdx.x * chunk), hi = min(n, lo + chunk);
  float local = 0.f;
  for (int i = lo; i < hi; ++i) local += f(i);
  float incl = block_scan_f(local, sh, total);
  float before = incl - local;
  bool crosses = ge ? (incl >= threshold) : (incl > threshold);
  if (threadIdx.x == 0) sh.misc[4] = NT;
  __syncthreads();
  if (crosses && hi > lo) atomicMin(&sh.misc[4], (int)threadIdx.x);
  __syncthreads();
  if ((int)threadIdx.x == sh.misc[4]) {
    float acc = before;
    int found = hi - 1;
    for (int i = lo; i < hi; ++i) {
      acc += f(i);
      if (ge ? (acc >= threshold) : (acc > threshold)) { found = i; break; }
    }
    sh.misc[5] = found;
  }
  __syncthreads();
  int r = sh.misc[4] == NT ? n : sh.misc[5];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(NT)
sample_kernel(const float* __restrict__ logits, size_t row_stride, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, unsigned long long* __restrict__ rng,
              const int* __restrict__ slot_of_row, int* __restrict__ out, unsigned long long* __restrict__ scratch,
              int scratch_stride, unsigned long long* __restrict__ split_best, int* __restrict__ split_count) {
  __shared__ Shared sh;
  __shared__ int last_of_row;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int n_split = gridDim.y, part = blockIdx.y;
  const float* row = logits + (size_t)r * row_stride;
  const int slot = slot_of_row[r];
  if (slot < 0) {  // a padding row of a fixed-size batch
    if (threadIdx.x == 0 && part == 0) out[r] = -1;
    return;
  }
  const float temp = temperature[slot];
  if (!(temp > 0.f) || V <= 1) {
    if (n_split == 1) {
      int id = block_argmax(row, V, sh);
      if (threadIdx.x == 0) out[r] = id;
      return;
    }
    // A greedy row of a large vocabulary, cut over the CTAs of the row (one CTA alone reads 128,256 logits in
    // 28 us at its own pace): each takes the best of its part, the last to arrive takes the best of those. The
    // word orders by value, then by lowest id, so the result is the one CTA's.
    const int per = (V + n_split - 1) / n_split;
    const int lo = part * per, hi = min(V, lo + per);
    const unsigned long long best = block_argmax_word(row, lo, hi, sh);
    if (threadIdx.x == 0) {
      split_best[(size_t)r * n_split + part] = best;
      __threadfence();
      last_of_row = atomicAdd(&split_count[r], 1) == n_split - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!last_of_row) return;
    __threadfence();
    if (threadIdx.x < 32) {
      unsigned long long b = 0ull;
      for (int i = threadIdx.x; i < n_split; i += 32) {
        const unsigned long long c = *reinterpret_cast<volatile unsigned long long*>(&split_best[(size_t)r * n_split + i]);
        b = c > b ? c : b;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
        b = other > b ? other : b;
      }
      if (threadIdx.x == 0) {
        out[r] = argmax_id(b);
        split_count[r] = 0;  // ready for the next launch
      }
    }
    return;
  }
  if (part > 0) return;  // a row that draws is one CTA's work
  const int K = top_k[slot];
  const float P = top_p[slot];
  unsigned long long* state = rng + slot;

  // finite candidates and their maximum
  float mx = -INFINITY;
  int finite = 0;
  for (int i = threadIdx.x; i < V; i += NT) {
    float v = row[i] / temp;
    if (ordered_key(v) != 0u) { mx = fmaxf(mx, v); ++finite; }
  }
  mx = block_max(mx, sh);
  int n_finite;
  block_scan_i(finite, sh, &n_finite);
  if (n_finite == 0) {
    int id = block_argmax(row, V, sh);
    if (threadIdx.x == 0) out[r] = id;
    return;
  }
  const bool ranked = K > 0 && K < V;
  int result = -1;

  if (ranked && min(K, n_finite) <= SMEM_CAND) {
    int m = min(K, n_finite);
    select_sorted(row, V, temp, m, sh);
    result = finish_sorted_smem(m, mx, 0.f, P, state, sh);
  } else if (!ranked && P >= 1.0f) {
    // whole vocabulary, in id order
    float sum = 0.f;
    for (int i = threadIdx.x; i < V; i += NT) {
      float v = row[i] / temp;
      if (ordered_key(v) != 0u) sum += expf(v - mx);
    }
    sum = block_sum(sum, sh);
    auto prob = [&](int i) {
      float v = row[i] / temp;
      return ordered_key(v) != 0u ? expf(v - mx) / sum : 0.f;
    };
    float total;
    prefix_find(prob, V, INFINITY, false, sh, &total);
    float u = 0.f;
    if (threadIdx.x == 0) sh.fmisc[0] = next_uniform(state);
    __syncthreads();
    u = sh.fmisc[0];
    float dummy;
    int idx = prefix_find(prob, V, u * total, false, sh, &dummy);
    if (idx >= V) {  // rounding left the target above every prefix: the last candidate
      int last = -1;
      for (int i = threadIdx.x; i < V; i += NT) if (prob(i) > 0.f) last = max(last, i);
      last = (int)block_max((float)last, sh);
      idx = last;
    }
    result = idx;
  } else {
    // nucleus over the whole vocabulary (probabilities of the full distribution), or a top_k above 1024
    float sum = 0.f;
    bool done = false;
    if (!ranked) {
      for (int i = threadIdx.x; i < V; i += NT) {
        float v = row[i] / temp;
        if (ordered_key(v) != 0u) sum += expf(v - mx);
      }
      sum = block_sum(sum, sh);
      for (int m = 256; m <= SMEM_CAND && !done; m *= 4) {
        int mm = min(m, n_finite);
        select_sorted(row, V, temp, mm, sh);
        float part = 0.f;
        for (int i = threadIdx.x; i < mm; i += NT) part += expf(key_value((unsigned)(sh.cand[i] >> 32)) - mx);
        float mass = block_sum(part, sh) / sum;
        if (mass >= P || mm >= n_finite) {
          result = finish_sorted_smem(mm, mx, sum, P, state, sh);
          done = true;
        }
      }
    }
    if (!done) {
      if (scratch == nullptr) {
        if (threadIdx.x == 0) out[r] = -1;
        return;
      }
      // sort the whole vocabulary in this row's scratch
      unsigned long long* keys = scratch + (size_t)r * scratch_stride;
      int n2 = 1;
      while (n2 < V) n2 <<= 1;  // the host checked that a scratch row holds this many words
      for (int i = threadIdx.x; i < n2; i += NT)
        keys[i] = i < V ? (ordered_key(row[i] / temp) ? composite(ordered_key(row[i] / temp), (unsigned)i) : 0ull) : 0ull;
      __syncthreads();
      for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
          for (int i = threadIdx.x; i < n2; i += NT) {
            int j = i ^ stride;
            if (j > i) {
              bool desc = (i & size) == 0;
              unsigned long long a = keys[i], b = keys[j];
              if ((a < b) == desc) { keys[i] = b; keys[j] = a; }
            }
          }
          __syncthreads();
        }
      }
      int m = ranked ? min(K, n_finite) : n_finite;
      auto raw = [&](int i) { return expf(key_value((unsigned)(keys[i] >> 32)) - mx); };
      float denom = sum;
      float dummy;
      if (ranked) prefix_find(raw, m, INFINITY, false, sh, &denom);
      auto prob = [&](int i) { return raw(i) / denom; };
      int cut = prefix_find(prob, m, P, true, sh, &dummy);
      int keep = cut >= m ? m : cut + 1;
      float total;
      prefix_find(prob, keep, INFINITY, false, sh, &total);
      if (threadIdx.x == 0) sh.fmisc[0] = next_uniform(state);
      __syncthreads();
      float u = sh.fmisc[0];
      int idx = prefix_find(prob, keep, u * total, false, sh, &dummy);
      if (idx >= keep) idx = keep - 1;
      result = (int)(0xFFFFFFFFu - (unsigned)(keys[idx] & 0xFFFFFFFFull));
    }
  }
  if (result < 0) result = block_argmax(row, V, sh);
  if (threadIdx.x == 0) out[r] = result;
}

__global__ void __launch_bounds__(NT)
argmax_kernel(const float* __restrict__ logits, size_t row_stride, int V, int* __restrict__ out) {
  __shared__ Shared sh;
  int id = block_argmax(logits + (size_t)blockIdx.x * row_stride, V, sh);
  if (threadIdx.x == 0) out[blockIdx.x] = id;
}

}  // namespace

// out[r] = index of the first maximum of logits[r, 0..V)
CUCA_API int cuca_argmax(const float* logits, size_t row_stride, int n_rows, int V, int* out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(V > 0, "argmax: empty vocabulary");
  argmax_kernel<<<n_rows, NT, 0, stream>>>(logits, row_stride, V, out);
  CUCA_CHECK_LAUNCH("argmax");
  return 0;
}

namespace {
__global__ void suppress_kernel(float* __restrict__ logits, size_t row_stride, int V, const int* __restrict__ ids, int n) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  if (id >= 0 && id < V) logits[(size_t)blockIdx.y * row_stride + id] = -INFINITY;
}
}  // namespace

// logits[r, ids[i]] = -inf for every row: tokens that must never be sampled
// (src/provider/local/tokenizer/mod.rs:131-151, engine/scheduler.rs:1554). Ids outside the vocabulary are skipped.
CUCA_API int cuca_suppress_tokens(float* logits, size_t row_stride, int n_rows, int V, const int* ids, int n,
                                  cudaStream_t stream) {
  if (n_rows == 0 || n == 0) return 0;
  CUCA_REQUIRE(n_rows <= 65535, "suppress_tokens: too many rows");
  cuca_launch(suppress_kernel, dim3((n + 127) / 128, n_rows), dim3(128), 0, stream, true, logits, row_stride, V, ids, n);
  CUCA_CHECK_LAUNCH("suppress_tokens");
  return 0;
}

// Smallest scratch row (in 64-bit words) that lets cuca_sample sort a whole vocabulary of V ids.
CUCA_API int cuca_sample_scratch_stride(int V) {
  int n = 1;
  while (n < V) n <<= 1;
  return n;
}

// One token per row. temperature/top_k/top_p and rng (SplitMix64 states, advanced once per drawn token)
// are per request slot and indexed by slot_of_row[r]. scratch: n_rows * scratch_stride 64-bit words (may be null: rows that
// would need it then yield -1).
// split_best / split_count (may be null): split_rows x CUCA_SAMPLE_MAX_SPLIT 64-bit words and split_rows zeroed
// counters (left zeroed), with which the greedy rows of a large vocabulary are cut over several CTAs each.
CUCA_API int cuca_sample_max_split() { return 32; }
CUCA_API int cuca_sample(const float* logits, size_t row_stride, int n_rows, int V, const float* temperature,
                         const int* top_k, const float* top_p, unsigned long long* rng, const int* slot_of_row,
                         int* out, unsigned long long* scratch, int scratch_stride, unsigned long long* split_best,
                         int* split_count, int split_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(V > 0, "sample: empty vocabulary");
  CUCA_REQUIRE(scratch == nullptr || scratch_stride >= cuca_sample_scratch_stride(V),
               "sample: scratch rows of %d words are too short for a vocabulary of %d", scratch_stride, V);
  // about 8 K logits per CTA; rows times parts need not exceed a few hundred CTAs
  int n_split = 1;
  if (split_best && split_count && n_rows <= split_rows) {
    n_split = (V + 8191) / 8192;
    if (n_split > cuca_sample_max_split()) n_split = cuca_sample_max_split();
    while (n_split > 1 && n_rows * n_split > 1024) n_split /= 2;
    if (n_split < 1) n_split = 1;
  }
  cuca_launch(sample_kernel, dim3(n_rows, n_split), dim3(NT), 0, stream, true, logits, row_stride, V, temperature, top_k, top_p,
              rng, slot_of_row, out, scratch, scratch_stride, split_best, split_count);
  CUCA_CHECK_LAUNCH("sample");
  return 0;
}

namespace {
__global__ void decode_advance_kernel(int* __restrict__ tokens, int* __restrict__ positions,
                                      const int* __restrict__ slot_of_row, const int* __restrict__ sampled,
                                      int* __restrict__ history, int* __restrict__ counter, int n, int max_steps,
                                      const int* __restrict__ err, int* __restrict__ err_out) {
  pdl_trigger();
  pdl_wait();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  int step = *counter;
  if (i == 0 && err && err_out) *err_out = *err;
  if (i < n) {
    if (slot_of_row[i] >= 0) {
      tokens[i] = sampled[i];
      positions[i] += 1;
    }
    if (history && step < max_steps) history[(size_t)step * n + i] = sampled[i];
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) *counter = step + 1;
}
}  // namespace

// After a decode step: every live row's sampled token becomes its next input and its position moves on, so the
// same captured step can run again without the host; sampled tokens are also appended to history[step][row].
// One block only (n <= 1024), so the counter update is ordered after every read of it. `err_out` (may be null)
// receives the device error word as it stands after the step's kernels, so that the host's one read of the
// sampled tokens can bring it along.
CUCA_API int cuca_decode_advance(int* tokens, int* positions, const int* slot_of_row, const int* sampled,
                                 int* history, int* counter, int n, int max_steps, const int* err, int* err_out,
                                 cudaStream_t stream) {
  if (n == 0) return 0;
  CUCA_REQUIRE(n <= 1024, "decode_advance: at most 1024 rows");
  cuca_launch(decode_advance_kernel, dim3(1), dim3(1024), 0, stream, true, tokens, positions, slot_of_row, sampled,
              history, counter, n, max_steps, err, err_out);
  CUCA_CHECK_LAUNCH("decode_advance");
  return 0;
}
