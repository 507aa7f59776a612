// Next-token choice from float32 logits.
//
// temperature[row] <= 0: the index of the largest logit (the lowest index among equals).
// Otherwise: p_i = exp((x_i - max) / temperature); nucleus filter with lite_llama's rule (a token
// stays when the probability mass of all tokens more likely than it is <= top_p of the total, so
// the most likely one always stays); then one draw from the kept tokens by the uniform number
// u[row] in [0, 1), walking them in vocabulary order.  The caller supplies u, so the result does
// not depend on what else is in the batch.
//
// The filter needs no sort: with f(x) = sum of p_j over p_j > x, the kept tokens are exactly those
// with p_i >= x*, where x* is the smallest float with f(x*) <= top_p * total.  Positive floats
// order like their bit patterns, and p <= 1 has 30 significant pattern bits, so x* is found ten
// bits at a time: a histogram of probability mass over the top ten bits says which bucket x* lies
// in and how much of the budget is left for it, a second histogram over the next ten bits of that
// bucket's tokens narrows it again, a third one ends it.  Masses are added as 64-bit fixed-point
// numbers (p * 2^40): integer sums do not depend on their order, so the histograms can be built
// with atomics by 32 blocks per row and the choice is still the same in every run.
// Six launches per call (row maxima by slices; three histogram levels; the kept mass by slices;
// the draw), 32 blocks per row in the first five, so that a few rows still use many SMs.
// `probs` is scratch memory of [rows, vocab] floats; `work` of kSampleWorkPerRow 64-bit words per
// row, zero before the first call and left zero again by every call.
#include "common.cuh"

namespace ptl {


__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if (lane == 0) { sv[warp] = v; si[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    float tv = lane < nwarps ? sv[lane] : -INFINITY;
    int ti = lane < nwarps ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, tv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, ti, o);
      if (ov > tv || (ov == tv && oi < ti)) { tv = ov; ti = oi; }
    }
    if (lane == 0) { sv[32] = tv; si[32] = ti; }
  }
  __syncthreads();
  v = sv[32];
  idx = si[32];
}

// log softmax(logits[row])[tokens[row]] of the unscaled logits
// (lite_llama/generete_with_probs.py:154-165 takes the same quantity with log_softmax + gather),
// in two stages so that a few rows still use many SMs: the maximum and the sum of exp(x - maximum)
// of each of 32 slices of a row, then the 32 pairs of a row brought to one maximum and added in slice order.
constexpr int kLogprobChunks = 32;
constexpr int kLogprobThreads = 256;

__global__ void __launch_bounds__(kLogprobThreads)
token_logprob_partial_kernel(float* __restrict__ part_max, float* __restrict__ part_sum, const float* __restrict__ logits,
                             int vocab, long long ld) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const int per = (vocab + kLogprobChunks - 1) / kLogprobChunks;
  const int lo = chunk * per, hi = min(lo + per, vocab);
  const float* x = logits + (size_t)row * ld;
  float mx = -INFINITY;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) mx = fmaxf(mx, x[i]);
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) sum += expf(x[i] - mx);
  sum = block_sum(sum, red);
  if (threadIdx.x == 0) {
    part_max[row * kLogprobChunks + chunk] = mx;
    part_sum[row * kLogprobChunks + chunk] = sum;
  }
}

__global__ void token_logprob_final_kernel(float* __restrict__ out, const float* __restrict__ part_max,
                                           const float* __restrict__ part_sum, const float* __restrict__ logits,
                                           const int* __restrict__ tokens, int vocab, long long ld) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, lane = threadIdx.x;
  const float m = part_max[row * kLogprobChunks + lane];
  float mx = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float mine = m == -INFINITY ? 0.f : part_sum[row * kLogprobChunks + lane] * expf(m - mx);
  float sum = 0.f;
  for (int k = 0; k < kLogprobChunks; ++k) sum += __shfl_sync(0xffffffffu, mine, k);      // in slice order
  if (lane == 0) {
    const int t = tokens[row];
    out[row] = (t >= 0 && t < vocab) ? logits[(size_t)row * ld + t] - mx - logf(sum) : -INFINITY;
  }
}

// Greedy choice for whole batches in two stages, so that a few rows still use many SMs:
// stage 1 finds the best (value, index) of each of `chunks` slices of a row, stage 2 the best of those.
constexpr int kArgmaxChunks = 32;
constexpr int kArgmaxThreads = 256;

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_partial_kernel(float* __restrict__ part_val, int* __restrict__ part_idx, const float* __restrict__ logits,
                      int vocab, long long ld) {
  __shared__ float sv[33];
  __shared__ int si[33];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const int per = (vocab + kArgmaxChunks - 1) / kArgmaxChunks;
  const int lo = chunk * per, hi = min(lo + per, vocab);
  const float* x = logits + (size_t)row * ld;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = x[i];
    if (v > best || (v == best && i < besti)) { best = v; besti = i; }
  }
  block_argmax(best, besti, sv, si);
  if (threadIdx.x == 0) {
    part_val[row * kArgmaxChunks + chunk] = best;
    part_idx[row * kArgmaxChunks + chunk] = besti;
  }
}

__global__ void argmax_final_kernel(int* __restrict__ tokens, const float* __restrict__ part_val,
                                    const int* __restrict__ part_idx) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, lane = threadIdx.x;
  float v = part_val[row * kArgmaxChunks + lane];
  int idx = part_idx[row * kArgmaxChunks + lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  if (lane == 0) tokens[row] = idx;
}


// ---------------------------------------------------------------- temperature and nucleus sampling
constexpr int kSampleBuckets = 1024;                     // ten pattern bits per level
constexpr int kSampleLevelThreads = 256;
constexpr int kSampleBatch = 8;                          // loads a thread has in flight
constexpr int kSampleWorkPerRow = 3 * kSampleBuckets + 64;   // 64-bit words of `work` per row: three histograms, 32 kept masses, the cut
constexpr float kSampleFixedPoint = 1099511627776.f;     // 2^40

__device__ __forceinline__ unsigned long long mass_of(float e) { return __float2ull_rz(e * kSampleFixedPoint); }

__device__ __forceinline__ unsigned long long warp_scan_u64(unsigned long long v, int lane) {     // inclusive
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// Inclusive scan over the block's threads in thread order (up to 1,024 threads); every thread also
// gets the block's total.  `scratch` holds 33 words.
__device__ __forceinline__ unsigned long long block_scan_u64(unsigned long long v, unsigned long long* scratch,
                                                             unsigned long long& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_scan_u64(v, lane);
  __syncthreads();                                       // (scratch may still be read from the scan before)
  if (lane == 31) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long t = lane < nwarps ? scratch[lane] : 0ull;
    t = warp_scan_u64(t, lane);
    scratch[lane] = t;
    if (lane == 31) scratch[32] = t;
  }
  __syncthreads();
  if (warp > 0) v += scratch[warp - 1];
  total = scratch[32];
  return v;
}

// Where x* lies among the buckets of one histogram: the smallest bucket b such that the mass in
// the buckets above b is <= budget, and what is left of the budget after that mass.  Every thread
// of a 256-thread block calls it with its four buckets h[0..3] = buckets 4 (255 - t) .. + 3 (thread 0
// has the top four) and gets both, and the histogram's total mass.
__device__ __forceinline__ void find_bucket(const unsigned long long (&h)[4], unsigned long long budget,
                                            unsigned long long* scratch, int* s_bucket, unsigned long long* s_left,
                                            int& bucket, unsigned long long& left) {
  const int b0 = kSampleBuckets - 4 * ((int)threadIdx.x + 1);
  const unsigned long long mine = h[0] + h[1] + h[2] + h[3];
  unsigned long long total;
  const unsigned long long incl = block_scan_u64(mine, scratch, total);
  unsigned long long above = incl - mine;                // mass in the buckets above this thread's four
  // the predicate "mass above b <= budget" holds for the top bucket and, going down, up to some bucket: the last one is it
  int best = -1;
  unsigned long long best_left = 0ull;
#pragma unroll
  for (int j = 3; j >= 0; --j) {                         // from this thread's highest bucket down
    if (above <= budget) { best = b0 + j; best_left = budget - above; }
    above += h[j];
  }
  // the smallest such bucket over the block: threads further down hold smaller buckets
  if (best >= 0) atomicMin(s_bucket + 1, best);
  __syncthreads();
  if (best >= 0 && best == s_bucket[1]) *s_left = best_left;
  __syncthreads();
  bucket = s_bucket[1];
  left = *s_left;
}

struct SampleLevelArgs {
  const float* logits;
  float* probs;
  const float* temperature;
  const float* top_p;
  const float* part_val;          // [rows][32] maxima of the slices of every row
  unsigned long long* work;       // [rows][kSampleWorkPerRow]: three histograms, the kept mass of the 32 slices, the cut
  int vocab;
  long long ld;
};

// total mass, budget, and down LEVELS histograms of the row: the pattern bits of x* found so far.
// Every thread of a 256-thread block calls it; s_bucket[1] need not be prepared.  The buckets of all
// levels are fetched at once, before the first scan: the levels then cost no trip to L2 each.
template <int LEVELS>
__device__ __forceinline__ unsigned descend(const unsigned long long* __restrict__ work, float top_p,
                                            unsigned long long* scratch, int* s_bucket, unsigned long long* s_left) {
  unsigned long long h[LEVELS][4];
  const int b0 = kSampleBuckets - 4 * ((int)threadIdx.x + 1);
#pragma unroll
  for (int level = 0; level < LEVELS; ++level)
#pragma unroll
    for (int j = 0; j < 4; ++j) h[level][j] = __ldcg(work + level * kSampleBuckets + b0 + j);
  unsigned long long total;
  block_scan_u64(h[0][0] + h[0][1] + h[0][2] + h[0][3], scratch, total);
  unsigned long long budget = top_p >= 1.f ? total : (unsigned long long)((double)top_p * (double)total);
  unsigned prefix = 0u;
#pragma unroll
  for (int level = 0; level < LEVELS; ++level) {
    __syncthreads();
    if (threadIdx.x == 0) s_bucket[1] = kSampleBuckets;
    __syncthreads();
    int bucket;
    find_bucket(h[level], budget, scratch, s_bucket, s_left, bucket, budget);
    prefix = (prefix << 10) | (unsigned)bucket;
  }
  return prefix;
}

// A block's histogram of mass lives in shared memory as three 32-bit counters per bucket (14 bits
// of the 42-bit mass each: 32-bit shared-memory adds are native, 64-bit ones are compare-and-swap
// loops that crawl when many threads meet in a bucket); a slice has few enough tokens that none overflows.
__device__ __forceinline__ void hist_add(unsigned* hist, unsigned bucket, unsigned long long q) {
  atomicAdd(hist + bucket, (unsigned)(q & 0x3fffu));
  atomicAdd(hist + kSampleBuckets + bucket, (unsigned)((q >> 14) & 0x3fffu));
  atomicAdd(hist + 2 * kSampleBuckets + bucket, (unsigned)(q >> 28));
}

// LEVEL 0: p = exp((x - max) / T) into `probs`, histogram of mass over pattern bits 29..20.
// LEVEL 1: bucket of level 0 from its histogram, histogram over bits 19..10 of that bucket's tokens.
// LEVEL 2: likewise over bits 9..0.
// LEVEL 3: the cut is known: the kept mass of this block's slice (and, from slice 0, the cut itself).
template <int LEVEL>
__global__ void __launch_bounds__(kSampleLevelThreads)
sample_level_kernel(const SampleLevelArgs a) {
  __shared__ unsigned hist[3 * kSampleBuckets];
  __shared__ unsigned long long scratch[33];
  __shared__ int s_bucket[2];
  __shared__ unsigned long long s_left;
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x / kArgmaxChunks, chunk = blockIdx.x % kArgmaxChunks;
  const float temp = a.temperature[row];
  if (!(temp > 0.f)) return;                             // a greedy row: the last kernel takes the largest logit
  const int tid = threadIdx.x;
  if (LEVEL < 3)
    for (int b = tid; b < 3 * kSampleBuckets; b += blockDim.x) hist[b] = 0u;
  unsigned long long* work = a.work + (size_t)row * kSampleWorkPerRow;
  float* pr = a.probs + (size_t)row * a.vocab;
  const int per = (a.vocab + kArgmaxChunks - 1) / kArgmaxChunks;
  const int lo = chunk * per, hi = min(lo + per, a.vocab);
  unsigned prefix = 0u;
  if constexpr (LEVEL >= 1) prefix = descend<LEVEL>(work, a.top_p[row], scratch, s_bucket, &s_left);
  __syncthreads();
  if (LEVEL == 0) {
    float mx = -INFINITY;
    for (int k = 0; k < kArgmaxChunks; ++k) mx = fmaxf(mx, a.part_val[row * kArgmaxChunks + k]);
    const float inv_t = 1.0f / temp;
    const float* x = a.logits + (size_t)row * a.ld;
    // (loads in batches of eight ahead of the adds: an atomic between two loads would make every load wait for the one before)
    for (int base = lo + tid; base < hi; base += kSampleBatch * kSampleLevelThreads) {
      float v[kSampleBatch];
#pragma unroll
      for (int j = 0; j < kSampleBatch; ++j) {
        const int i = base + j * kSampleLevelThreads;
        v[j] = i < hi ? __ldg(x + i) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < kSampleBatch; ++j) {
        const int i = base + j * kSampleLevelThreads;
        if (i < hi) {
          const float e = expf((v[j] - mx) * inv_t);
          pr[i] = e;
          hist_add(hist, min(__float_as_uint(e) >> 20, (unsigned)kSampleBuckets - 1u), mass_of(e));     // (p <= 1 stays below; a NaN must not leave the table)
        }
      }
    }
  } else if (LEVEL < 3) {
    const int shift = LEVEL == 1 ? 10 : 0;
    for (int base = lo + tid; base < hi; base += kSampleBatch * kSampleLevelThreads) {
      float v[kSampleBatch];
#pragma unroll
      for (int j = 0; j < kSampleBatch; ++j) {
        const int i = base + j * kSampleLevelThreads;
        v[j] = i < hi ? __ldcg(pr + i) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < kSampleBatch; ++j) {
        const unsigned pat = __float_as_uint(v[j]);
        if (base + j * kSampleLevelThreads < hi && (pat >> (shift + 10)) == prefix)
          hist_add(hist, (pat >> shift) & (kSampleBuckets - 1), mass_of(v[j]));
      }
    }
  } else {
    unsigned long long mine = 0ull, kept;
    for (int base = lo + tid; base < hi; base += kSampleBatch * kSampleLevelThreads) {
      float v[kSampleBatch];
#pragma unroll
      for (int j = 0; j < kSampleBatch; ++j) {
        const int i = base + j * kSampleLevelThreads;
        v[j] = i < hi ? __ldcg(pr + i) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < kSampleBatch; ++j)
        if (base + j * kSampleLevelThreads < hi && __float_as_uint(v[j]) >= prefix) mine += mass_of(v[j]);
    }
    block_scan_u64(mine, scratch, kept);
    if (tid == 0) {
      work[3 * kSampleBuckets + chunk] = kept;
      if (chunk == 0) work[3 * kSampleBuckets + kArgmaxChunks] = prefix;
    }
    return;
  }
  __syncthreads();
  unsigned long long* out = work + LEVEL * kSampleBuckets;
  for (int b = tid; b < kSampleBuckets; b += blockDim.x) {
    const unsigned long long q = (unsigned long long)hist[b] + ((unsigned long long)hist[kSampleBuckets + b] << 14) +
                                 ((unsigned long long)hist[2 * kSampleBuckets + b] << 28);
    if (q) atomicAdd(out + b, q);
  }
}

// One block per row: the slice that holds the draw from the 32 slices' kept masses, the token
// inside it.  Leaves the row's histograms zero.
__global__ void __launch_bounds__(kSampleLevelThreads)
sample_draw_kernel(int* __restrict__ tokens, const SampleLevelArgs a, const int* __restrict__ part_idx,
                   const float* __restrict__ u) {
  __shared__ unsigned long long scratch[33];
  __shared__ int s_owner;
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, tid = threadIdx.x;
  // the largest of the slices' maxima, the lowest index among equals
  int top_idx = 0;
  {
    float v = tid < kArgmaxChunks ? a.part_val[row * kArgmaxChunks + tid] : -INFINITY;
    int idx = tid < kArgmaxChunks ? part_idx[row * kArgmaxChunks + tid] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    top_idx = idx;                                       // (valid in warp 0)
  }
  const float temp = a.temperature ? a.temperature[row] : 0.f;
  if (!(temp > 0.f)) {
    if (tid == 0) tokens[row] = top_idx;
    return;
  }
  unsigned long long* work = a.work + (size_t)row * kSampleWorkPerRow;
  const unsigned long long* kept = work + 3 * kSampleBuckets;
  const unsigned cut_bits = (unsigned)__ldcg(kept + kArgmaxChunks);
  // which slice: lane k of every warp holds slice k's kept mass; a scan over the lanes
  const int lane = tid & 31;
  const unsigned long long c = __ldcg(kept + lane);
  const unsigned long long c_incl = warp_scan_u64(c, lane);
  const unsigned long long kept_total = __shfl_sync(0xffffffffu, c_incl, 31);
  const unsigned long long target = (unsigned long long)((double)u[row] * (double)kept_total);    // < kept_total because u < 1
  const unsigned holds = __ballot_sync(0xffffffffu, c > 0ull && c_incl - c <= target && target < c_incl);
  const int chunk = holds ? __ffs(holds) - 1 : -1;
  const unsigned long long before_chunk = __shfl_sync(0xffffffffu, c_incl - c, chunk < 0 ? 0 : chunk);
  for (int b = tid; b < 3 * kSampleBuckets; b += blockDim.x) work[b] = 0ull;      // zero again for the next call
  if (tid == 0) s_owner = -1;
  __syncthreads();
  if (chunk < 0) {                                       // (no mass survived the fixed-point conversion: it cannot, the largest p is 1)
    if (tid == 0) tokens[row] = top_idx;
    return;
  }
  const float* pr = a.probs + (size_t)row * a.vocab;
  const int per = (a.vocab + kArgmaxChunks - 1) / kArgmaxChunks;
  const int lo = chunk * per, hi = min(lo + per, a.vocab);
  const int mine_n = (hi - lo + blockDim.x - 1) / blockDim.x;
  const int c0 = min(lo + tid * mine_n, hi), c1 = min(c0 + mine_n, hi);
  unsigned long long mine = 0ull;
  for (int i0 = c0; i0 < c1; i0 += kSampleBatch) {
    float v[kSampleBatch];
#pragma unroll
    for (int j = 0; j < kSampleBatch; ++j) v[j] = i0 + j < c1 ? __ldcg(pr + i0 + j) : 0.f;
#pragma unroll
    for (int j = 0; j < kSampleBatch; ++j)
      if (i0 + j < c1 && __float_as_uint(v[j]) >= cut_bits) mine += mass_of(v[j]);
  }
  unsigned long long chunk_total;
  const unsigned long long incl = before_chunk + block_scan_u64(mine, scratch, chunk_total);
  const unsigned long long before = incl - mine;
  if (mine > 0ull && before <= target && target < incl) s_owner = tid;        // exactly one thread's tokens hold the target
  __syncthreads();
  if (tid == s_owner) {
    unsigned long long acc = before;
    int choice = c0;
    bool found = false;
    for (int i0 = c0; i0 < c1 && !found; i0 += kSampleBatch) {
      float v[kSampleBatch];                             // (fetched together: one trip to L2 per batch, not per token)
#pragma unroll
      for (int j = 0; j < kSampleBatch; ++j) v[j] = i0 + j < c1 ? __ldcg(pr + i0 + j) : 0.f;
#pragma unroll
      for (int j = 0; j < kSampleBatch; ++j) {
        const unsigned long long q = mass_of(v[j]);
        if (!found && i0 + j < c1 && __float_as_uint(v[j]) >= cut_bits && q > 0ull) {
          choice = i0 + j;
          acc += q;
          found = acc > target;
        }
      }
    }
    tokens[row] = choice;
  }
}

}  // namespace ptl

// scratch: rows * 32 floats and rows * 32 ints
PTL_EXPORT int ptl_argmax(int* tokens, const float* logits, float* part_val, int* part_idx, int rows, int vocab,
                          long long ld, void* stream) {
  static_assert(ptl::kArgmaxChunks == 32, "the final stage is one warp");
  PTL_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab && rows <= 65535, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return 0;
  dim3 grid(ptl::kArgmaxChunks, rows);
  int rc = ptl::launch_kernel("argmax_partial", ptl::argmax_partial_kernel, grid, dim3(ptl::kArgmaxThreads), 0,
                              ptl::as_stream(stream), part_val, part_idx, logits, vocab, ld);
  if (rc) return rc;
  return ptl::launch_kernel("argmax_final", ptl::argmax_final_kernel, dim3(rows), dim3(32), 0, ptl::as_stream(stream), tokens,
                            (const float*)part_val, (const int*)part_idx);
}

// scratch: rows * 32 floats twice
PTL_EXPORT int ptl_token_logprob(float* out, const float* logits, const int* tokens, float* part_max, float* part_sum,
                                 int rows, int vocab, long long ld, void* stream) {
  using namespace ptl;
  static_assert(kLogprobChunks == 32, "the final stage is one warp");
  PTL_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "token_logprob: bad sizes rows=%d vocab=%d", rows, vocab);
  PTL_REQUIRE(part_max && part_sum, "token_logprob: needs the scratch of the slices' maxima and sums");
  if (rows == 0) return 0;
  for (int r0 = 0; r0 < rows; r0 += 65535) {              // (blockIdx.y is the row: up to 65,535 a launch)
    const int n = rows - r0 < 65535 ? rows - r0 : 65535;
    int rc = launch_kernel("token_logprob_partial", token_logprob_partial_kernel, dim3(kLogprobChunks, n), dim3(kLogprobThreads), 0,
                           as_stream(stream), part_max + (size_t)r0 * kLogprobChunks, part_sum + (size_t)r0 * kLogprobChunks,
                           logits + (size_t)r0 * ld, vocab, ld);
    if (rc) return rc;
  }
  return launch_kernel("token_logprob_final", token_logprob_final_kernel, dim3(rows), dim3(32), 0, as_stream(stream), out,
                       (const float*)part_max, (const float*)part_sum, logits, tokens, vocab, ld);
}

// Greedy rows (temperature == nullptr or <= 0) take the largest logit; the others are sampled as the
// head of this file says.  `part_val`, `part_idx`: scratch of rows * 32 floats and ints; `probs`
// [rows, vocab] floats; `work` rows * ptl_sample_work_words() 64-bit words, zero before the first
// call (every call leaves them zero).  Without temperature only the first two are needed.
PTL_EXPORT int ptl_sample_work_words() { return ptl::kSampleWorkPerRow; }
PTL_EXPORT int ptl_sample(int* tokens, const float* logits, float* probs, const float* temperature,
                          const float* top_p, const float* u, float* part_val, int* part_idx,
                          unsigned long long* work, int rows, int vocab, long long ld, void* stream) {
  using namespace ptl;
  PTL_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d ld=%lld", rows, vocab, ld);
  PTL_REQUIRE(part_val && part_idx, "sample: needs the scratch of the slices' maxima");
  PTL_REQUIRE(temperature == nullptr || (probs && top_p && u && work), "sample: temperature sampling needs probs and work scratch, top_p and u");
  PTL_REQUIRE((long long)rows * kArgmaxChunks <= 0x7fffffffLL, "sample: too many rows");
  PTL_REQUIRE(temperature == nullptr || vocab < kArgmaxChunks * (1 << 18), "sample: a vocabulary of %d is too large for the 32-bit counters of a slice", vocab);
  if (rows == 0) return 0;
  cudaStream_t s = as_stream(stream);
  // the slices' maxima (blockIdx.y is the row there: up to 65,535 rows a launch)
  for (int r0 = 0; r0 < rows; r0 += 65535) {
    const int n = rows - r0 < 65535 ? rows - r0 : 65535;
    int rc = launch_kernel("argmax_partial", argmax_partial_kernel, dim3(kArgmaxChunks, n), dim3(kArgmaxThreads), 0, s,
                           part_val + (size_t)r0 * kArgmaxChunks, part_idx + (size_t)r0 * kArgmaxChunks, logits + (size_t)r0 * ld, vocab, ld);
    if (rc) return rc;
  }
  SampleLevelArgs a{logits, probs, temperature, top_p, part_val, work, vocab, ld};
  if (temperature) {
    const dim3 grid((unsigned)rows * kArgmaxChunks), block(kSampleLevelThreads);
    if (int rc = launch_kernel("sample_level0", sample_level_kernel<0>, grid, block, 0, s, a)) return rc;
    if (int rc = launch_kernel("sample_level1", sample_level_kernel<1>, grid, block, 0, s, a)) return rc;
    if (int rc = launch_kernel("sample_level2", sample_level_kernel<2>, grid, block, 0, s, a)) return rc;
    if (int rc = launch_kernel("sample_kept", sample_level_kernel<3>, grid, block, 0, s, a)) return rc;
  }
  return launch_kernel("sample_draw", sample_draw_kernel, dim3(rows), dim3(kSampleLevelThreads), 0, s, tokens, a, (const int*)part_idx, u);
}

PTL_EXPORT const char* ptl_last_error() { return ptl::error_buffer(); }
// Switches programmatic dependent launch of the library's kernels on (default) or off.
PTL_EXPORT void ptl_set_dependent_launch(int enabled) { ptl::pdl_flag() = enabled ? 1 : 0; }
PTL_EXPORT int ptl_get_dependent_launch() { return ptl::pdl_flag(); }

// Measurement only (see common.cuh): from now on the decode step's kernels stamp %globaltimer into
// `buffer` (device memory, 16 words per launch, `slots` launches); ptl_timeline_end() stops that and
// says how many slots were handed out.  A captured graph keeps the slots it was captured with.
PTL_EXPORT void ptl_timeline_begin(unsigned long long* buffer, int slots) {
  ptl::timeline_state() = ptl::TimelineState{buffer, slots, 0};
}
PTL_EXPORT int ptl_timeline_end() {
  const int used = ptl::timeline_state().next;
  ptl::timeline_state() = ptl::TimelineState{nullptr, 0, 0};
  return used;
}
PTL_EXPORT int ptl_abi_version() { return 1; }
