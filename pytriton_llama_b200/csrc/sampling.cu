// Next-token choice from float32 logits, one block per row.
//
// temperature[row] <= 0: the index of the largest logit (the lowest index among equals).
// Otherwise: p_i = exp((x_i - max) / temperature); nucleus filter with lite_llama's rule (a token
// stays when the probability mass of all tokens more likely than it is <= top_p of the total, so
// the most likely one always stays); then one draw from the kept tokens by the uniform number
// u[row] in [0, 1), walking them in vocabulary order.  The caller supplies u, so the result does
// not depend on what else is in the batch.
//
// The filter needs no sort: with f(x) = sum of p_j over p_j > x, the kept tokens are exactly those
// with p_i >= x*, where x* is the smallest float with f(x*) <= top_p * total; x* is found by
// bisection on the bit pattern (positive floats order like their bits).
// `probs` is scratch memory of [rows, vocab] floats.
#include "common.cuh"

namespace ptl {

constexpr int kSampleThreads = 1024;

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

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(int* __restrict__ tokens, const float* __restrict__ logits, float* __restrict__ probs,
              const float* __restrict__ temperature, const float* __restrict__ top_p,
              const float* __restrict__ u, int vocab, long long ld) {
  __shared__ float sv[33];
  __shared__ int si[33];
  __shared__ float red[33];
  __shared__ float chunk_sum[kSampleThreads];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ld;
  const int tid = threadIdx.x;

  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = x[i];
    if (v > best || (v == best && i < besti)) { best = v; besti = i; }
  }
  block_argmax(best, besti, sv, si);
  const float temp = temperature ? temperature[row] : 0.f;
  if (!(temp > 0.f)) {
    if (tid == 0) tokens[row] = besti;
    return;
  }
  float* pr = probs + (size_t)row * vocab;
  const float inv_t = 1.0f / temp;
  float part = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float e = expf((x[i] - best) * inv_t);
    pr[i] = e;
    part += e;
  }
  const float total = block_sum(part, red);
  const float budget = top_p[row] * total;

  // bisection for the smallest bit pattern b with f(float(b)) <= budget
  unsigned lo = 0u, hi = __float_as_uint(1.0f);  // f(1) = 0 because the largest p is exactly 1
  {
    float s = 0.f;
    for (int i = tid; i < vocab; i += blockDim.x) { const float e = pr[i]; if (e > 0.f) s += e; }
    s = block_sum(s, red);
    if (s <= budget) hi = 0u;  // everything stays
  }
  while (hi - lo > 1u && hi != 0u) {
    const unsigned mid = lo + (hi - lo) / 2u;
    const float thr = __uint_as_float(mid);
    float s = 0.f;
    for (int i = tid; i < vocab; i += blockDim.x) { const float e = pr[i]; if (e > thr) s += e; }
    s = block_sum(s, red);
    if (s <= budget) hi = mid; else lo = mid;
  }
  const float cut = __uint_as_float(hi);

  // draw: contiguous chunk per thread, exclusive scan over the chunk sums, walk inside one chunk
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int c0 = min(tid * per, vocab), c1 = min(c0 + per, vocab);
  float mine = 0.f;
  for (int i = c0; i < c1; ++i) { const float e = pr[i]; if (e >= cut) mine += e; }
  chunk_sum[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    float kept_total = 0.f;
    for (int k = 0; k < blockDim.x; ++k) kept_total += chunk_sum[k];
    const float target = u[row] * kept_total;
    float run = 0.f;       // kept mass of the chunks before `owner`
    int owner = -1;
    int last = 0;          // the last non-empty chunk catches a target that rounding pushed past the end
    float before_last = 0.f;
    for (int k = 0; k < blockDim.x; ++k) {
      const float c = chunk_sum[k];
      if (c > 0.f) {
        if (run + c > target) { owner = k; break; }
        last = k;
        before_last = run;
        run += c;
      }
    }
    if (owner < 0) { owner = last; run = before_last; }
    const int o0 = min(owner * per, vocab), o1 = min(o0 + per, vocab);
    int choice = besti;
    float acc = run;
    for (int i = o0; i < o1; ++i) {
      const float e = pr[i];
      if (e >= cut) {
        choice = i;
        acc += e;
        if (acc > target) break;
      }
    }
    tokens[row] = choice;
  }
}

// log softmax(logits[row])[tokens[row]] of the unscaled logits, one block per row
// (lite_llama/generete_with_probs.py:154-165 takes the same quantity with log_softmax + gather).
__global__ void __launch_bounds__(kSampleThreads)
token_logprob_kernel(float* __restrict__ out, const float* __restrict__ logits, const int* __restrict__ tokens,
                     int vocab, long long ld) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ld;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, x[i]);
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) sum += expf(x[i] - mx);
  sum = block_sum(sum, red);
  if (threadIdx.x == 0) {
    const int t = tokens[row];
    out[row] = (t >= 0 && t < vocab) ? x[t] - mx - logf(sum) : -INFINITY;
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

PTL_EXPORT int ptl_token_logprob(float* out, const float* logits, const int* tokens, int rows, int vocab, long long ld,
                                 void* stream) {
  PTL_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "token_logprob: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return 0;
  return ptl::launch_kernel("token_logprob", ptl::token_logprob_kernel, dim3(rows), dim3(ptl::kSampleThreads), 0,
                            ptl::as_stream(stream), out, logits, tokens, vocab, ld);
}

PTL_EXPORT int ptl_sample(int* tokens, const float* logits, float* probs, const float* temperature,
                          const float* top_p, const float* u, int rows, int vocab, long long ld,
                          void* stream) {
  PTL_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d ld=%lld", rows, vocab, ld);
  PTL_REQUIRE(temperature == nullptr || (probs && top_p && u), "sample: temperature sampling needs probs scratch, top_p and u");
  if (rows == 0) return 0;
  return ptl::launch_kernel("sample", ptl::sample_kernel, dim3(rows), dim3(ptl::kSampleThreads), 0, ptl::as_stream(stream),
                            tokens, logits, probs, temperature, top_p, u, vocab, ld);
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
