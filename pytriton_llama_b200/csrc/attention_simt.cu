// Attention over the paged cache on the CUDA cores, for any mix of prompt portions and single
// decoded tokens: one warp per (token, query head), optional split of the key range over
// blockIdx.z with a merge kernel.  Everything but the stored q/k/v is float32: scores, running
// maximum, sum, accumulator, merge.  It is the float32 path's attention and the reference
// against which faster kernels are checked.
//
// With float32 inputs the two sums of attention are compensated, still in 32-bit arithmetic: the
// score q.k keeps the rounding error of every product and partial sum in a second float (a dot
// product as if summed in twice the precision), and the accumulator of P.V and the softmax sum are
// (high, low) pairs of floats.  Scores of size 10 make softmax weights as wrong (relatively) as the
// score is (absolutely), and a plain 64-term sum is wrong by a few 1e-7 there: over 16 layers of a
// 2,048-wide model these sums, not the matrix products, were what kept logits 8e-5 from a float64
// computation.  bfloat16 inputs (this kernel as the fallback for head sizes the tensor-core
// kernels leave) take plain sums: their inputs are a thousand times coarser than that.
//
// Token t (request r = tok_req[t], position p = positions[t]) sees keys lo..p of its request,
// lo = max(0, p - window + 1) when window > 0, else 0.  Key n lives in page
// block_table[r][n / page_size] at offset n % page_size of the layer's cache
// [pages][2 (k,v)][nkv][page_size][d].  Query head h reads kv head h / (nq / nkv).
#include "common.cuh"

namespace ptl {

constexpr int kMaxDimPerLane = 8;   // head sizes up to 256
constexpr int kWarpsPerBlock = 4;

// (hi, lo) += a * b without losing the rounding error of the product or of the sum
__device__ __forceinline__ void two_fma(float& hi, float& lo, float a, float b) {
  const float h = __fmul_rn(a, b);
  const float r = fmaf(a, b, -h);                             // the product's rounding error, exactly
  const float t = __fadd_rn(hi, h);
  const float z = __fsub_rn(t, hi);
  const float e = __fadd_rn(__fsub_rn(hi, __fsub_rn(t, z)), __fsub_rn(h, z));   // the sum's rounding error, exactly
  hi = t;
  lo = __fadd_rn(lo, __fadd_rn(e, r));
}
// (hi, lo) *= c
__device__ __forceinline__ void two_scale(float& hi, float& lo, float c) {
  const float h = __fmul_rn(hi, c);
  lo = fmaf(lo, c, fmaf(hi, c, -h));
  hi = h;
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
paged_attention_simt_kernel(T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                            const T* __restrict__ q, const T* __restrict__ cache,
                            const int* __restrict__ block_table, const int* __restrict__ tok_req,
                            const int* __restrict__ positions, int q_stride, int out_stride,
                            int bt_stride, int nq, int nkv, int d, int page_size, float scale,
                            int window, int splits, int num_pages) {
  extern __shared__ float qs_all[];  // [warps][d] scaled query
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * kWarpsPerBlock + warp;
  if (h >= nq) return;
  const int split = blockIdx.z;
  float* qs = qs_all + warp * d;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * d;
  constexpr bool kCompensated = sizeof(T) == 4;
  for (int i = lane; i < d; i += 32) qs[i] = kCompensated ? to_f32(qrow[i]) : to_f32(qrow[i]) * scale;
  __syncwarp();

  const int r = tok_req[t];        // r < 0: a padding row of a fixed-size batch; it sees no key and yields zeros
  const int p = positions[t];
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int nkeys = r < 0 ? 0 : p - lo + 1;
  int chunk = (nkeys + splits - 1) / splits;
  chunk = (chunk + 31) & ~31;
  const int k_begin = lo + split * chunk;
  const int k_end = r < 0 ? k_begin : min(lo + (split + 1) * chunk, p + 1);
  const int kvh = h / (nq / nkv);
  const size_t plane = (size_t)nkv * page_size * d;
  const int* bt = block_table + (size_t)(r < 0 ? 0 : r) * bt_stride;
  constexpr int VN = Vec16<T>::N;

  float m = -INFINITY, l = 0.f, l_lo = 0.f;
  float acc[kMaxDimPerLane], acc_lo[kMaxDimPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDimPerLane; ++i) { acc[i] = 0.f; acc_lo[i] = 0.f; }

  for (int k0 = k_begin; k0 < k_end; k0 += 32) {
    const int key = k0 + lane;
    bool valid = key < k_end;
    size_t base = 0;  // element offset of this lane's key row (k plane)
    float s = -INFINITY;
    const int page = valid ? bt[key / page_size] : 0;
    if (page < 0 || page >= num_pages) valid = false;  // never follow a table entry outside the pool
    if (valid) {
      base = ((size_t)page * 2) * plane + ((size_t)kvh * page_size + key % page_size) * d;
      const T* kp = cache + base;
      float dot = 0.f, dot_lo = 0.f;
      for (int i = 0; i < d; i += VN) {
        Vec16<T> kv = load16(kp + i);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          if constexpr (kCompensated) two_fma(dot, dot_lo, qs[i + e], kv.get(e));
          else dot = fmaf(qs[i + e], kv.get(e), dot);
        }
      }
      s = kCompensated ? __fadd_rn(dot, dot_lo) * scale : dot;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pr = valid ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);  // m = -inf on the first block gives 0
    if constexpr (kCompensated) {
      if (alpha != 1.f) {                 // (uniform over the warp) the maximum grew: everything so far shrinks
        two_scale(l, l_lo, alpha);
#pragma unroll
        for (int i = 0; i < kMaxDimPerLane; ++i) two_scale(acc[i], acc_lo[i], alpha);
      }
      two_fma(l, l_lo, warp_sum(pr), 1.f);
    } else {
      l = l * alpha + warp_sum(pr);
#pragma unroll
      for (int i = 0; i < kMaxDimPerLane; ++i) acc[i] *= alpha;
    }
    m = m_new;
    const int nvalid = min(32, k_end - k0);
    for (int j = 0; j < nvalid; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pr, j);
      const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      if (pj == 0.f) continue;   // uniform over the warp: a skipped key has no valid address
      const T* vp = cache + (size_t)bj + plane;
#pragma unroll
      for (int i = 0; i < kMaxDimPerLane; ++i) {
        const int dd = lane + 32 * i;
        if (dd < d) {
          if constexpr (kCompensated) two_fma(acc[i], acc_lo[i], pj, to_f32(vp[dd]));
          else acc[i] = fmaf(pj, to_f32(vp[dd]), acc[i]);
        }
      }
    }
  }
  if constexpr (kCompensated) {
    l = __fadd_rn(l, l_lo);
#pragma unroll
    for (int i = 0; i < kMaxDimPerLane; ++i) acc[i] = __fadd_rn(acc[i], acc_lo[i]);
  }

  if (splits == 1) {
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o = out + (size_t)t * out_stride + (size_t)h * d;
#pragma unroll
    for (int i = 0; i < kMaxDimPerLane; ++i) {
      const int dd = lane + 32 * i;
      if (dd < d) o[dd] = from_f32<T>(acc[i] * inv);
    }
  } else {
    const size_t idx = ((size_t)t * nq + h) * splits + split;
    float* pa = part_acc + idx * d;
#pragma unroll
    for (int i = 0; i < kMaxDimPerLane; ++i) {
      const int dd = lane + 32 * i;
      if (dd < d) pa[dd] = acc[i];
    }
    if (lane == 0) { part_ml[idx * 2] = m; part_ml[idx * 2 + 1] = l; }
  }
}

// Merge of the per-split partial results: out = sum_z e^{m_z - M} acc_z / sum_z e^{m_z - M} l_z.
// One warp per (token, head); the lanes share the weights of the splits and split the head's
// dimensions among them.
constexpr int kMergeWarps = 4;
template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32)
attention_merge_kernel(T* __restrict__ out, const float* __restrict__ part_acc,
                       const float* __restrict__ part_ml, int out_stride, int nq, int d,
                       int splits, const int* __restrict__ items, int n_rows) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x * kMergeWarps + warp;       // (row, head) pair
  if (pair >= n_rows * nq) return;
  const int ti = pair / nq, h = pair % nq;
  const int t = items ? items[ti] : ti;
  const size_t idx0 = ((size_t)t * nq + h) * splits;
  // lane z holds the (max, sum) pair of split z, 32 splits at a time; the weights are then handed
  // round by shuffles, so the loads of the partial accumulators below do not wait on one another
  float M = -INFINITY;
  for (int z = lane; z < splits; z += 32) M = fmaxf(M, part_ml[(idx0 + z) * 2]);
  M = warp_max(M);
  float L = 0.f;
  float acc[kMaxDimPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDimPerLane; ++i) acc[i] = 0.f;
  for (int z0 = 0; z0 < splits; z0 += 32) {
    const int z = z0 + lane;
    float wz = 0.f;
    if (z < splits) {
      const float mz = part_ml[(idx0 + z) * 2];
      if (mz > -INFINITY) {
        wz = expf(mz - M);
        L += wz * part_ml[(idx0 + z) * 2 + 1];
      }
    }
    const int n = min(32, splits - z0);
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
      const float wj = __shfl_sync(0xffffffffu, wz, j);
      const float* pa = part_acc + (idx0 + z0 + j) * d;      // an empty split wrote zeros here
#pragma unroll
      for (int i = 0; i < kMaxDimPerLane; ++i) {
        const int dd = lane + 32 * i;
        if (dd < d) acc[i] = fmaf(wj, pa[dd], acc[i]);
      }
    }
  }
  L = warp_sum(L);
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  T* o = out + (size_t)t * out_stride + (size_t)h * d;
#pragma unroll
  for (int i = 0; i < kMaxDimPerLane; ++i) {
    const int dd = lane + 32 * i;
    if (dd < d) o[dd] = from_f32<T>(acc[i] * inv);
  }
}

template <typename T>
int paged_attention_simt(void* out, const void* q, const void* cache, const int* block_table,
                         const int* tok_req, const int* positions, float* part_acc, float* part_ml,
                         int tokens, int q_stride, int out_stride, int bt_stride, int nq, int nkv, int d,
                         int page_size, float scale, int window, int splits, int num_pages, void* stream) {
  PTL_REQUIRE(tokens >= 0 && nq > 0 && nkv > 0 && page_size > 0, "paged_attention: bad sizes");
  PTL_REQUIRE(nq % nkv == 0, "paged_attention: %d query heads are no multiple of %d kv heads", nq, nkv);
  PTL_REQUIRE(d % 16 == 0 && d >= 16 && d <= 32 * kMaxDimPerLane, "paged_attention: head size %d must be a multiple of 16 in [16, %d]", d, 32 * kMaxDimPerLane);
  PTL_REQUIRE(splits >= 1 && splits <= 65535, "paged_attention: splits=%d", splits);
  PTL_REQUIRE(splits == 1 || (part_acc && part_ml), "paged_attention: splits > 1 need scratch buffers");
  PTL_REQUIRE(window >= 0 && num_pages > 0, "paged_attention: window must be >= 0 and the pool non-empty");
  PTL_REQUIRE(aligned16(q) && aligned16(cache) && (q_stride * sizeof(T)) % 16 == 0, "paged_attention: q and cache must be 16-byte aligned");
  if (tokens == 0) return 0;
  dim3 grid(tokens, (nq + kWarpsPerBlock - 1) / kWarpsPerBlock, splits);
  const size_t smem = (size_t)kWarpsPerBlock * d * sizeof(float);
  int rc = launch_kernel("paged_attention", paged_attention_simt_kernel<T>, grid, dim3(kWarpsPerBlock * 32), smem,
                         as_stream(stream), (T*)out, part_acc, part_ml, (const T*)q, (const T*)cache, block_table, tok_req,
                         positions, q_stride, out_stride, bt_stride, nq, nkv, d, page_size, scale, window, splits, num_pages);
  if (rc) return rc;
  if (splits > 1) {
    const long long pairs = (long long)tokens * nq;
    rc = launch_kernel("attention_merge", attention_merge_kernel<T>, dim3((unsigned)((pairs + kMergeWarps - 1) / kMergeWarps)),
                       dim3(kMergeWarps * 32), 0, as_stream(stream), (T*)out, (const float*)part_acc, (const float*)part_ml,
                       out_stride, nq, d, splits, (const int*)nullptr, tokens);
  }
  return rc;
}

// Merge for the tensor-core decode kernel: `items` (or 0..tokens-1) names the token rows.
int attention_merge_bf16(void* out, const float* part_acc, const float* part_ml, int tokens, int out_stride,
                         int nq, int d, int splits, const int* items, void* stream) {
  const long long pairs = (long long)tokens * nq;
  return launch_kernel("attention_merge", attention_merge_kernel<__nv_bfloat16>,
                       dim3((unsigned)((pairs + kMergeWarps - 1) / kMergeWarps)), dim3(kMergeWarps * 32), 0, as_stream(stream),
                       (__nv_bfloat16*)out, part_acc, part_ml, out_stride, nq, d, splits, items, tokens);
}

}  // namespace ptl

PTL_EXPORT int ptl_paged_attention_simt_f32(void* out, const void* q, const void* cache, const int* block_table, const int* tok_req, const int* positions, float* part_acc, float* part_ml, int tokens, int q_stride, int out_stride, int bt_stride, int nq, int nkv, int d, int page_size, float scale, int window, int splits, int num_pages, void* stream) {
  return ptl::paged_attention_simt<float>(out, q, cache, block_table, tok_req, positions, part_acc, part_ml, tokens, q_stride, out_stride, bt_stride, nq, nkv, d, page_size, scale, window, splits, num_pages, stream);
}
PTL_EXPORT int ptl_paged_attention_simt_bf16(void* out, const void* q, const void* cache, const int* block_table, const int* tok_req, const int* positions, float* part_acc, float* part_ml, int tokens, int q_stride, int out_stride, int bt_stride, int nq, int nkv, int d, int page_size, float scale, int window, int splits, int num_pages, void* stream) {
  return ptl::paged_attention_simt<__nv_bfloat16>(out, q, cache, block_table, tok_req, positions, part_acc, part_ml, tokens, q_stride, out_stride, bt_stride, nq, nkv, d, page_size, scale, window, splits, num_pages, stream);
}
