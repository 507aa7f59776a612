// out[M, N] = X[M, K] * W[N, K]^T in bfloat16 for steps of up to 8 tokens and weight matrices of a
// few megabytes (the q|k|v and output projections of a decode step): a kernel bound by latency, not
// by bandwidth.  The tcgen05 product splits such a K range over a cluster of eight blocks and pays
// for tensor-memory allocation, a ring of TMA stages, remote shared-memory stores and two cluster
// barriers: 4 to 6 us for 1 to 2 us worth of weights.  Here a block owns 8 output features for the
// whole K range, so nothing crosses blocks:
//   * before the wait on the predecessor kernel every warp requests its K slice of the block's 8
//     weight rows into shared memory (cp.async; weights depend on no earlier kernel);
//   * after the wait the same warp requests its slice of the tokens, and without any block-wide
//     barrier runs its mma.sync m16n8k16 steps (weights are the 16-row operand, rows 8..15 zero;
//     the 8 token columns are the other operand) as soon as its own copies have landed;
//   * the eight warps' partial sums meet in shared memory, are added in warp order (deterministic)
//     and go through the same epilogues as the tcgen05 product: bfloat16 or float32 store, or add
//     into the float32 residual, optionally preparing the next RMS norm's input (xs = bfloat16(new
//     residual * norm weight) and one sum of squares per token and block), and optionally finishing
//     the norm before it (every output row scaled by rsqrt(mean of the token's squares + eps)).
// Sizes: M <= 8, K % 8 == 0, and as many blocks as are resident at once (the launcher says no
// otherwise and the caller takes the tcgen05 product).
#include "mma_utils.cuh"

namespace ptl {

constexpr int kSmallRows = 8;        // output features per block
constexpr int kSmallTokens = 8;      // token columns of the MMA
constexpr int kSmallWarps = 8;
constexpr int kSmallPad = 8;         // bfloat16 of padding per shared-memory row: rows start in different banks

struct SmallGemmParams {
  void* out;
  const __nv_bfloat16* X;
  const __nv_bfloat16* W;
  int M, N, K, ld_out;
  int k_per_warp;                    // multiple of 16
  // add epilogue preparing the next norm (all null otherwise)
  __nv_bfloat16* xs;
  const float* norm_w;
  float* sumsq;
  int xs_ld, sumsq_ld;
  // finishing the norm before this product
  const float* scale_sumsq;
  int scale_slots, scale_ld;
  float scale_eps, scale_inv_n;
  unsigned long long* timeline;
  int timeline_kind;
};

// EPI: 0 bfloat16 store, 1 float32 store, 2 add into the float32 residual
template <int EPI>
__global__ void __launch_bounds__(kSmallWarps * 32, 3)
gemm_small_kernel(const SmallGemmParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0 && p.timeline) { timeline_stamp(p.timeline, 0); if (blockIdx.x == 0) p.timeline[0] = p.timeline_kind; }
  const int kpad = kSmallWarps * p.k_per_warp;                 // K rounded up to the warps' slices
  const int row_elems = kpad + kSmallPad;
  __nv_bfloat16* sW = reinterpret_cast<__nv_bfloat16*>(smem_raw);                        // [8][row_elems]
  __nv_bfloat16* sX = sW + kSmallRows * row_elems;                                        // [8][row_elems]
  float* s_part = reinterpret_cast<float*>(sX + kSmallTokens * row_elems);                // [warps][8 rows][8 tokens]
  float* s_scale = s_part + kSmallWarps * kSmallRows * kSmallTokens;                      // [8 tokens]
  const int n0 = blockIdx.x * kSmallRows;
  const int k0 = warp * p.k_per_warp;
  const int chunks = p.k_per_warp / 8;                         // 16-byte chunks of a row's slice

  // ---- this warp's slice of the weights: 8 rows x k_per_warp, zero beyond N and K
  for (int e = lane; e < kSmallRows * chunks; e += 32) {
    const int r = e / chunks, c = e % chunks;
    const int k = k0 + c * 8;
    const bool valid = n0 + r < p.N && k < p.K;
    cp_async_16(smem_u32(sW + r * row_elems + k), p.W + (size_t)(valid ? n0 + r : 0) * p.K + (valid ? k : 0), valid);
  }
  cp_async_commit();
  pdl_wait();
  pdl_launch_dependents();
  if (tid == 0) timeline_stamp(p.timeline, 1);
  // ---- its slice of the tokens
  for (int e = lane; e < kSmallTokens * chunks; e += 32) {
    const int r = e / chunks, c = e % chunks;
    const int k = k0 + c * 8;
    const bool valid = r < p.M && k < p.K;
    cp_async_16(smem_u32(sX + r * row_elems + k), p.X + (size_t)(valid ? r : 0) * p.K + (valid ? k : 0), valid);
  }
  cp_async_commit();
  // what the epilogue adds to or multiplies by is fetched under the copies: thread (token, row)
  const int e_tok = tid / kSmallRows, e_row = tid % kSmallRows;
  const int n = n0 + e_row;
  const bool e_valid = tid < kSmallRows * kSmallTokens && e_tok < p.M && n < p.N;
  float have = 0.f, nw = 0.f;
  if (EPI == 2 && e_valid) {
    have = __ldcg((const float*)p.out + (size_t)e_tok * p.ld_out + n);
    if (p.xs) nw = __ldg(p.norm_w + n);
  }
  if (p.scale_sumsq) {
    // the scale of every token: 32 threads per token add its slots up
    const int tok = tid >> 5;
    float sum = 0.f;
    if (tok < p.M)
      for (int k = lane; k < p.scale_slots; k += 32) sum += __ldcg(p.scale_sumsq + (size_t)tok * p.scale_ld + k);
    sum = warp_sum(sum);
    if (lane == 0) s_scale[tok] = tok < p.M ? rsqrtf(sum * p.scale_inv_n + p.scale_eps) : 0.f;
  }
  cp_async_wait<0>();
  __syncwarp();
  if (tid == 0) timeline_stamp(p.timeline, 2);

  // ---- the warp's partial sums: rows 0..7 of the 16-row operand are the block's weight rows
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  {
    // ldmatrix x4: matrices 0, 1 = weights (k 0..7, k 8..15 of the step), 2, 3 = tokens likewise
    const int mat = lane >> 3, rr = lane & 7;
    const __nv_bfloat16* base = (mat < 2 ? sW : sX) + rr * row_elems + k0 + (mat & 1) * 8;
    uint32_t addr = smem_u32(base);
#pragma unroll 4
    for (int ks = 0; ks < p.k_per_warp; ks += 16, addr += 32) {
      uint32_t f[4];
      ldmatrix_x4(f, addr);
      const uint32_t a[4] = {f[0], 0u, f[1], 0u};              // a0 (rows 0..7, k 0..7), a2 (rows 0..7, k 8..15); rows 8..15 are zero
      mma_bf16_16816(acc, a, f[2], f[3]);
    }
  }
  // c0, c1: row lane / 4, tokens 2 (lane % 4) ..+1
  {
    float* dst = s_part + (warp * kSmallRows + (lane >> 2)) * kSmallTokens + 2 * (lane & 3);
    dst[0] = acc[0];
    dst[1] = acc[1];
  }
  __syncthreads();
  if (tid == 0) { timeline_stamp(p.timeline, 3); timeline_stamp(p.timeline, 4); }

  // ---- epilogue: thread (token, row) adds the warps' partial sums in order
  float r_new = 0.f;
  if (tid < kSmallRows * kSmallTokens) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kSmallWarps; ++w) v += s_part[(w * kSmallRows + e_row) * kSmallTokens + e_tok];
    if (p.scale_sumsq) v *= s_scale[e_tok];
    if (e_valid) {
      if (EPI == 0) ((__nv_bfloat16*)p.out)[(size_t)e_tok * p.ld_out + n] = __float2bfloat16_rn(v);
      else if (EPI == 1) ((float*)p.out)[(size_t)e_tok * p.ld_out + n] = v;
      else {
        r_new = have + v;
        ((float*)p.out)[(size_t)e_tok * p.ld_out + n] = r_new;
        if (p.xs) p.xs[(size_t)e_tok * p.xs_ld + n] = __float2bfloat16_rn(r_new * nw);
      }
    }
    if (EPI == 2 && p.xs) {
      // the token's sum of squares over this block's 8 features: the 8 lanes that hold them
      float sq = e_valid ? r_new * r_new : 0.f;
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      if (e_row == 0 && e_tok < p.M) p.sumsq[(size_t)e_tok * p.sumsq_ld + blockIdx.x] = sq;
    }
  }
  if (tid == 0) timeline_stamp(p.timeline, 5);
}

template <int EPI>
static int launch_small(const SmallGemmParams& p, int blocks, size_t smem, cudaStream_t stream) {
  static SmemRaised raised = {};
  if (int rc = raise_shared_memory("gemm_small", gemm_small_kernel<EPI>, 100 * 1024, raised)) return rc;
  return launch_kernel("gemm_small", gemm_small_kernel<EPI>, dim3(blocks), dim3(kSmallWarps * 32), smem, stream, p);
}

}  // namespace ptl

// Returns 0, -1 on an error, or -2 when the sizes are not this kernel's (more than 8 tokens, K no
// multiple of 8, rows too long for three blocks per SM, or more blocks than are resident at once):
// the caller then takes the tcgen05 product.  Arguments as ptl_gemm_tc_bf16_norm (epi 0, 1 or 2);
// with `xs` a token gets one slot of `sumsq` per 8 features, *slots_out = ceil(N / 8).
PTL_EXPORT int ptl_gemm_small_bf16(void* out, const void* X, const void* W, int M, int N, int K, int ld_out, int epi,
                                   void* xs, const float* norm_w, float* sumsq, int sumsq_ld, int* slots_out,
                                   const float* scale_sumsq, int scale_slots, int scale_ld, float scale_eps, void* stream) {
  using namespace ptl;
  PTL_REQUIRE(M >= 0 && N > 0 && K > 0 && ld_out > 0, "gemm_small: bad sizes M=%d N=%d K=%d", M, N, K);
  if (M > kSmallTokens || K % 8 != 0 || epi < 0 || epi > 2) return -2;
  if (M == 0) return 0;
  PTL_REQUIRE(aligned16(X) && aligned16(W), "gemm_small: operands must be 16-byte aligned");
  SmallGemmParams p{};
  p.out = out; p.X = (const __nv_bfloat16*)X; p.W = (const __nv_bfloat16*)W;
  p.M = M; p.N = N; p.K = K; p.ld_out = ld_out;
  p.k_per_warp = ((K + kSmallWarps - 1) / kSmallWarps + 15) / 16 * 16;
  const int row_elems = kSmallWarps * p.k_per_warp + kSmallPad;
  const size_t smem = (size_t)(kSmallRows + kSmallTokens) * row_elems * 2 + (kSmallWarps * kSmallRows * kSmallTokens + kSmallTokens) * 4;
  const int blocks = (N + kSmallRows - 1) / kSmallRows;
  static int resident = 0;                                // blocks of this kernel the device holds at once: three per SM
  if (!resident) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    resident = 3 * (sms > 0 ? sms : 148);
  }
  if (smem > 74 * 1024 || blocks > resident) return -2;
  if (xs) {
    if (epi != 2) return -2;
    PTL_REQUIRE(norm_w && sumsq && slots_out && sumsq_ld >= blocks, "gemm_small: the next norm's input needs its weight, the sums (a slot per 8 features) and a place for their count");
    p.xs = (__nv_bfloat16*)xs; p.norm_w = norm_w; p.sumsq = sumsq; p.xs_ld = N; p.sumsq_ld = sumsq_ld;
    *slots_out = blocks;
  }
  if (scale_sumsq) {
    if (epi == 2) return -2;
    PTL_REQUIRE(scale_slots > 0 && scale_ld >= scale_slots && scale_eps > 0.f, "gemm_small: bad row scale arguments");
    p.scale_sumsq = scale_sumsq; p.scale_slots = scale_slots; p.scale_ld = scale_ld; p.scale_eps = scale_eps;
    p.scale_inv_n = 1.0f / (float)K;
  }
  p.timeline = timeline_slot();
  p.timeline_kind = 20 + epi;
  cudaStream_t s = as_stream(stream);
  switch (epi) {
    case 0: return launch_small<0>(p, blocks, smem, s);
    case 1: return launch_small<1>(p, blocks, smem, s);
    default: return launch_small<2>(p, blocks, smem, s);
  }
}
