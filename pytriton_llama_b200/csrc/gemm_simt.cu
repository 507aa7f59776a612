// out[M, N] (+)= A[M, K] * W[N, K]^T on the CUDA cores in float32: the true 32-bit matrix product
// of the float32 path (no tensor-core mode that drops mantissa bits), and a library-free check for
// the bfloat16 tensor-core kernels.  Any M, N, K; both operands are K-contiguous.
//
// Summation order, the same for every tile shape, so that a row's result does not depend on how
// many rows the call has (a prompt portion and a single decoded token give the same bits):
// the K range is cut into chunks of 32; inside a chunk the products are added one by one with
// fused multiply-adds, k ascending, into a fresh accumulator; the chunk sums are added to the
// running total with a compensated (Kahan) addition.  A plain running sum over K = 8,192 terms is
// wrong by about K/4 ulp of a term, which over 16 layers of a 2,048-wide model reaches 3e-4 in the
// logits; with chunks the error of a product is that of one chunk, a few ulp.
#include "common.cuh"

namespace ptl {

constexpr int kSimtChunk = 32;       // k values per chunk: the tile depth of every kernel shape

// sum += chunk, with the rounding error of the addition carried in `comp`
__device__ __forceinline__ void kahan_add(float& sum, float& comp, float chunk) {
  const float y = __fsub_rn(chunk, comp);
  const float t = __fadd_rn(sum, y);
  comp = __fsub_rn(__fsub_rn(t, sum), y);
  sum = t;
}

template <typename TI, typename TO, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(TO* __restrict__ out, const TI* __restrict__ A, const TI* __restrict__ W,
                 int M, int N, int K, int lda, int ldw, int ldo, int accumulate, int vec_ok) {
  constexpr int BK = kSimtChunk;
  constexpr int THREADS = (BM / TM) * (BN / TN);
  static_assert(TM % 4 == 0 || TM == 2 || TM == 1, "rows per thread");
  pdl_wait();
  pdl_launch_dependents();
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN);  // along N
  const int ty = tid / (BN / TN);  // along M
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN], sum[TM][TN], comp[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) { sum[i][j] = 0.f; comp[i][j] = 0.f; }

  for (int k0 = 0; k0 < K; k0 += BK) {
    if (vec_ok) {
      // float32 operands whose rows start on 16-byte boundaries: four k values per load
      if constexpr (sizeof(TI) == 4) {
        for (int e = tid; e < BM * (BK / 4); e += THREADS) {
          const int r = e / (BK / 4), c4 = e % (BK / 4);
          const int gm = m0 + r, gk = k0 + c4 * 4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gm < M && gk < K) v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(A) + (size_t)gm * lda + gk);
          As[c4 * 4 + 0][r] = v.x; As[c4 * 4 + 1][r] = v.y; As[c4 * 4 + 2][r] = v.z; As[c4 * 4 + 3][r] = v.w;
        }
        for (int e = tid; e < BN * (BK / 4); e += THREADS) {
          const int r = e / (BK / 4), c4 = e % (BK / 4);
          const int gn = n0 + r, gk = k0 + c4 * 4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gn < N && gk < K) v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(W) + (size_t)gn * ldw + gk);
          Ws[c4 * 4 + 0][r] = v.x; Ws[c4 * 4 + 1][r] = v.y; Ws[c4 * 4 + 2][r] = v.z; Ws[c4 * 4 + 3][r] = v.w;
        }
      }
    } else {
      // any element type and alignment: consecutive threads walk along K so that global reads coalesce
      for (int e = tid; e < BM * BK; e += THREADS) {
        const int r = e / BK, c = e % BK;
        const int gm = m0 + r, gk = k0 + c;
        As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
      }
      for (int e = tid; e < BN * BK; e += THREADS) {
        const int r = e / BK, c = e % BK;
        const int gn = n0 + r, gk = k0 + c;
        Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) kahan_add(sum[i][j], comp[i][j], acc[i][j]);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      TO* o = out + (size_t)gm * ldo + gn;
      float v = sum[i][j];
      if (accumulate) v += to_f32(*o);
      *o = from_f32<TO>(v);
    }
  }
}

template <typename TI, typename TO>
int gemm_simt(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldo,
              int accumulate, void* stream) {
  PTL_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  PTL_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm_simt: pitches smaller than rows");
  if (M == 0) return 0;
  const int vec_ok = sizeof(TI) == 4 && K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && aligned16(A) && aligned16(W);
  if (M > 32) {
    constexpr int BM = 128, BN = 64, TM = 8, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    PTL_REQUIRE(grid.y <= 65535, "gemm_simt: M=%d too large", M);
    return launch_kernel("gemm_simt", gemm_simt_kernel<TI, TO, BM, BN, TM, TN>, grid, dim3((BM / TM) * (BN / TN)), 0,
                         as_stream(stream), (TO*)out, (const TI*)A, (const TI*)W, M, N, K, lda, ldw, ldo, accumulate, vec_ok);
  } else {
    // few rows: narrow tiles so that the weight matrix is spread over many blocks
    constexpr int BM = 32, BN = 16, TM = 4, TN = 1;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    return launch_kernel("gemm_simt", gemm_simt_kernel<TI, TO, BM, BN, TM, TN>, grid, dim3((BM / TM) * (BN / TN)), 0,
                         as_stream(stream), (TO*)out, (const TI*)A, (const TI*)W, M, N, K, lda, ldw, ldo, accumulate, vec_ok);
  }
}

}  // namespace ptl

PTL_EXPORT int ptl_gemm_simt_f32(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldo, int accumulate, void* stream) {
  return ptl::gemm_simt<float, float>(out, A, W, M, N, K, lda, ldw, ldo, accumulate, stream);
}
PTL_EXPORT int ptl_gemm_simt_bf16(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldo, int accumulate, void* stream) {
  return ptl::gemm_simt<__nv_bfloat16, __nv_bfloat16>(out, A, W, M, N, K, lda, ldw, ldo, accumulate, stream);
}
PTL_EXPORT int ptl_gemm_simt_bf16_f32out(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldo, int accumulate, void* stream) {
  return ptl::gemm_simt<__nv_bfloat16, float>(out, A, W, M, N, K, lda, ldw, ldo, accumulate, stream);
}
