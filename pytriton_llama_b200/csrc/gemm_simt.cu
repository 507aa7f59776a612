// out[M, N] (+)= A[M, K] * W[N, K]^T on the CUDA cores with float32 multiply-adds in a fixed
// k order: the true 32-bit matrix product of the float32 path (no tensor-core mode that drops
// mantissa bits), and a library-free check for the bfloat16 tensor-core kernels.
// Any M, N, K; both operands are K-contiguous.
#include "common.cuh"

namespace ptl {

template <typename TI, typename TO, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(TO* __restrict__ out, const TI* __restrict__ A, const TI* __restrict__ W,
                 int M, int N, int K, int lda, int ldw, int ldo, int accumulate) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN);  // along N
  const int ty = tid / (BN / TN);  // along M
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // cooperative loads: consecutive threads walk along K so that global reads coalesce
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
    __syncthreads();
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
      float v = acc[i][j];
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
  if (M > 32) {
    constexpr int BM = 128, BN = 64, BK = 16, TM = 8, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    PTL_REQUIRE(grid.y <= 65535, "gemm_simt: M=%d too large", M);
    return launch_kernel("gemm_simt", gemm_simt_kernel<TI, TO, BM, BN, BK, TM, TN>, grid, dim3((BM / TM) * (BN / TN)), 0,
                         as_stream(stream), (TO*)out, (const TI*)A, (const TI*)W, M, N, K, lda, ldw, ldo, accumulate);
  } else {
    constexpr int BM = 32, BN = 64, BK = 32, TM = 2, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    return launch_kernel("gemm_simt", gemm_simt_kernel<TI, TO, BM, BN, BK, TM, TN>, grid, dim3((BM / TM) * (BN / TN)), 0,
                         as_stream(stream), (TO*)out, (const TI*)A, (const TI*)W, M, N, K, lda, ldw, ldo, accumulate);
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
