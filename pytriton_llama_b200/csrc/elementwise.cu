// Row-wise kernels: embedding gather, residual add fused with RMSNorm, SiLU(gate)*up.
// Each takes any width (no power of two needed); 16-byte packets are used when the row pitch
// allows it, scalars otherwise.
#include "common.cuh"

namespace ptl {

// ------------------------------------------------------------------ embedding
// out[t, :] = table[ids[t], :].  An id outside [0, vocab) writes zeros and raises *status.
template <typename T>
__global__ void embed_gather_kernel(T* __restrict__ out, const T* __restrict__ table,
                                    const int* __restrict__ ids, int hidden, int vocab,
                                    int vec_ok, int* __restrict__ status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0 && status) atomicExch(status, 1);
  T* dst = out + (size_t)t * hidden;
  const T* src = table + (size_t)(bad ? 0 : id) * hidden;
  constexpr int VN = Vec16<T>::N;
  if (vec_ok) {
    for (int i = threadIdx.x * VN; i < hidden; i += blockDim.x * VN) {
      Vec16<T> v = load16(src + i);
      if (bad) {
#pragma unroll
        for (int k = 0; k < VN; ++k) v.set(k, 0.f);
      }
      store16(dst + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = bad ? from_f32<T>(0.f) : src[i];
  }
}

// ------------------------------------------------------------------ add + RMSNorm
// For output row m (input row r = rows ? rows[m] : m):
//   s = (residual_in ? residual_in[r] : 0) + (x ? x[r] : 0)          in float32
//   residual_out[m] = s                                              (if residual_out)
//   y[m] = s * rsqrt(mean(s^2) + eps) * w                            rounded once to T
// The row is kept in shared memory between the two passes.
template <typename T>
__global__ void add_rmsnorm_kernel(T* __restrict__ y, float* __restrict__ residual_out,
                                   const float* __restrict__ residual_in, const T* __restrict__ x,
                                   const float* __restrict__ w, const int* __restrict__ rows,
                                   int hidden, float eps, int vec_ok) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x;
  const int r = rows ? rows[m] : m;
  const float* rin = residual_in ? residual_in + (size_t)r * hidden : nullptr;
  const T* xin = x ? x + (size_t)r * hidden : nullptr;
  float* rout = residual_out ? residual_out + (size_t)m * hidden : nullptr;
  T* yo = y + (size_t)m * hidden;
  float ss = 0.f;
  if (vec_ok) {
    // four elements per thread and turn: 16-byte packets of the float32 arrays, 8 or 16 bytes of T
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float4 s = rin ? *reinterpret_cast<const float4*>(rin + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (xin) {
        if constexpr (sizeof(T) == 4) {
          const float4 v = *reinterpret_cast<const float4*>(xin + i);
          s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        } else {
          const uint2 raw = *reinterpret_cast<const uint2*>(xin + i);
          const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          s.x += __bfloat162float(a.x); s.y += __bfloat162float(a.y);
          s.z += __bfloat162float(b.x); s.w += __bfloat162float(b.y);
        }
      }
      *reinterpret_cast<float4*>(row + i) = s;
      if (rout && (xin || rout != rin)) *reinterpret_cast<float4*>(rout + i) = s;   // unchanged rows are not rewritten
      ss += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
    ss = block_sum(ss, red);
    const float rrms = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      const float4 s = *reinterpret_cast<const float4*>(row + i);
      const float4 g = *reinterpret_cast<const float4*>(w + i);
      if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(yo + i) = make_float4(s.x * rrms * g.x, s.y * rrms * g.y, s.z * rrms * g.z, s.w * rrms * g.w);
      } else {
        uint2 o;
        *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(s.x * rrms * g.x, s.y * rrms * g.y);
        *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(s.z * rrms * g.z, s.w * rrms * g.w);
        *reinterpret_cast<uint2*>(yo + i) = o;
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float s = rin ? rin[i] : 0.f;
    if (xin) s += to_f32(xin[i]);
    row[i] = s;
    ss += s * s;
  }
  ss = block_sum(ss, red);
  const float rrms = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float s = row[i];
    if (rout && (xin || rout != rin)) rout[i] = s;
    yo[i] = from_f32<T>(s * rrms * w[i]);
  }
}

// The same for many rows of a width of N4 * 128: one warp per row, the row in registers (N4 packets
// of four per lane), no shared memory and no block-wide barrier.
template <typename T, int N4>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(T* __restrict__ y, float* __restrict__ residual_out, const float* __restrict__ residual_in,
                        const T* __restrict__ x, const float* __restrict__ w, const int* __restrict__ rows, int out_rows,
                        float eps) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int hidden = N4 * 128;
  const int lane = threadIdx.x & 31;
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= out_rows) return;
  const int r = rows ? rows[m] : m;
  const float* rin = residual_in ? residual_in + (size_t)r * hidden : nullptr;
  const T* xin = x ? x + (size_t)r * hidden : nullptr;
  float* rout = residual_out ? residual_out + (size_t)m * hidden : nullptr;
  T* yo = y + (size_t)m * hidden;
  float4 s[N4];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < N4; ++k) {
    const int i = (k * 32 + lane) * 4;
    s[k] = rin ? __ldcg(reinterpret_cast<const float4*>(rin + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (xin) {
      if constexpr (sizeof(T) == 4) {
        const float4 v = *reinterpret_cast<const float4*>(xin + i);
        s[k].x += v.x; s[k].y += v.y; s[k].z += v.z; s[k].w += v.w;
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(xin + i);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        s[k].x += __bfloat162float(a.x); s[k].y += __bfloat162float(a.y);
        s[k].z += __bfloat162float(b.x); s[k].w += __bfloat162float(b.y);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < N4; ++k) ss += s[k].x * s[k].x + s[k].y * s[k].y + s[k].z * s[k].z + s[k].w * s[k].w;
  ss = warp_sum(ss);
  const float rrms = 1.0f / sqrtf(ss / (float)hidden + eps);
  const bool write_back = rout && (xin || rout != rin);      // unchanged rows are not rewritten
#pragma unroll
  for (int k = 0; k < N4; ++k) {
    const int i = (k * 32 + lane) * 4;
    if (write_back) *reinterpret_cast<float4*>(rout + i) = s[k];
    const float4 g = __ldg(reinterpret_cast<const float4*>(w + i));
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(yo + i) = make_float4(s[k].x * rrms * g.x, s[k].y * rrms * g.y, s[k].z * rrms * g.z, s[k].w * rrms * g.w);
    } else {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(s[k].x * rrms * g.x, s[k].y * rrms * g.y);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(s[k].z * rrms * g.z, s[k].w * rrms * g.w);
      *reinterpret_cast<uint2*>(yo + i) = o;
    }
  }
}

// ------------------------------------------------------------------ SiLU(gate) * up
// gu is [T, 2*inter] (gate columns first); out[t, i] = g * sigmoid(g) * u in float32.
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter, int vec_ok) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.y;
  const T* g = gu + (size_t)t * 2 * inter;
  const T* u = g + inter;
  T* o = out + (size_t)t * inter;
  constexpr int VN = Vec16<T>::N;
  if (vec_ok) {
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * VN;
    if (i < inter) {
      Vec16<T> a = load16(g + i), b = load16(u + i), c;
#pragma unroll
      for (int k = 0; k < VN; ++k) {
        const float gv = a.get(k);
        c.set(k, gv / (1.0f + expf(-gv)) * b.get(k));
      }
      store16(o + i, c);
    }
  } else {
    for (int k = 0; k < VN; ++k) {
      const int i = (blockIdx.x * blockDim.x + threadIdx.x) * VN + k;
      if (i < inter) {
        const float gv = to_f32(g[i]);
        o[i] = from_f32<T>(gv / (1.0f + expf(-gv)) * to_f32(u[i]));
      }
    }
  }
}

// tokens[i] = sampled[src[i]] where src[i] >= 0: a step whose input token is the one the previous
// step sampled takes it on the device, before the host has read it.
__global__ void take_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                   const int* __restrict__ sampled, int n, int n_sampled) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int s = src[i];
  if (s >= 0 && s < n_sampled) tokens[i] = sampled[s];
}

// acc[i] = (((acc[i] + parts[0][i]) + parts[1][i]) + ...): the partial sums of a product whose K
// range was cut into parts, added into the residual in a fixed order (n4 groups of four values;
// part s starts s * stride4 groups after the first).
__global__ void add_partials_kernel(float4* __restrict__ acc, const float4* __restrict__ parts, int n_parts, size_t n4, size_t stride4) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 a = acc[i];
  float4 q[8];
  for (int s0 = 0; s0 < n_parts; s0 += 8) {
#pragma unroll
    for (int s = 0; s < 8; ++s) q[s] = s0 + s < n_parts ? __ldcg(parts + (size_t)(s0 + s) * stride4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (s0 + s < n_parts) { a.x += q[s].x; a.y += q[s].y; a.z += q[s].z; a.w += q[s].w; }
  }
  acc[i] = a;
}

template <typename T>
int embed_gather(void* out, const void* table, const int* ids, int tokens, int hidden, int vocab,
                 int* status, void* stream) {
  PTL_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embed_gather: bad sizes tokens=%d hidden=%d vocab=%d", tokens, hidden, vocab);
  if (tokens == 0) return 0;
  const int vec_ok = (hidden % Vec16<T>::N == 0) && aligned16(out) && aligned16(table);
  int threads = 128;
  return launch_kernel("embed_gather", embed_gather_kernel<T>, dim3(tokens), dim3(threads), 0, as_stream(stream),
                       (T*)out, (const T*)table, ids, hidden, vocab, vec_ok, status);
}

template <typename T>
int add_rmsnorm(void* y, float* residual_out, const float* residual_in, const void* x, const float* w,
                const int* rows, int out_rows, int hidden, float eps, void* stream) {
  PTL_REQUIRE(out_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", out_rows, hidden);
  PTL_REQUIRE(residual_in || x, "add_rmsnorm: needs a residual or an input");
  PTL_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
  if (out_rows == 0) return 0;
  const size_t smem = (size_t)hidden * sizeof(float);
  PTL_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: hidden=%d does not fit the row buffer (max %d)", hidden, 200 * 1024 / 4);
  static SmemRaised raised = {};                      // one per instance of this template
  if (smem > 48 * 1024)
    if (int rc = raise_shared_memory("add_rmsnorm", add_rmsnorm_kernel<T>, 200 * 1024, raised)) return rc;
  const int vec_ok = hidden % 4 == 0 && aligned16(y) && aligned16(w) && (!x || aligned16(x)) &&
                     (!residual_in || aligned16(residual_in)) && (!residual_out || aligned16(residual_out));
  // many rows of a common width: a warp per row
  if (vec_ok && out_rows >= 256 && hidden % 512 == 0 && hidden <= 4096) {
    const dim3 grid((out_rows + 7) / 8), block(256);
#define PTL_NORM_ROWS(N4) launch_kernel("add_rmsnorm", add_rmsnorm_warp_kernel<T, N4>, grid, block, 0, as_stream(stream), \
                                        (T*)y, residual_out, residual_in, (const T*)x, w, rows, out_rows, eps)
    switch (hidden) {
      case 512: return PTL_NORM_ROWS(4);
      case 1024: return PTL_NORM_ROWS(8);
      case 1536: return PTL_NORM_ROWS(12);
      case 2048: return PTL_NORM_ROWS(16);
      case 2560: return PTL_NORM_ROWS(20);
      case 3072: return PTL_NORM_ROWS(24);
      case 3584: return PTL_NORM_ROWS(28);
      default: return PTL_NORM_ROWS(32);
    }
#undef PTL_NORM_ROWS
  }
  int threads = hidden >= 8192 ? 1024 : (hidden >= 2048 ? 512 : (hidden >= 1024 ? 256 : 128));
  return launch_kernel("add_rmsnorm", add_rmsnorm_kernel<T>, dim3(out_rows), dim3(threads), smem, as_stream(stream),
                       (T*)y, residual_out, residual_in, (const T*)x, w, rows, hidden, eps, vec_ok);
}

template <typename T>
int silu_mul(void* out, const void* gu, int tokens, int inter, void* stream) {
  PTL_REQUIRE(tokens >= 0 && inter > 0, "silu_mul: bad sizes tokens=%d inter=%d", tokens, inter);
  PTL_REQUIRE(tokens <= 65535, "silu_mul: at most 65535 rows per call, got %d", tokens);
  if (tokens == 0) return 0;
  constexpr int VN = Vec16<T>::N;
  const int vec_ok = (inter % VN == 0) && aligned16(out) && aligned16(gu);
  const int threads = 256;
  dim3 grid((inter + threads * VN - 1) / (threads * VN), tokens);
  return launch_kernel("silu_mul", silu_mul_kernel<T>, grid, dim3(threads), 0, as_stream(stream), (T*)out, (const T*)gu,
                       inter, vec_ok);
}

}  // namespace ptl

namespace ptl {

// y[t, :] = xs[t, :] * rsqrt(sum of the token's `slots` partial sums of squares / width + eps): finishes an RMS norm
// whose input a product's epilogue prepared (xs = bfloat16(residual * weight)), for a reader that cannot apply
// the row scale itself.  One block per token.
__global__ void __launch_bounds__(256)
finish_norm_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ xs, const float* __restrict__ sumsq,
                   int slots, int sumsq_ld, int width, float eps) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  float sum = 0.f;
  for (int k = threadIdx.x; k < slots; k += blockDim.x) sum += __ldcg(sumsq + (size_t)t * sumsq_ld + k);
  sum = block_sum(sum, red);
  const float scale = rsqrtf(sum / (float)width + eps);
  const __nv_bfloat16* src = xs + (size_t)t * width;
  __nv_bfloat16* dst = y + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = __float2bfloat16_rn(__bfloat162float(src[i]) * scale);
}

}  // namespace ptl

PTL_EXPORT int ptl_finish_norm_bf16(void* y, const void* xs, const float* sumsq, int tokens, int slots, int sumsq_ld, int width,
                                    float eps, void* stream) {
  PTL_REQUIRE(tokens >= 0 && slots > 0 && sumsq_ld >= slots && width > 0 && eps > 0.f, "finish_norm: bad sizes tokens=%d slots=%d width=%d", tokens, slots, width);
  if (tokens == 0) return 0;
  return ptl::launch_kernel("finish_norm", ptl::finish_norm_kernel, dim3(tokens), dim3(256), 0, ptl::as_stream(stream),
                            (__nv_bfloat16*)y, (const __nv_bfloat16*)xs, sumsq, slots, sumsq_ld, width, eps);
}

PTL_EXPORT int ptl_take_tokens(int* tokens, const int* src, const int* sampled, int n, int n_sampled, void* stream) {
  PTL_REQUIRE(n >= 0 && n_sampled >= 0, "take_tokens: bad sizes n=%d sampled=%d", n, n_sampled);
  if (n == 0) return 0;
  return ptl::launch_kernel("take_tokens", ptl::take_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0,
                            ptl::as_stream(stream), tokens, src, sampled, n, n_sampled);
}

PTL_EXPORT int ptl_add_partials(float* acc, const float* parts, int n_parts, long long n, long long stride, void* stream) {
  PTL_REQUIRE(n_parts > 0 && n >= 0 && stride >= n, "add_partials: bad sizes parts=%d n=%lld stride=%lld", n_parts, n, stride);
  PTL_REQUIRE(n % 4 == 0 && stride % 4 == 0 && ptl::aligned16(acc) && ptl::aligned16(parts), "add_partials: sizes must be multiples of 4 values and pointers 16-byte aligned");
  if (n == 0) return 0;
  const size_t n4 = (size_t)n / 4;
  return ptl::launch_kernel("add_partials", ptl::add_partials_kernel, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0,
                            ptl::as_stream(stream), (float4*)acc, (const float4*)parts, n_parts, n4, (size_t)stride / 4);
}

PTL_EXPORT int ptl_embed_gather_f32(void* out, const void* table, const int* ids, int tokens, int hidden, int vocab, int* status, void* stream) {
  return ptl::embed_gather<float>(out, table, ids, tokens, hidden, vocab, status, stream);
}
PTL_EXPORT int ptl_embed_gather_bf16(void* out, const void* table, const int* ids, int tokens, int hidden, int vocab, int* status, void* stream) {
  return ptl::embed_gather<__nv_bfloat16>(out, table, ids, tokens, hidden, vocab, status, stream);
}
PTL_EXPORT int ptl_add_rmsnorm_f32(void* y, float* residual_out, const float* residual_in, const void* x, const float* w, const int* rows, int out_rows, int hidden, float eps, void* stream) {
  return ptl::add_rmsnorm<float>(y, residual_out, residual_in, x, w, rows, out_rows, hidden, eps, stream);
}
PTL_EXPORT int ptl_add_rmsnorm_bf16(void* y, float* residual_out, const float* residual_in, const void* x, const float* w, const int* rows, int out_rows, int hidden, float eps, void* stream) {
  return ptl::add_rmsnorm<__nv_bfloat16>(y, residual_out, residual_in, x, w, rows, out_rows, hidden, eps, stream);
}
PTL_EXPORT int ptl_silu_mul_f32(void* out, const void* gu, int tokens, int inter, void* stream) {
  return ptl::silu_mul<float>(out, gu, tokens, inter, stream);
}
PTL_EXPORT int ptl_silu_mul_bf16(void* out, const void* gu, int tokens, int inter, void* stream) {
  return ptl::silu_mul<__nv_bfloat16>(out, gu, tokens, inter, stream);
}
