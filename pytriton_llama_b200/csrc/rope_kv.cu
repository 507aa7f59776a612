// Rotary position encoding of q and k, fused with the write of k and v into the paged cache.
//
// qkv is the projection output of one step, [tokens, (nq + 2*nkv) * d]: q heads, then k heads,
// then v heads, head-major with d contiguous.  For token t at position p and frequency index j
// the angle is float(p) * inv_freq[j] in float32; the pair (x[j], x[j + rot/2]) of a head turns
// into (x1*cos - x2*sin, x2*cos + x1*sin).  q is rewritten in place; rotated k and plain v go to
// cache slot `slots[t]` (page = slot / page_size, offset = slot % page_size; a negative slot
// skips the write).  Cache layout of one layer: [pages][2 (k,v)][nkv][page_size][d].
// inv_freq == nullptr leaves q and k unrotated (a mixer with another position encoding).
#include "common.cuh"

namespace ptl {

template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; };

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                     T* __restrict__ cache, int nq, int nkv, int d, int rot,
                                     int page_size, int write_cache, long long num_slots, int vec2_ok) {
  extern __shared__ float cs[];            // cos[rot/2], sin[rot/2] of this token's angles
  // positions, slots and frequencies are inputs of the step, not results of the kernel before this
  // one: the angles are worked out while that kernel still runs
  const int t = blockIdx.x;
  const int row_len = (nq + 2 * nkv) * d;
  T* row = qkv + (size_t)t * row_len;
  const float pos = (float)__ldcg(positions + t);
  int slot = write_cache ? __ldcg(slots + t) : -1;
  if (slot >= num_slots) slot = -1;  // never write outside the pool
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot % page_size : 0;
  const size_t plane = (size_t)nkv * page_size * d;         // one of k / v inside a page
  T* kdst = cache ? cache + ((size_t)page * 2) * plane + (size_t)off * d : nullptr;
  T* vdst = cache ? kdst + plane : nullptr;
  const int half = rot / 2;
  if (inv_freq) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float s, c;
      sincosf(pos * inv_freq[j], &s, &c);   // the accurate version: angles reach thousands of radians
      cs[j] = c;
      cs[half + j] = s;
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  const int pairs_per_head = d - half;  // `half` rotated pairs, then d - rot pass-through elements
  if (vec2_ok) {
    // two neighbouring frequencies per thread: 4-byte (bfloat16) or 8-byte (float32) accesses
    using V2 = typename Pair<T>::type;
    const int half2 = half / 2;
    for (int e = threadIdx.x; e < (nq + nkv) * half2; e += blockDim.x) {
      const int h = e / half2;
      const int j = (e % half2) * 2;
      T* head = row + (size_t)h * d;
      const V2 a = *reinterpret_cast<const V2*>(head + j), b = *reinterpret_cast<const V2*>(head + j + half);
      float x1a = to_f32(a.x), x1b = to_f32(a.y), x2a = to_f32(b.x), x2b = to_f32(b.y);
      float o1a = x1a, o1b = x1b, o2a = x2a, o2b = x2b;
      if (inv_freq) {
        const float ca = cs[j], cb = cs[j + 1], sa = cs[half + j], sb = cs[half + j + 1];
        rope_rotate(x1a, x2a, ca, sa, o1a, o2a);
        rope_rotate(x1b, x2b, cb, sb, o1b, o2b);
      }
      V2 r1, r2;
      r1.x = from_f32<T>(o1a); r1.y = from_f32<T>(o1b);
      r2.x = from_f32<T>(o2a); r2.y = from_f32<T>(o2b);
      *reinterpret_cast<V2*>(head + j) = r1;
      *reinterpret_cast<V2*>(head + j + half) = r2;
      if (h >= nq && slot >= 0) {
        T* kd = kdst + (size_t)(h - nq) * page_size * d;
        *reinterpret_cast<V2*>(kd + j) = r1;
        *reinterpret_cast<V2*>(kd + j + half) = r2;
      }
    }
    if (slot >= 0 && vdst) {
      // values: 16-byte packets
      constexpr int VN = Vec16<T>::N;
      const T* vsrc = row + (size_t)(nq + nkv) * d;
      for (int e = threadIdx.x * VN; e < nkv * d; e += blockDim.x * VN) {
        const int h = e / d, i = e % d;
        store16(vdst + (size_t)h * page_size * d + i, load16(vsrc + e));
      }
    }
    return;
  }
  // q and k heads
  for (int e = threadIdx.x; e < (nq + nkv) * pairs_per_head; e += blockDim.x) {
    const int h = e / pairs_per_head;
    const int j = e % pairs_per_head;
    T* head = row + (size_t)h * d;
    const bool is_k = h >= nq;
    T* kd = (is_k && slot >= 0) ? kdst + (size_t)(h - nq) * page_size * d : nullptr;
    if (j < half) {
      const float x1 = to_f32(head[j]), x2 = to_f32(head[j + half]);
      float o1 = x1, o2 = x2;
      if (inv_freq) {
        rope_rotate(x1, x2, cs[j], cs[half + j], o1, o2);
      }
      const T r1 = from_f32<T>(o1), r2 = from_f32<T>(o2);
      head[j] = r1;
      head[j + half] = r2;
      if (kd) { kd[j] = r1; kd[j + half] = r2; }
    } else {
      const int i = rot + (j - half);  // untouched tail when rot < d
      if (kd) kd[i] = head[i];
    }
  }
  // v heads
  if (slot >= 0 && vdst) {
    const T* vsrc = row + (size_t)(nq + nkv) * d;
    for (int e = threadIdx.x; e < nkv * d; e += blockDim.x) {
      const int h = e / d, i = e % d;
      vdst[(size_t)h * page_size * d + i] = vsrc[e];
    }
  }
}

// The same for whole heads rotated (rot == d) and rows of whole 16-byte packets: four tokens per
// block, every access a 16-byte packet (a thread takes 4 or 8 neighbouring frequencies of a head:
// the packet at j and the one at j + d/2; or a packet of v on its way to the cache).  Steps of many
// tokens are bound by the memory here: 4-byte accesses left a third of its rate unused.
constexpr int kRopeTokensPerBlock = 4;
#ifndef PTL_ROPE_PACKET_TOKENS
#define PTL_ROPE_PACKET_TOKENS 64
#endif
constexpr int kRopePacketTokens = PTL_ROPE_PACKET_TOKENS;   // steps of at least this many tokens take the packet kernel

template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_write_packets_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                             const int* __restrict__ slots, T* __restrict__ cache, int tokens, int nq, int nkv, int d,
                             int page_size, int write_cache, long long num_slots) {
  extern __shared__ float cs[];            // per token of the block: cos[d/2], sin[d/2]
  __shared__ int s_slot[kRopeTokensPerBlock];
  constexpr int N = Vec16<T>::N;
  const int half = d / 2;
  const int t0 = blockIdx.x * kRopeTokensPerBlock;
  // positions, slots and frequencies are inputs of the step, not results of the kernel before this one
  if (threadIdx.x < kRopeTokensPerBlock) {
    const int t = t0 + threadIdx.x;
    int slot = (write_cache && t < tokens) ? __ldcg(slots + t) : -1;
    if (slot >= num_slots) slot = -1;      // never write outside the pool
    s_slot[threadIdx.x] = slot;
  }
  if (inv_freq) {
    for (int e = threadIdx.x; e < kRopeTokensPerBlock * half; e += blockDim.x) {
      const int tt = e / half, j = e % half;
      if (t0 + tt < tokens) {
        float sn, c;
        sincosf((float)__ldcg(positions + t0 + tt) * inv_freq[j], &sn, &c);   // the accurate version: angles reach thousands of radians
        cs[tt * d + j] = c;
        cs[tt * d + half + j] = sn;
      }
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  const int row_len = (nq + 2 * nkv) * d;
  const int chunks = half / N;                               // packets per half head
  const int rot_items = (nq + nkv) * chunks, v_items = nkv * (d / N);
  const int per_token = rot_items + v_items;
  const size_t plane = (size_t)nkv * page_size * d;          // one of k / v inside a page
  for (int e = threadIdx.x; e < kRopeTokensPerBlock * per_token; e += blockDim.x) {
    const int tt = e / per_token, r = e % per_token, t = t0 + tt;
    if (t >= tokens) break;
    T* row = qkv + (size_t)t * row_len;
    const int slot = s_slot[tt];
    T* kdst = slot >= 0 ? cache + ((size_t)(slot / page_size) * 2) * plane + (size_t)(slot % page_size) * d : nullptr;
    if (r < rot_items) {
      const int h = r / chunks, j = (r % chunks) * N;
      T* head = row + (size_t)h * d;
      Vec16<T> a = load16(head + j), b = load16(head + j + half);
      if (inv_freq) {
        const float* c = cs + tt * d + j;
        const float* sn = c + half;
#pragma unroll
        for (int i = 0; i < N; ++i) {
          float o1, o2;
          rope_rotate(a.get(i), b.get(i), c[i], sn[i], o1, o2);
          a.set(i, o1);
          b.set(i, o2);
        }
      }
      store16(head + j, a);
      store16(head + j + half, b);
      if (h >= nq && kdst) {
        T* kd = kdst + (size_t)(h - nq) * page_size * d;
        store16(kd + j, a);
        store16(kd + j + half, b);
      }
    } else if (kdst) {
      const int rv = r - rot_items, h = rv / (d / N), i = (rv % (d / N)) * N;
      store16(kdst + plane + (size_t)h * page_size * d + i, load16(row + (size_t)(nq + nkv + h) * d + i));
    }
  }
}

// (cos, sin) of angle float(position) * inv_freq[j] for every token and frequency, for kernels that
// rotate without working the angles out themselves: table [tokens, half].
__global__ void rope_table_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int tokens, int half) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= tokens * half) return;
  const float pos = (float)positions[i / half];
  float s, c;
  sincosf(pos * inv_freq[i % half], &s, &c);
  table[i] = make_float2(c, s);
}

template <typename T>
int rope_kv_write(void* qkv, const int* positions, const float* inv_freq, const int* slots, void* cache,
                  int tokens, int nq, int nkv, int d, int rot, int page_size, long long num_slots,
                  void* stream) {
  PTL_REQUIRE(tokens >= 0 && nq > 0 && nkv > 0 && d > 0, "rope_kv_write: bad sizes");
  PTL_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "rope_kv_write: rotary width %d must be even and <= head size %d", rot, d);
  PTL_REQUIRE(cache == nullptr || (page_size > 0 && slots != nullptr && num_slots > 0), "rope_kv_write: a cache needs slots and a page size");
  if (tokens == 0) return 0;
  // the paired path needs the whole head rotated, whole 16-byte packets per head and aligned rows
  const int vec2_ok = rot == d && d % 16 == 0 && aligned16(qkv) && (cache == nullptr || aligned16(cache)) &&
                      ((size_t)(nq + 2 * nkv) * d * sizeof(T)) % 16 == 0;
  // many tokens: four per block and 16-byte packets throughout
  if (vec2_ok && tokens >= kRopePacketTokens && (d / 2) % Vec16<T>::N == 0 && (size_t)kRopeTokensPerBlock * d * sizeof(float) <= 40 * 1024)
    return launch_kernel("rope_kv_write", rope_kv_write_packets_kernel<T>, dim3((tokens + kRopeTokensPerBlock - 1) / kRopeTokensPerBlock),
                         dim3(256), (size_t)kRopeTokensPerBlock * d * sizeof(float), as_stream(stream), (T*)qkv, positions, inv_freq,
                         slots, (T*)cache, tokens, nq, nkv, d, page_size, (int)(cache != nullptr), num_slots);
  const int work = vec2_ok ? (nq + nkv) * (d / 4) : (nq + nkv) * (d - rot / 2);
  const int threads = work >= 2048 ? 256 : 128;
  return launch_kernel("rope_kv_write", rope_kv_write_kernel<T>, dim3(tokens), dim3(threads), (size_t)rot * sizeof(float),
                       as_stream(stream), (T*)qkv, positions, inv_freq, slots, (T*)cache, nq, nkv, d, rot, page_size,
                       (int)(cache != nullptr), num_slots, vec2_ok);
}

}  // namespace ptl

PTL_EXPORT int ptl_rope_table(void* table, const int* positions, const float* inv_freq, int tokens, int half, void* stream) {
  PTL_REQUIRE(tokens >= 0 && half > 0 && table && positions && inv_freq, "rope_table: bad arguments");
  if (tokens == 0) return 0;
  const int n = tokens * half;
  return ptl::launch_kernel("rope_table", ptl::rope_table_kernel, dim3((n + 255) / 256), dim3(256), 0, ptl::as_stream(stream),
                            (float2*)table, positions, inv_freq, tokens, half);
}

PTL_EXPORT int ptl_rope_kv_write_f32(void* qkv, const int* positions, const float* inv_freq, const int* slots, void* cache, int tokens, int nq, int nkv, int d, int rot, int page_size, long long num_slots, void* stream) {
  return ptl::rope_kv_write<float>(qkv, positions, inv_freq, slots, cache, tokens, nq, nkv, d, rot, page_size, num_slots, stream);
}
PTL_EXPORT int ptl_rope_kv_write_bf16(void* qkv, const int* positions, const float* inv_freq, const int* slots, void* cache, int tokens, int nq, int nkv, int d, int rot, int page_size, long long num_slots, void* stream) {
  return ptl::rope_kv_write<__nv_bfloat16>(qkv, positions, inv_freq, slots, cache, tokens, nq, nkv, d, rot, page_size, num_slots, stream);
}
