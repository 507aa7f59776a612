// Attention of prompt portions over the paged cache in bfloat16 (flash-attention style, warp-level
// tensor cores): one block per (tile of up to 64 consecutive query tokens of one request, query
// head); four warps of 16 query rows each walk the request's keys in tiles of 64, brought from
// the pages by a ring of cp.async stages.  A portion that follows a cached prefix simply has
// positions that start later: every query attends over the pages up to its own position, so the
// step's own keys (written to their pages before this kernel runs) and older ones are treated
// alike.  Scores, running max and sum, and the accumulator are float32; P is rounded to bfloat16
// for the second product, as lite_llama's kernel does (lite_llama/kernels/flashattentionv2.py:55).
//
// tiles[i] = {request row, first token index, rows (1..64), position of the first token}.
#include "mma_utils.cuh"

namespace ptl {

constexpr int kPfRows = 64;       // query rows per block
constexpr int kPfKeys = 64;       // keys per tile
constexpr int kPfWarps = 4;

template <int D> struct PrefillCfg {
  static constexpr int kStages = 3;
  static constexpr int kChunks = D / 8;
  static constexpr int kTileBytes = kPfKeys * D * 2;
  static constexpr int kQBytes = kPfRows * D * 2;
  static constexpr int kSmem = kQBytes + kStages * 2 * kTileBytes;
};

template <int D>
__global__ void __launch_bounds__(kPfWarps * 32)
prefill_attention_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q,
                         const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table,
                         const int* __restrict__ tiles, int q_stride, int out_stride, int bt_stride, int nq,
                         int nkv, int page_size, float scale_log2, int window, int num_pages) {
  using Cfg = PrefillCfg<D>;
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int* tl = tiles + 4 * blockIdx.x;
  const int req = tl[0], tok0 = tl[1], rows = tl[2], pos0 = tl[3];
  const int h = blockIdx.y;
  const int kvh = h / (nq / nkv);
  const int k_lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int k_end = pos0 + rows;                 // one past the last key any row of the tile sees
  const int ntiles = (k_end - k_lo + kPfKeys - 1) / kPfKeys;
  const int* bt = block_table + (size_t)req * bt_stride;
  const size_t plane = (size_t)nkv * page_size * D;
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t kv_smem = q_smem + Cfg::kQBytes;

  auto load_tile = [&](int tile, int stage) {
    const uint32_t kbase = kv_smem + stage * 2 * Cfg::kTileBytes;
    const uint32_t vbase = kbase + Cfg::kTileBytes;
#pragma unroll
    for (int i = 0; i < kPfKeys * Cfg::kChunks / (kPfWarps * 32); ++i) {
      const int idx = tid + i * kPfWarps * 32;
      const int row = idx / Cfg::kChunks, ch = idx % Cfg::kChunks;
      const int key = k_lo + tile * kPfKeys + row;
      bool valid = key < k_end;
      int page = valid ? bt[key / page_size] : 0;
      if (page < 0 || page >= num_pages) { valid = false; page = 0; }
      const __nv_bfloat16* src = cache + ((size_t)page * 2) * plane + ((size_t)kvh * page_size + key % page_size) * D + ch * 8;
      const uint32_t off = tile_offset<D>(row, ch);
      cp_async_16(kbase + off, src, valid);
      cp_async_16(vbase + off, src + plane, valid);
    }
  };

  // ---- the query tile goes through shared memory into A fragments (group 0 of the ring)
#pragma unroll
  for (int i = 0; i < kPfRows * Cfg::kChunks / (kPfWarps * 32); ++i) {
    const int idx = tid + i * kPfWarps * 32;
    const int row = idx / Cfg::kChunks, ch = idx % Cfg::kChunks;
    const bool valid = row < rows;
    const __nv_bfloat16* src = q + (size_t)(tok0 + (valid ? row : 0)) * q_stride + (size_t)h * D + ch * 8;
    cp_async_16(q_smem + tile_offset<D>(row, ch), src, valid);
  }
  cp_async_commit();
#pragma unroll
  for (int s = 0; s < Cfg::kStages - 1; ++s) {
    if (s < ntiles) load_tile(s, s);
    cp_async_commit();
  }
  cp_async_wait<Cfg::kStages - 1>();      // the query group is complete
  __syncthreads();
  uint32_t qa[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int id = lane >> 3;
    const int row = warp * 16 + (id & 1) * 8 + (lane & 7);
    ldmatrix_x4(qa[ks], q_smem + tile_offset<D>(row, 2 * ks + (id >> 1)));
  }

  const int qpos0 = pos0 + warp * 16 + g;        // position of row g of this warp; row g+8 is 8 later
  const int warp_qmin = pos0 + warp * 16, warp_qmax = pos0 + warp * 16 + 15;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  for (int tile = 0; tile < ntiles; ++tile) {
    cp_async_wait<Cfg::kStages - 2>();
    __syncthreads();
    {
      const int nxt = tile + Cfg::kStages - 1;
      if (nxt < ntiles) load_tile(nxt, nxt % Cfg::kStages);
      cp_async_commit();
    }
    const int key_first = k_lo + tile * kPfKeys;
    if (key_first > warp_qmax) continue;                       // wholly above this warp's diagonal
    if (window > 0 && key_first + kPfKeys - 1 < warp_qmin - window + 1) continue;   // wholly before its window
    const int stage = tile % Cfg::kStages;
    const uint32_t kbase = kv_smem + stage * 2 * Cfg::kTileBytes;
    const uint32_t vbase = kbase + Cfg::kTileBytes;

    float s[kPfKeys / 8][4];
#pragma unroll
    for (int nt = 0; nt < kPfKeys / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < kPfKeys / 16; ++np) {
        uint32_t kb[4];
        const int id = lane >> 3;
        const int krow = np * 16 + (id >> 1) * 8 + (lane & 7);
        ldmatrix_x4(kb, kbase + tile_offset<D>(krow, 2 * ks + (id & 1)));
        mma_bf16_16816(s[2 * np], qa[ks], kb[0], kb[1]);
        mma_bf16_16816(s[2 * np + 1], qa[ks], kb[2], kb[3]);
      }
    }
    // scale and mask: causal, window, end of range
    const bool need_mask = (key_first + kPfKeys - 1 > warp_qmin) ||
                           (window > 0 && key_first < warp_qmax - window + 1);
#pragma unroll
    for (int nt = 0; nt < kPfKeys / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nt][e] * scale_log2;
        if (need_mask) {
          const int key = key_first + nt * 8 + 2 * c + (e & 1);
          const int qp = qpos0 + (e >> 1) * 8;
          if (key > qp || (window > 0 && key < qp - window + 1)) v = -INFINITY;
        }
        s[nt][e] = v;
      }
    }
    uint32_t pa[kPfKeys / 16][4];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < kPfKeys / 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * hh], s[nt][2 * hh + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hh], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m_run[hh] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < kPfKeys / 8; ++nt) {
        const float p0 = exp2f(s[nt][2 * hh] - m_use), p1 = exp2f(s[nt][2 * hh + 1] - m_use);
        sum += p0 + p1;
        pa[nt >> 1][(nt & 1) * 2 + hh] = pack_bf16(p0, p1);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[hh] = l_run[hh] * alpha + sum;
      m_run[hh] = m_new;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) { o[i][2 * hh] *= alpha; o[i][2 * hh + 1] *= alpha; }
    }
#pragma unroll
    for (int kk = 0; kk < kPfKeys / 16; ++kk) {
#pragma unroll
      for (int nt = 0; nt < D / 8; nt += 2) {
        uint32_t vb[4];
        const int id = lane >> 3;
        const int vrow = kk * 16 + (id & 1) * 8 + (lane & 7);
        ldmatrix_x4_trans(vb, vbase + tile_offset<D>(vrow, nt + (id >> 1)));
        mma_bf16_16816(o[nt], pa[kk], vb[0], vb[1]);
        mma_bf16_16816(o[nt + 1], pa[kk], vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int row = warp * 16 + g + hh * 8;
    if (row >= rows) continue;
    const float inv = l_run[hh] > 0.f ? 1.0f / l_run[hh] : 0.f;
    __nv_bfloat16* dst = out + (size_t)(tok0 + row) * out_stride + (size_t)h * D + 2 * c;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2 * hh] * inv, o[i][2 * hh + 1] * inv);
    }
  }
}

template <int D>
int launch_prefill(void* out, const void* q, const void* cache, const int* block_table, const int* tiles, int n_tiles,
                   int q_stride, int out_stride, int bt_stride, int nq, int nkv, int page_size, float scale,
                   int window, int num_pages, void* stream) {
  using Cfg = PrefillCfg<D>;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    PTL_REQUIRE(e == cudaSuccess, "prefill_attention: cannot raise shared memory: %s", cudaGetErrorString(e));
    raised = true;
  }
  PTL_REQUIRE(nq <= 65535, "prefill_attention: at most 65535 query heads");
  dim3 grid(n_tiles, nq);
  return launch_kernel("prefill_attention", prefill_attention_kernel<D>, grid, dim3(kPfWarps * 32), Cfg::kSmem,
                       as_stream(stream), (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache,
                       block_table, tiles, q_stride, out_stride, bt_stride, nq, nkv, page_size,
                       scale * 1.4426950408889634f, window, num_pages);
}

}  // namespace ptl

// Returns 0 on success; -2 if this kernel does not take the sizes; -1 on an error.
PTL_EXPORT int ptl_prefill_attention_bf16(void* out, const void* q, const void* cache, const int* block_table,
                                          const int* tiles, int n_tiles, int q_stride, int out_stride, int bt_stride,
                                          int nq, int nkv, int d, int page_size, float scale, int window,
                                          int num_pages, void* stream) {
  using namespace ptl;
  PTL_REQUIRE(n_tiles >= 0 && nq > 0 && nkv > 0 && page_size > 0 && num_pages > 0, "prefill_attention: bad sizes");
  PTL_REQUIRE(nq % nkv == 0, "prefill_attention: %d query heads are no multiple of %d kv heads", nq, nkv);
  if (d != 64 && d != 128) return -2;
  PTL_REQUIRE(aligned16(q) && aligned16(cache) && aligned16(out) && q_stride % 8 == 0 && out_stride % 2 == 0,
              "prefill_attention: q, cache and out must be 16-byte aligned");
  if (n_tiles == 0) return 0;
  if (d == 64)
    return launch_prefill<64>(out, q, cache, block_table, tiles, n_tiles, q_stride, out_stride, bt_stride, nq, nkv,
                              page_size, scale, window, num_pages, stream);
  return launch_prefill<128>(out, q, cache, block_table, tiles, n_tiles, q_stride, out_stride, bt_stride, nq, nkv,
                             page_size, scale, window, num_pages, stream);
}
