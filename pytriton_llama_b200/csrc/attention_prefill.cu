// Attention of prompt portions over the paged cache in bfloat16 (flash-attention style, warp-level
// tensor cores): one block per (tile of up to 128 consecutive query tokens of one request, query
// head); its warps (32 query rows each for head size 64, 16 for 128) walk the request's keys in
// tiles of 64, brought from the pages by a ring of cp.async stages; every key and value fragment
// read from shared memory serves all row tiles of the warp.  A portion that follows a cached prefix simply has
// positions that start later: every query attends over the pages up to its own position, so the
// step's own keys (written to their pages before this kernel runs) and older ones are treated
// alike.  Scores, running max and sum, and the accumulator are float32; P is rounded to bfloat16
// for the second product, as lite_llama's kernel does (lite_llama/kernels/flashattentionv2.py:55).
//
// tiles[i] = {request row, first token index, rows (0..128; 0: nothing to do), position of the first token}.
#include "mma_utils.cuh"

namespace ptl {

#ifndef PTL_PF_MT
#define PTL_PF_MT 2
#endif
constexpr int kPfRows = 128;      // query rows per block
constexpr int kPfKeys = 64;       // keys per tile
constexpr int kPfStagedPages = 1024;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));   // exact 0 for -inf; P is rounded to bfloat16 anyway
  return y;
}

// MT = 16-row tiles per warp: 2 for head size 64 (4 warps), 1 for 128 (8 warps).
template <int D, int MT> struct PrefillCfg {
  static constexpr int kWarps = kPfRows / (16 * MT);
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kStages = 3;
  static constexpr int kChunks = D / 8;
  static constexpr int kTileBytes = kPfKeys * D * 2;
  static constexpr int kQBytes = kPfRows * D * 2;
  static constexpr int kSmem = kQBytes + kStages * 2 * kTileBytes;
};

template <int D, int MT>
__global__ void __launch_bounds__(PrefillCfg<D, MT>::kThreads)
prefill_attention_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q,
                         const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table,
                         const int* __restrict__ tiles, int q_stride, int out_stride, int bt_stride, int nq,
                         int nkv, int page_size, float scale_log2, int window, int num_pages, int page_shift) {
  using Cfg = PrefillCfg<D, MT>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_pages[kPfStagedPages];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int* tl = tiles + 4 * (gridDim.x - 1 - blockIdx.x);   // later tiles see more keys: start them first
  const int req = tl[0], tok0 = tl[1], rows = tl[2], pos0 = tl[3];
  if (rows <= 0) return;                          // an empty second half of a pair of tiles
  const int h = blockIdx.y;
  const int kvh = h / (nq / nkv);
  const int k_lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int k_end = pos0 + rows;                 // one past the last key any row of the tile sees
  const int ntiles = (k_end - k_lo + kPfKeys - 1) / kPfKeys;
  const int* bt_global = block_table + (size_t)req * bt_stride;
  const size_t plane = (size_t)nkv * page_size * D;
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t kv_smem = q_smem + Cfg::kQBytes;

  // block-table entries of the key range in shared memory (when they fit)
  const int first_block = k_lo / page_size;
  const int n_blocks = (k_end - 1) / page_size - first_block + 1;
  const bool staged = n_blocks <= kPfStagedPages;
  if (staged) {
    for (int i = tid; i < n_blocks; i += Cfg::kThreads) s_pages[i] = bt_global[first_block + i];
  }
  const int* bt = staged ? s_pages - first_block : bt_global;

  constexpr int kRowsPerPass = Cfg::kThreads / Cfg::kChunks;
  constexpr int kPasses = kPfKeys / kRowsPerPass;
  const int my_row = tid / Cfg::kChunks, my_ch = tid % Cfg::kChunks;
  const bool fast_pages = page_shift >= 0;
  const size_t my_const = ((size_t)kvh * page_size) * D + my_ch * 8;
  auto load_tile = [&](int tile, int stage) {
    const uint32_t kbase = kv_smem + stage * 2 * Cfg::kTileBytes;
    const uint32_t vbase = kbase + Cfg::kTileBytes;
    const int k0 = k_lo + tile * kPfKeys;
#pragma unroll
    for (int i = 0; i < kPasses; ++i) {
      const int row = my_row + i * kRowsPerPass;
      const int key = k0 + row;
      bool valid = key < k_end;
      int page, off;
      if (fast_pages) {
        page = valid ? bt[key >> page_shift] : 0;
        off = key & (page_size - 1);
      } else {
        page = valid ? bt[key / page_size] : 0;
        off = key % page_size;
      }
      if (page < 0 || page >= num_pages) { valid = false; page = 0; }
      const __nv_bfloat16* src = cache + ((size_t)page * 2) * plane + (size_t)off * D + my_const;
      const uint32_t dst = tile_offset<D>(row, my_ch);
      cp_async_16(kbase + dst, src, valid);
      cp_async_16(vbase + dst, src + plane, valid);
    }
  };

  // ---- the query tile goes through shared memory into A fragments (group 0 of the ring)
#pragma unroll
  for (int i = 0; i < kPfRows * Cfg::kChunks / Cfg::kThreads; ++i) {
    const int idx = tid + i * Cfg::kThreads;
    const int row = idx / Cfg::kChunks, ch = idx % Cfg::kChunks;
    const bool valid = row < rows;
    const __nv_bfloat16* src = q + (size_t)(tok0 + (valid ? row : 0)) * q_stride + (size_t)h * D + ch * 8;
    cp_async_16(q_smem + tile_offset<D>(row, ch), src, valid);
  }
  cp_async_commit();
  if (staged) __syncthreads();                    // the staged table is read by load_tile
#pragma unroll
  for (int s = 0; s < Cfg::kStages - 1; ++s) {
    if (s < ntiles) load_tile(s, s);
    cp_async_commit();
  }
  cp_async_wait<Cfg::kStages - 1>();      // the query group is complete
  __syncthreads();
  const int wrow0 = warp * 16 * MT;                // first row of this warp
  uint32_t qa[MT][D / 16][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int id = lane >> 3;
      const int row = wrow0 + mt * 16 + (id & 1) * 8 + (lane & 7);
      ldmatrix_x4(qa[mt][ks], q_smem + tile_offset<D>(row, 2 * ks + (id >> 1)));
    }

  const int warp_qmin = pos0 + wrow0, warp_qmax = pos0 + wrow0 + 16 * MT - 1;
  float m_run[MT][2], l_run[MT][2];
  float o[MT][D / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f; }
  }

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

    float s[MT][kPfKeys / 8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < kPfKeys / 8; ++nt) { s[mt][nt][0] = s[mt][nt][1] = s[mt][nt][2] = s[mt][nt][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < kPfKeys / 16; ++np) {
        uint32_t kb[4];
        const int id = lane >> 3;
        const int krow = np * 16 + (id >> 1) * 8 + (lane & 7);
        ldmatrix_x4(kb, kbase + tile_offset<D>(krow, 2 * ks + (id & 1)));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {                      // each key fragment serves every row tile of the warp
          mma_bf16_16816(s[mt][2 * np], qa[mt][ks], kb[0], kb[1]);
          mma_bf16_16816(s[mt][2 * np + 1], qa[mt][ks], kb[2], kb[3]);
        }
      }
    }
    const bool need_mask = (key_first + kPfKeys - 1 > warp_qmin) ||
                           (window > 0 && key_first < warp_qmax - window + 1);
    uint32_t pa[MT][kPfKeys / 16][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int qpos0 = pos0 + wrow0 + mt * 16 + g;
#pragma unroll
      for (int nt = 0; nt < kPfKeys / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[mt][nt][e] * scale_log2;
          if (need_mask) {
            const int key = key_first + nt * 8 + 2 * c + (e & 1);
            const int qp = qpos0 + (e >> 1) * 8;
            if (key > qp || (window > 0 && key < qp - window + 1)) v = -INFINITY;
          }
          s[mt][nt][e] = v;
        }
      }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < kPfKeys / 8; ++nt) mx = fmaxf(mx, fmaxf(s[mt][nt][2 * hh], s[mt][nt][2 * hh + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[mt][hh], mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = fast_exp2(m_run[mt][hh] - m_use);
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < kPfKeys / 8; ++nt) {
          const float p0 = fast_exp2(s[mt][nt][2 * hh] - m_use), p1 = fast_exp2(s[mt][nt][2 * hh + 1] - m_use);
          sum += p0 + p1;
          pa[mt][nt >> 1][(nt & 1) * 2 + hh] = pack_bf16(p0, p1);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_run[mt][hh] = l_run[mt][hh] * alpha + sum;
        m_run[mt][hh] = m_new;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[mt][i][2 * hh] *= alpha; o[mt][i][2 * hh + 1] *= alpha; }
      }
    }
#pragma unroll
    for (int kk = 0; kk < kPfKeys / 16; ++kk) {
#pragma unroll
      for (int nt = 0; nt < D / 8; nt += 2) {
        uint32_t vb[4];
        const int id = lane >> 3;
        const int vrow = kk * 16 + (id & 1) * 8 + (lane & 7);
        ldmatrix_x4_trans(vb, vbase + tile_offset<D>(vrow, nt + (id >> 1)));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16_16816(o[mt][nt], pa[mt][kk], vb[0], vb[1]);
          mma_bf16_16816(o[mt][nt + 1], pa[mt][kk], vb[2], vb[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int row = wrow0 + mt * 16 + g + hh * 8;
      if (row >= rows) continue;
      const float inv = l_run[mt][hh] > 0.f ? 1.0f / l_run[mt][hh] : 0.f;
      __nv_bfloat16* dst = out + (size_t)(tok0 + row) * out_stride + (size_t)h * D + 2 * c;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[mt][i][2 * hh] * inv, o[mt][i][2 * hh + 1] * inv);
      }
    }
}

template <int D, int MT>
int launch_prefill(void* out, const void* q, const void* cache, const int* block_table, const int* tiles, int n_tiles,
                   int q_stride, int out_stride, int bt_stride, int nq, int nkv, int page_size, float scale,
                   int window, int num_pages, void* stream) {
  using Cfg = PrefillCfg<D, MT>;
  static SmemRaised raised = {};
  if (int rc = raise_shared_memory("prefill_attention", prefill_attention_kernel<D, MT>, Cfg::kSmem, raised)) return rc;
  PTL_REQUIRE(nq <= 65535, "prefill_attention: at most 65535 query heads");
  int page_shift = -1;
  for (int b = 0; b < 20; ++b) if ((1 << b) == page_size) page_shift = b;
  dim3 grid(n_tiles, nq);
  return launch_kernel("prefill_attention", prefill_attention_kernel<D, MT>, grid, dim3(Cfg::kThreads), Cfg::kSmem,
                       as_stream(stream), (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache,
                       block_table, tiles, q_stride, out_stride, bt_stride, nq, nkv, page_size,
                       scale * 1.4426950408889634f, window, num_pages, page_shift);
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
    return launch_prefill<64, PTL_PF_MT>(out, q, cache, block_table, tiles, n_tiles, q_stride, out_stride, bt_stride, nq, nkv,
                                 page_size, scale, window, num_pages, stream);
  return launch_prefill<128, 1>(out, q, cache, block_table, tiles, n_tiles, q_stride, out_stride, bt_stride, nq, nkv,
                                page_size, scale, window, num_pages, stream);
}
