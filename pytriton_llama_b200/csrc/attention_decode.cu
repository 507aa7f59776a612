// Decode attention over the paged cache in bfloat16: one block per (single-token request, kv
// head, split of the key range).  All query heads of the group ride in the 16 rows of one
// m16n8k16 tile, so each key and value is fetched from HBM once for the whole group; the kernel
// is a streaming read of the cache.  Four warps share 64-key tiles brought in by a ring of
// cp.async stages (16 keys per warp and tile), keep their own running max / sum / accumulator in
// float32 and are merged through shared memory at the end.  With splits > 1 the partial results of
// a (token, kv head) are combined in one of three ways: up to 8 splits with 128-key tiles form a
// thread-block cluster, every warp sends its partial rows into the shared memory of the block
// that owns the row (distributed shared memory), and after one cluster barrier the owners
// finish them; otherwise the block writes an unnormalised partial result to global memory and
// the block that finishes last combines them (or, without counters, the kernel `attention_merge`
// of attention_simt.cu does).
//
// The token list `items` names the tokens of the step that take this path (nullptr: tokens
// 0..n-1).  Token t of request r = tok_req[t] at position p sees keys max(0, p-window+1)..p;
// r < 0 marks a padding row, which yields zeros.
#include "mma_utils.cuh"

namespace ptl {

constexpr int kDecWarps = 4;

__device__ __forceinline__ float dec_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));   // 0 for -inf; P is rounded to bfloat16 anyway
  return y;
}
constexpr int kDecStagedPages = 512;    // block-table entries of a block's key range kept in shared memory (8,192 keys with pages of 16)

// KP = groups of 16 keys per warp and tile: 1 (64-key tiles, four blocks per SM) for large batches,
// 2 (128-key tiles, two blocks per SM, fewer barriers per key) when few blocks are in flight.
template <int D, int KP> struct DecodeCfg {
  static constexpr int kKeys = 64 * KP;
  // 64-key tiles: three stages (48 KB for D = 64, four blocks per SM).  128-key tiles: two stages, so that
  // two blocks leave room for a block of the product that follows to move in and fetch its weights
  // early (alone the kernel is 2 us slower with two stages, a decode step 2 % faster)
  static constexpr int kStages = KP == 2 ? 2 : 3;
  static constexpr int kChunks = D / 8;                       // 16-byte chunks per row
  static constexpr int kTileBytes = kKeys * D * 2;             // one of K / V
  static constexpr int kSmem = kStages * 2 * kTileBytes;
};

template <int D, int KP>
__global__ void __launch_bounds__(kDecWarps * 32)
decode_attention_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                        const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                        const int* __restrict__ block_table, const int* __restrict__ items,
                        const int* __restrict__ tok_req, const int* __restrict__ positions, int q_stride,
                        int out_stride, int bt_stride, int nq, int nkv, int page_size, float scale_log2,
                        int window, int splits, int num_pages, int page_shift, int* __restrict__ counters,
                        int cluster_merge, int fused, const float* __restrict__ inv_freq,
                        const int* __restrict__ slots, unsigned long long* timeline) {
  using Cfg = DecodeCfg<D, KP>;
  constexpr int kDecKeys = Cfg::kKeys;
  constexpr int kDecKP = KP;
  extern __shared__ __align__(128) unsigned char smem[];
  if (threadIdx.x == 0 && timeline) { timeline_stamp(timeline, 0); if (blockIdx.x == 0) timeline[0] = 1; }
  // with a cluster, peers write into this block's shared memory later on: none may do so before
  // every block runs, which the wait that matches this arrival establishes
  if (cluster_merge) cluster_arrive();
  // Everything up to the wait below reads only what the kernel directly before this one does not
  // write: the step's integers, the block table, and keys and values of earlier positions (the
  // predecessor writes q and the slot of position p).  So it runs under the predecessor's tail.
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int split = blockIdx.x % splits;
  const int kvh = (blockIdx.x / splits) % nkv;
  const int ti = blockIdx.x / (splits * nkv);
  const int t = items ? __ldcg(items + ti) : ti;
  const int G = nq / nkv;
  const int r = __ldcg(tok_req + t);
  const int p = __ldcg(positions + t);
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int nkeys = r < 0 ? 0 : p - lo + 1;
  int chunk_keys = (nkeys + splits - 1) / splits;
  chunk_keys = (chunk_keys + kDecKeys - 1) / kDecKeys * kDecKeys;
  const int k_begin = lo + split * chunk_keys;
  const int k_end = r < 0 ? k_begin : min(k_begin + chunk_keys, p + 1);
  const int ntiles = k_end > k_begin ? (k_end - k_begin + kDecKeys - 1) / kDecKeys : 0;
  const int* bt_global = block_table + (size_t)(r < 0 ? 0 : r) * bt_stride;
  const size_t plane = (size_t)nkv * page_size * D;
  const uint32_t smem_base = smem_u32(smem);

  // ---- the block-table entries of this block's key range go to shared memory once (when they
  // fit), so that the copies of a tile never wait on a global load for their page
  __shared__ int s_pages[kDecStagedPages];
  const int first_block = ntiles > 0 ? k_begin / page_size : 0;
  const int n_blocks = ntiles > 0 ? (k_end - 1) / page_size - first_block + 1 : 0;
  const bool staged = n_blocks <= kDecStagedPages;
  if (staged) {
    for (int i = tid; i < n_blocks; i += kDecWarps * 32) s_pages[i] = __ldcg(bt_global + first_block + i);
    __syncthreads();
  }
  const int* bt = staged ? s_pages - first_block : bt_global;

  // ---- with `fused` the kernel does the work of rope_kv_write for its single tokens itself: q is
  // the unrotated projection; the angles of position p depend on nothing the predecessor writes
  __shared__ float s_cs[D];                                   // cos[D/2], sin[D/2]
  if (fused && inv_freq && tid < D / 2) {
    float sn, cs;
    sincosf((float)p * inv_freq[tid], &sn, &cs);             // as rope_kv_write_kernel does
    s_cs[tid] = cs;
    s_cs[D / 2 + tid] = sn;
  }

  // ---- loader: 64 keys x D of K and of V per tile, 16 bytes per cp.async, zero fill past the range.
  // Thread `tid` always copies chunk tid % kChunks of rows tid / kChunks + i * (128 / kChunks).
  // When pages hold a power-of-two multiple of 16 keys and the range starts on a multiple of 16,
  // each group of 16 consecutive rows lies in one page: one table entry per group, shifts instead
  // of divisions.  Other page sizes take the general path.
  constexpr int kRowsPerPass = kDecWarps * 32 / Cfg::kChunks;       // 16 for D = 64, 8 for D = 128
  constexpr int kPasses = kDecKeys / kRowsPerPass;
  const int my_row = tid / Cfg::kChunks, my_ch = tid % Cfg::kChunks;
  const bool fast_pages = page_shift >= 4 && (k_begin & 15) == 0;
  const size_t my_const = ((size_t)kvh * page_size) * D + my_ch * 8;
  auto load_tile = [&](int tile, int stage) {
    const uint32_t kbase = smem_base + stage * 2 * Cfg::kTileBytes;
    const uint32_t vbase = kbase + Cfg::kTileBytes;
    const int k0 = k_begin + tile * kDecKeys;
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

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  // the first tiles are requested before the wait when none of them holds position p
  const int first_tiles = min(ntiles, Cfg::kStages - 1);
  const bool early = first_tiles > 0 && k_begin + first_tiles * kDecKeys <= p;
  if (early) {
#pragma unroll
    for (int s = 0; s < Cfg::kStages - 1; ++s) {
      if (s < ntiles) load_tile(s, s);
      cp_async_commit();
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  if (tid == 0) timeline_stamp(timeline, 1);
  // With `fused`, the block whose key range ends at position p owns the token's new key and
  // value: it rotates the key, sends both to the cache (for later steps; nothing in this step waits
  // for that) and keeps them in shared memory to put them into its last tile, whose copy from the
  // cache still holds what was in the slot before.
  __shared__ __align__(16) __nv_bfloat16 s_new[2 * D];
  bool owner = fused && slots && r >= 0 && ntiles > 0 && k_end == p + 1;
  if (fused) __syncthreads();                                 // the angles are in place
  if (owner) {
    const int slot = __ldcg(slots + t);                       // the same for every thread of the block
    owner = slot >= 0 && slot < (long long)num_pages * page_size;   // a layer that does not write reads the cache as it is
    if (owner) {
    const bool store = true;
    const __nv_bfloat16* ksrc = q + (size_t)t * q_stride + (size_t)(nq + kvh) * D;
    __nv_bfloat16* kdst = const_cast<__nv_bfloat16*>(cache) + ((size_t)(slot / page_size) * 2) * plane +
                          ((size_t)kvh * page_size + slot % page_size) * D;
    if (tid < D / 2) {
      const float x1 = __bfloat162float(ksrc[tid]), x2 = __bfloat162float(ksrc[tid + D / 2]);
      float o1 = x1, o2 = x2;
      if (inv_freq) rope_rotate(x1, x2, s_cs[tid], s_cs[D / 2 + tid], o1, o2);
      const __nv_bfloat16 b1 = __float2bfloat16_rn(o1), b2 = __float2bfloat16_rn(o2);
      s_new[tid] = b1;
      s_new[tid + D / 2] = b2;
      if (store) { kdst[tid] = b1; kdst[tid + D / 2] = b2; }
    } else if (tid - D / 2 < D / 8) {
      const int ch = tid - D / 2;
      const uint4 v = *reinterpret_cast<const uint4*>(ksrc + (size_t)nkv * D + ch * 8);
      *reinterpret_cast<uint4*>(s_new + D + ch * 8) = v;
      if (store) *reinterpret_cast<uint4*>(kdst + plane + ch * 8) = v;
    }
    }
  }
  // ---- query fragments: row g (and g+8) of the tile is query head kvh*G + g (zero beyond the group)
  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* qrow = q + (size_t)t * q_stride + (size_t)kvh * G * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int col = ks * 16 + 2 * c;
      qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)g * D + col) : 0u;
      qa[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)(g + 8) * D + col) : 0u;
      qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)g * D + col + 8) : 0u;
      qa[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow + (size_t)(g + 8) * D + col + 8) : 0u;
    }
    if (fused && inv_freq) {
      // element pairs (j, j + D/2) lie in the same thread: fragments ks and ks + D/32
      constexpr int KH = D / 32;
#pragma unroll
      for (int ks = 0; ks < KH; ++ks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = ks * 16 + (i >= 2 ? 8 : 0) + 2 * c;
          const float2 a = unpack_bf16(qa[ks][i]), b = unpack_bf16(qa[ks + KH][i]);
          float o1x, o2x, o1y, o2y;
          rope_rotate(a.x, b.x, s_cs[j], s_cs[D / 2 + j], o1x, o2x);
          rope_rotate(a.y, b.y, s_cs[j + 1], s_cs[D / 2 + j + 1], o1y, o2y);
          qa[ks][i] = pack_bf16(o1x, o1y);
          qa[ks + KH][i] = pack_bf16(o2x, o2y);
        }
      }
    }
  }

  if (!early) {
#pragma unroll
    for (int s = 0; s < Cfg::kStages - 1; ++s) {
      if (s < ntiles) load_tile(s, s);
      cp_async_commit();
    }
  }
  for (int tile = 0; tile < ntiles; ++tile) {
    cp_async_wait<Cfg::kStages - 2>();
    __syncthreads();
    if (tile == 0 && tid == 0) timeline_stamp(timeline, 2);
    {
      const int nxt = tile + Cfg::kStages - 1;
      if (nxt < ntiles) load_tile(nxt, nxt % Cfg::kStages);
      cp_async_commit();
    }
    const int stage = tile % Cfg::kStages;
    const uint32_t kbase = smem_base + stage * 2 * Cfg::kTileBytes;
    const uint32_t vbase = kbase + Cfg::kTileBytes;
    if (owner && tile == ntiles - 1) {
      // the token's own key and value take their place in the tile (row p of the range)
      const int prow = p - (k_begin + tile * kDecKeys);
      if (tid < 2 * Cfg::kChunks) {
        const int ch = tid % Cfg::kChunks;
        const uint4 v = *reinterpret_cast<const uint4*>(s_new + (tid / Cfg::kChunks) * D + ch * 8);
        st_shared_16((tid < Cfg::kChunks ? kbase : vbase) + tile_offset<D>(prow, ch), v);
      }
      __syncthreads();
    }
    const int row0 = warp * 16 * kDecKP;                      // this warp's keys of the tile
    // S = Q K^T: two n-tiles of 8 keys per group of 16
    float sc[kDecKP][2][4];
#pragma unroll
    for (int kp = 0; kp < kDecKP; ++kp)
#pragma unroll
      for (int e = 0; e < 4; ++e) { sc[kp][0][e] = 0.f; sc[kp][1][e] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int kp = 0; kp < kDecKP; ++kp) {
        uint32_t kb[4];
        const int id = lane >> 3;
        const int krow = row0 + kp * 16 + (id >> 1) * 8 + (lane & 7);
        ldmatrix_x4(kb, kbase + tile_offset<D>(krow, 2 * ks + (id & 1)));
        mma_bf16_16816(sc[kp][0], qa[ks], kb[0], kb[1]);
        mma_bf16_16816(sc[kp][1], qa[ks], kb[2], kb[3]);
      }
    }
    // mask keys past the range, scale into log2 units
    const int key0 = k_begin + tile * kDecKeys + row0 + 2 * c;
#pragma unroll
    for (int kp = 0; kp < kDecKP; ++kp)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kk0 = key0 + kp * 16 + (e & 1), kk1 = kk0 + 8;
        sc[kp][0][e] = kk0 < k_end ? sc[kp][0][e] * scale_log2 : -INFINITY;
        sc[kp][1][e] = kk1 < k_end ? sc[kp][1][e] * scale_log2 : -INFINITY;
      }
    // online softmax for rows g (e = 0,1) and g+8 (e = 2,3)
    uint32_t pa[kDecKP][4];
#pragma unroll
    for (int kp = 0; kp < kDecKP; ++kp) { pa[kp][0] = pa[kp][1] = pa[kp][2] = pa[kp][3] = 0u; }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (h == 1 && G <= 8) break;          // rows 8..15 of the tile are padding for groups of up to 8 heads
      float mx = -INFINITY;
#pragma unroll
      for (int kp = 0; kp < kDecKP; ++kp)
        mx = fmaxf(mx, fmaxf(fmaxf(sc[kp][0][2 * h], sc[kp][0][2 * h + 1]), fmaxf(sc[kp][1][2 * h], sc[kp][1][2 * h + 1])));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[h], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = dec_exp2(m_run[h] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int kp = 0; kp < kDecKP; ++kp) {
        const float p00 = dec_exp2(sc[kp][0][2 * h] - m_use), p01 = dec_exp2(sc[kp][0][2 * h + 1] - m_use);
        const float p10 = dec_exp2(sc[kp][1][2 * h] - m_use), p11 = dec_exp2(sc[kp][1][2 * h + 1] - m_use);
        sum += p00 + p01 + p10 + p11;
        pa[kp][h] = pack_bf16(p00, p01);          // a0 / a1: keys 2c..2c+1
        pa[kp][2 + h] = pack_bf16(p10, p11);      // a2 / a3: keys 8+2c..
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[h] = l_run[h] * alpha + sum;
      m_run[h] = m_new;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) { o[i][2 * h] *= alpha; o[i][2 * h + 1] *= alpha; }
    }
    // O += P V over this warp's keys
#pragma unroll
    for (int kp = 0; kp < kDecKP; ++kp) {
#pragma unroll
      for (int nt = 0; nt < D / 8; nt += 2) {
        uint32_t vb[4];
        const int id = lane >> 3;
        const int vrow = row0 + kp * 16 + (id & 1) * 8 + (lane & 7);
        ldmatrix_x4_trans(vb, vbase + tile_offset<D>(vrow, nt + (id >> 1)));
        mma_bf16_16816(o[nt], pa[kp], vb[0], vb[1]);
        mma_bf16_16816(o[nt + 1], pa[kp], vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  if (tid == 0) timeline_stamp(timeline, 3);

  if (cluster_merge) {
    // ---- the splits of this (token, kv head) are the blocks of a cluster.  Row r of the group
    // belongs to block r % splits; every warp of every block sends its partial row there:
    // [splits * warps sources][rows owned][D accumulators, max, sum]
    float* recv = reinterpret_cast<float*>(smem + Cfg::kSmem);
    const int rows_own = (G + splits - 1) / splits;
    constexpr int kRow = D + 2;
    cluster_wait();
    const int src = split * kDecWarps + warp;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = g + 8 * h;
      if (row < G) {
        const uint32_t dst = map_to_peer(smem_u32(recv) + 4u * ((src * rows_own + row / splits) * kRow), row % splits);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) st_peer_f32x2(dst + 4u * (i * 8 + 2 * c), o[i][2 * h], o[i][2 * h + 1]);
        if (c == 0) st_peer_f32x2(dst + 4u * D, m_run[h], l_run[h]);
      }
    }
    cluster_arrive();
    cluster_wait();
    if (tid == 0) timeline_stamp(timeline, 4);
    const int nsrc = splits * kDecWarps;
    for (int e = tid; e < rows_own * D; e += kDecWarps * 32) {
      const int rloc = e / D, col = e % D;
      const int row = rloc * splits + split;
      if (row >= G) continue;
      float M = -INFINITY;
      for (int sidx = 0; sidx < nsrc; ++sidx) M = fmaxf(M, recv[(sidx * rows_own + rloc) * kRow + D]);
      float L = 0.f, acc = 0.f;
      for (int sidx = 0; sidx < nsrc; ++sidx) {
        const float* part = recv + (sidx * rows_own + rloc) * kRow;
        const float wgt = part[D] == -INFINITY ? 0.f : dec_exp2(part[D] - M);
        L += wgt * part[D + 1];
        acc += wgt * part[col];
      }
      out[(size_t)t * out_stride + (size_t)(kvh * G + row) * D + col] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
    if (tid == 0) timeline_stamp(timeline, 5);
    return;
  }

  if (r < 0 && splits > 1) {
    // A padding row has no keys.  Its blocks take no ticket below: a captured step may name the
    // same padding row in several items, and more than `splits` blocks on one counter would
    // leave it non-zero for the next call.  The row reads as zeros.
    if (split == 0)
      for (int e = tid; e < G * D; e += kDecWarps * 32)
        out[(size_t)t * out_stride + (size_t)kvh * G * D + e] = __float2bfloat16_rn(0.f);
    return;
  }

  // ---- merge the four warps through shared memory
  float* mo = reinterpret_cast<float*>(smem);                  // [warps][16][D]
  float* mml = mo + kDecWarps * 16 * D;                        // [warps][16][2]
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int col = i * 8 + 2 * c;
    mo[(warp * 16 + g) * D + col] = o[i][0];
    mo[(warp * 16 + g) * D + col + 1] = o[i][1];
    mo[(warp * 16 + g + 8) * D + col] = o[i][2];
    mo[(warp * 16 + g + 8) * D + col + 1] = o[i][3];
  }
  if (c == 0) {
    mml[(warp * 16 + g) * 2] = m_run[0];
    mml[(warp * 16 + g) * 2 + 1] = l_run[0];
    mml[(warp * 16 + g + 8) * 2] = m_run[1];
    mml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  for (int e = tid; e < G * D; e += kDecWarps * 32) {
    const int row = e / D, col = e % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, mml[(w * 16 + row) * 2]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = mml[(w * 16 + row) * 2];
      const float wgt = mw == -INFINITY ? 0.f : dec_exp2(mw - M);
      L += wgt * mml[(w * 16 + row) * 2 + 1];
      acc += wgt * mo[(w * 16 + row) * D + col];
    }
    const int h = kvh * G + row;
    if (splits == 1) {
      out[(size_t)t * out_stride + (size_t)h * D + col] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      const size_t idx = ((size_t)t * nq + h) * splits + split;
      part_acc[idx * D + col] = acc;
      if (col == 0) {
        part_ml[idx * 2] = M == -INFINITY ? -INFINITY : M * 0.6931471805599453f;   // natural-log units for the merge
        part_ml[idx * 2 + 1] = L;
      }
    }
  }
  if (splits == 1 || counters == nullptr) return;   // one split is final; without counters a second kernel merges

  // ---- the block that finishes last among the splits of this (token, kv head) merges them.
  // Nobody waits: every block publishes its partial result, then takes a ticket.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(counters + (size_t)t * nkv + kvh, 1);
    s_last = ticket == splits - 1;
    if (s_last) counters[(size_t)t * nkv + kvh] = 0;          // ready for the next call
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // partial results of the group's heads are contiguous: [G][splits][D] and [G][splits][2]
  const size_t idx0 = ((size_t)t * nq + (size_t)kvh * G) * splits;
  float* w = reinterpret_cast<float*>(smem);                   // [G][splits] maxima m, then weights e^{m - M}
  float* lz = w + G * splits;                                  // [G][splits] sums l
  float* inv_l = lz + G * splits;                              // [G]
  float4* red = reinterpret_cast<float4*>(smem + (((size_t)(2 * G * splits + 16) * 4 + 15) & ~(size_t)15));   // [z lanes][units of a pass]
  constexpr int kD4 = D / 4;
  const int units = G * kD4;                                   // (head, 4 dimensions)
  const int zlanes = units >= kDecWarps * 32 ? 1 : (kDecWarps * 32) / units;
  const int per_pass = (kDecWarps * 32) / zlanes;
  const int ul = tid % per_pass, zl = tid / per_pass;
  // every load of the merge that needs no weight is issued before anything is computed: the
  // maxima and sums, and this thread's first partial accumulators (one round trip to L2, not several)
  constexpr int kAhead = 4;
  float4 ahead[kAhead];
  {
    const int gh = ul / kD4, d4 = ul % kD4;
    const float4* src = reinterpret_cast<const float4*>(part_acc + (idx0 + (size_t)gh * splits) * D) + d4;
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      const int z = zl + i * zlanes;
      ahead[i] = (ul < units && zl < zlanes && z < splits) ? __ldcg(src + (size_t)z * kD4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  for (int e = tid; e < G * splits; e += kDecWarps * 32) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (idx0 + e) * 2));
    w[e] = ml.x;
    lz[e] = ml.y;
  }
  __syncthreads();
  if (tid < G) {
    float M = -INFINITY;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, w[tid * splits + z]);
    float L = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = w[tid * splits + z];
      const float wz = mz == -INFINITY ? 0.f : expf(mz - M);
      L += wz * lz[tid * splits + z];
      w[tid * splits + z] = wz;
    }
    inv_l[tid] = L > 0.f ? 1.0f / L : 0.f;
  }
  __syncthreads();
  for (int u0 = 0; u0 < units; u0 += per_pass) {
    const int u = u0 + ul;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (u < units && zl < zlanes) {
      const int gh = u / kD4, d4 = u % kD4;
      const float4* src = reinterpret_cast<const float4*>(part_acc + (idx0 + (size_t)gh * splits) * D) + d4;
      int z = zl;
      if (u0 == 0) {
#pragma unroll
        for (int i = 0; i < kAhead; ++i, z += zlanes) {
          if (z >= splits) break;
          const float wz = w[gh * splits + z];
          a.x = fmaf(wz, ahead[i].x, a.x); a.y = fmaf(wz, ahead[i].y, a.y); a.z = fmaf(wz, ahead[i].z, a.z); a.w = fmaf(wz, ahead[i].w, a.w);
        }
      }
#pragma unroll 8
      for (; z < splits; z += zlanes) {
        const float wz = w[gh * splits + z];
        const float4 v = __ldcg(src + (size_t)z * kD4);
        a.x = fmaf(wz, v.x, a.x); a.y = fmaf(wz, v.y, a.y); a.z = fmaf(wz, v.z, a.z); a.w = fmaf(wz, v.w, a.w);
      }
    }
    if (zl < zlanes) red[zl * per_pass + ul] = a;
    __syncthreads();
    if (zl == 0 && u < units) {
      for (int z = 1; z < zlanes; ++z) {
        const float4 b = red[z * per_pass + ul];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      const int gh = u / kD4, d4 = u % kD4;
      const float il = inv_l[gh];
      __nv_bfloat16* dst = out + (size_t)t * out_stride + (size_t)(kvh * G + gh) * D + d4 * 4;
      uint2 pk;
      pk.x = pack_bf16(a.x * il, a.y * il);
      pk.y = pack_bf16(a.z * il, a.w * il);
      *reinterpret_cast<uint2*>(dst) = pk;
    }
    __syncthreads();
  }
}

// defined in attention_simt.cu
int attention_merge_bf16(void* out, const float* part_acc, const float* part_ml, int tokens, int out_stride,
                         int nq, int d, int splits, const int* items, void* stream);

template <int D, int KP>
int launch_decode(void* out, float* part_acc, float* part_ml, const void* q, const void* cache,
                  const int* block_table, const int* items, const int* tok_req, const int* positions, int n_items,
                  int q_stride, int out_stride, int bt_stride, int nq, int nkv, int page_size, float scale,
                  int window, int splits, int num_pages, int* counters, void* stream, int fused,
                  const float* inv_freq, const int* slots) {
  using Cfg = DecodeCfg<D, KP>;
  static SmemRaised raised = {};                         // level 1: the ring; 2: the ring and the rows a cluster exchanges
  if (int rc = raise_shared_memory("decode_attention", decode_attention_kernel<D, KP>, Cfg::kSmem, raised, 1)) return rc;
  int page_shift = -1;                                   // log2(page_size) when it is a power of two
  for (int b = 0; b < 20; ++b) if ((1 << b) == page_size) page_shift = b;
  const long long blocks = (long long)n_items * nkv * splits;
  PTL_REQUIRE(blocks <= 0x7fffffffLL, "decode_attention: too many blocks");
  // a cluster per (token, kv head) when its splits fit one and the rows they exchange are small
  const int G = nq / nkv;
  const size_t recv_bytes = (size_t)splits * kDecWarps * ((G + splits - 1) / splits) * (D + 2) * sizeof(float);
  const bool cluster = KP == 2 && splits >= 2 && splits <= 8 && recv_bytes <= 16 * 1024;
  if (cluster)
    if (int rc = raise_shared_memory("decode_attention", decode_attention_kernel<D, KP>, Cfg::kSmem + 16 * 1024, raised, 2)) return rc;
  int rc = launch_kernel_cluster("decode_attention", decode_attention_kernel<D, KP>, dim3((unsigned)blocks), dim3(kDecWarps * 32),
                                 Cfg::kSmem + (cluster ? recv_bytes : 0), as_stream(stream), cluster ? splits : 1,
                                 (__nv_bfloat16*)out, part_acc, part_ml, (const __nv_bfloat16*)q,
                                 (const __nv_bfloat16*)cache, block_table, items, tok_req, positions, q_stride, out_stride, bt_stride,
                                 nq, nkv, page_size, scale * 1.4426950408889634f, window, splits, num_pages, page_shift, counters,
                                 cluster ? 1 : 0, fused, inv_freq, slots, timeline_slot());
  if (rc) return rc;
  if (cluster) return 0;
  if (splits > 1 && counters == nullptr)
    rc = attention_merge_bf16(out, part_acc, part_ml, n_items, out_stride, nq, D, splits, items, stream);
  return rc;
}

}  // namespace ptl

namespace ptl {

static int decode_attention_entry(void* out, float* part_acc, float* part_ml, const void* q, const void* cache,
                                  const int* block_table, const int* items, const int* tok_req, const int* positions,
                                  int n_items, int q_stride, int out_stride, int bt_stride, int nq, int nkv, int d,
                                  int page_size, float scale, int window, int splits, int num_pages, int* counters,
                                  void* stream, int fused, const float* inv_freq, const int* slots) {
  PTL_REQUIRE(n_items >= 0 && nq > 0 && nkv > 0 && page_size > 0 && num_pages > 0, "decode_attention: bad sizes");
  PTL_REQUIRE(nq % nkv == 0, "decode_attention: %d query heads are no multiple of %d kv heads", nq, nkv);
  if ((d != 64 && d != 128) || nq / nkv > 16) return -2;
  PTL_REQUIRE(splits >= 1 && (splits == 1 || (part_acc && part_ml)), "decode_attention: splits > 1 need scratch buffers");
  PTL_REQUIRE(counters == nullptr || splits <= 512, "decode_attention: at most 512 splits with in-kernel merging");
  PTL_REQUIRE(aligned16(q) && aligned16(cache) && q_stride % 8 == 0, "decode_attention: q and cache must be 16-byte aligned");
  PTL_REQUIRE(!fused || q_stride >= (nq + 2 * nkv) * d, "decode_attention: the fused form needs the whole q|k|v row, %d < %d", q_stride, (nq + 2 * nkv) * d);
  if (n_items == 0) return 0;
  // the in-kernel merge keeps a maximum and a sum per (head of the group, split) in shared memory
  if ((long long)(nq / nkv) * splits > 4096) counters = nullptr;
  // few blocks in flight: 128-key tiles; many: 64-key tiles and twice the blocks per SM
  const bool wide = (long long)n_items * nkv * splits <= 296;
#define PTL_DECODE_ARGS out, part_acc, part_ml, q, cache, block_table, items, tok_req, positions, n_items, q_stride, \
                        out_stride, bt_stride, nq, nkv, page_size, scale, window, splits, num_pages, counters, stream, \
                        fused, inv_freq, slots
  if (d == 64) return wide ? launch_decode<64, 2>(PTL_DECODE_ARGS) : launch_decode<64, 1>(PTL_DECODE_ARGS);
  return wide ? launch_decode<128, 2>(PTL_DECODE_ARGS) : launch_decode<128, 1>(PTL_DECODE_ARGS);
#undef PTL_DECODE_ARGS
}

}  // namespace ptl

// Returns 0 on success; -2 if this kernel does not take the sizes (the caller then uses the
// CUDA-core kernel); -1 on an error.  `counters` (one zeroed int per (token row, kv head), left
// zeroed again) lets the last block of a token's splits merge them inside the kernel; with
// nullptr a second kernel does the merge.  Splits are limited to 512 with counters.
PTL_EXPORT int ptl_decode_attention_bf16(void* out, float* part_acc, float* part_ml, const void* q, const void* cache,
                                         const int* block_table, const int* items, const int* tok_req,
                                         const int* positions, int n_items, int q_stride, int out_stride,
                                         int bt_stride, int nq, int nkv, int d, int page_size, float scale, int window,
                                         int splits, int num_pages, int* counters, void* stream) {
  return ptl::decode_attention_entry(out, part_acc, part_ml, q, cache, block_table, items, tok_req, positions, n_items,
                                     q_stride, out_stride, bt_stride, nq, nkv, d, page_size, scale, window, splits,
                                     num_pages, counters, stream, 0, nullptr, nullptr);
}

// The same for steps of single tokens only, with the work of ptl_rope_kv_write folded in: `qkv` is
// the unrotated projection [rows, (nq + 2 nkv) d]; every token's q and k are rotated by the angles
// position * inv_freq[j] over the whole head (inv_freq == nullptr: not at all), and its k and v
// are written to cache slot slots[row] before they are read (slots == nullptr or a negative slot:
// not written).  The q part of `qkv` is left as it was.
PTL_EXPORT int ptl_decode_attention_rope_bf16(void* out, float* part_acc, float* part_ml, const void* qkv, void* cache,
                                              const int* block_table, const int* items, const int* tok_req,
                                              const int* positions, int n_items, int q_stride, int out_stride,
                                              int bt_stride, int nq, int nkv, int d, int page_size, float scale,
                                              int window, int splits, int num_pages, int* counters,
                                              const float* inv_freq, const int* slots, void* stream) {
  return ptl::decode_attention_entry(out, part_acc, part_ml, qkv, cache, block_table, items, tok_req, positions, n_items,
                                     q_stride, out_stride, bt_stride, nq, nkv, d, page_size, scale, window, splits,
                                     num_pages, counters, stream, 1, inv_freq, slots);
}
