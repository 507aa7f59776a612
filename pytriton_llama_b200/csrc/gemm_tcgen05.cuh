// bfloat16 matrix product on the fifth-generation tensor cores: out = X[M,K] * W[N,K]^T with
// float32 accumulation in tensor memory (TMEM), operands staged by TMA into 128-byte-swizzled
// shared memory, `tcgen05.mma` issued by one thread, accumulators read back with `tcgen05.ld`
// for a fused epilogue.
//
// One block computes one 128 x BN tile.  The 128 rows are the rows of the "row operand", the BN
// columns the rows of the "column operand":
//   * many tokens (M > 64): row operand = X (128 tokens), column operand = W (BN features);
//   * few tokens (M <= 64, decoding): the operands are swapped -- row operand = W (128 features),
//     column operand = X (tokens padded to 16/32/64) -- so the tensor core runs full rows while
//     the kernel is a stream over the weights; the K range is split over the blocks of a thread-block
//     cluster (blockIdx.y = rank in the cluster, up to 8); block z owns the rows z*128/S.. of the
//     tile: every block sends its partial sums of those rows into the owner's shared memory
//     (distributed shared memory stores), and after one cluster barrier the owner adds them up in
//     rank order and runs the epilogue on them.
//
// Epilogues: 0 store bfloat16, 1 store float32, 2 add into a float32 residual [M,N] in place,
// 3 SiLU(gate)*up where the rows of W alternate gate_j, up_j (out is [M, N/2] bfloat16).
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 TMEM allocation + MMA issue (with few tokens
// warps 6..8 issue too), warps 2..9
// epilogue (warp w reads TMEM lanes 32*(w%4)..+31; with many tokens two warps share a lane quarter
// and take half of the columns each).  With many tokens a block walks several tiles and keeps two
// accumulators in TMEM, so the epilogue of one tile runs under the MMAs of the next.  Every wait on an mbarrier gives up after a
// bounded number of polls, records a code in *status, and the block drains and frees its TMEM.
//
// This header holds the kernel template and its launchers; three translation units instantiate it
// (few tokens, many tokens, many tokens on pairs of blocks) so that they compile side by side.
#pragma once
#include "tcgen05_utils.cuh"

namespace ptl {

constexpr int kTileRows = 128;     // rows of the row operand per block (MMA M)
constexpr int kTileK = 64;         // K per stage: 64 bfloat16 = one 128-byte swizzle row
constexpr int kGemmThreads = 320;   // TMA warp, MMA warp, eight epilogue warps (two per TMEM lane quarter)

struct GemmParams {
  void* out;
  int* status;           // set non-zero when a wait gave up
  int rows;              // rows of the row operand (tokens, or features when swapped)
  int cols;              // rows of the column operand
  int K;
  int ld_out;            // elements between tokens in `out`
  int swapped;
  int splits;
  int kb_per_split;
  int tiles_m;           // normal mode: tiles along the tokens and along the features
  int tiles_n;
  // The add epilogue can prepare the RMS norm that follows it (all null otherwise): with r the
  // new residual, xs = bfloat16(r * norm_w) [tokens, xs_ld] and sums of r^2 over slices of the
  // row, sumsq [tokens, sumsq_ld]: a slot per 16 features with few tokens, per half tile with many.
  __nv_bfloat16* xs;
  const float* norm_w;
  float* sumsq;
  int xs_ld;
  int sumsq_ld;
  // A product whose token operand is such an xs finishes the norm: every output row is scaled by
  // rsqrt(sum of the row's scale_slots slots * scale_inv_n + scale_eps) before the epilogue.
  const float* scale_sumsq;
  int scale_slots;
  int scale_ld;
  float scale_eps;
  float scale_inv_n;
  int tma_add;           // many tokens, add epilogue: the accumulator tiles are added into `out` by TMA (map_out)
  int ksplits;           // many tokens, float32 store: the K range is cut into this many parts (work units = tiles x parts),
                         // part s stores its partial sums as rows s * rows.. of `out` ([ksplits, rows, cols])
  // Epilogue 4, the q|k|v projection of a step with many tokens: rotary position encoding of q and k
  // and the write of k and v into the paged cache happen here.  rope_table [tokens, rope_d / 2] holds
  // (cos, sin) of every token's angles; rotated q goes to `out` (bfloat16, the q columns only),
  // rotated k and plain v to cache slot rope_slots[token] (negative: nowhere).
  const float2* rope_table;
  const int* rope_slots;
  __nv_bfloat16* rope_cache;     // [pages][2 (k, v)][rope_nkv][rope_page][rope_d]
  int rope_nq, rope_nkv, rope_d, rope_page;
  long long rope_num_slots;
  // How often a wait on a barrier polls before it gives up (kPollLimit in every product the engine
  // launches).  `withhold_first_load`, set by the self-test entry point alone, makes the block leave
  // out the load of its first stage's token tile, so that the stage never fills: the waits then
  // run out, and the test sees the status word, the drained roles and the block's clean exit.
  uint32_t poll_limit;
  int withhold_first_load;
  unsigned long long* timeline;   // measurements: where the first and the last block stamp %globaltimer (null: nowhere)
  int timeline_kind;
};

// PAIR: two blocks on the SMs of one TPC work as one (cta_group::2): an MMA of 256 token rows x BN
// features, of which each block holds its 128 rows of X, BN/2 rows of W and its 128 rows of the
// accumulator.  A pair fetches W once instead of twice: a third less traffic from L2 into shared
// memory, which is what bounds the many-token product (14-15 TB/s over all SMs).
template <int BN, bool PAIR = false> struct TcCfg {
  static_assert(!PAIR || BN >= 128, "pairs of blocks only with many tokens");
  static constexpr int kStages = PAIR ? 6 : (BN >= 192 ? 4 : (BN >= 128 ? 6 : (BN == 64 ? 3 : 4)));   // few tokens: small blocks, two or three per SM
  static constexpr int kRowBytes = kTileRows * kTileK * 2;     // 16 KB
  static constexpr int kColBytes = (PAIR ? BN / 2 : BN) * kTileK * 2;
  static constexpr int kStageBytes = kRowBytes + kColBytes;
  static constexpr int kAccBufs = BN >= 128 ? 2 : 1;           // many tokens: the epilogue of a tile overlaps the next tile's MMAs
  // few tokens: an MMA of 128 x BN x 16 is short, and one thread that waits for a stage, issues its
  // four MMAs and commits spends about 130 cycles per MMA, most of it on the wait; the tensor core
  // takes 40.  So several warps issue: issuer j takes the stages j, j + ways, ... and has an
  // accumulator of its own, and the epilogue adds the accumulators up.
  // A stage must always be waited for by the same issuer: a wait for the second filling of a
  // stage, made before its first filling has completed, would return at once (only the parity of
  // the phase is compared).  Hence as many issuers as stages, or a divisor of their number.
  static constexpr int kAccWays = BN >= 128 ? 1 : (BN == 64 ? 3 : 4);
  static_assert(kStages % kAccWays == 0, "every stage belongs to one issuer");
  static constexpr int kTmemCols = BN == 192 ? 512 : (BN >= 128 ? BN * kAccBufs : (BN == 64 ? 256 : (BN * kAccWays < 32 ? 32 : BN * kAccWays)));   // power of two >= 32
  static constexpr int kBarBytes = 512;                        // barriers and TMEM slot, then 64 per-token scales
  static constexpr int kPipeSmem = kStages * kStageBytes + kBarBytes;   // (the dynamic shared memory is declared 1024-byte aligned)
  // few tokens, K split over a cluster: where the peers' partial sums of this block's rows arrive
  static constexpr int kRecvBytes = BN < 128 ? BN * kTileRows * 4 : 0;
  // many tokens, add epilogue: two tiles of 128 rows x 32 float32 from which TMA adds into the residual
  static constexpr int kAddStageBytes = BN >= 128 ? 2 * kTileRows * 128 + 512 : 0;   // (+512: the tiles start 1024-byte aligned behind the barriers)
  static constexpr int kSmem = kPipeSmem + kRecvBytes + kAddStageBytes;
};

#ifndef PTL_VECTOR_REDUCE_COLUMNS
#define PTL_VECTOR_REDUCE_COLUMNS 64
#endif
constexpr int kVectorReduceColumns = PTL_VECTOR_REDUCE_COLUMNS;   // column tiles from this width on add partial sums four rows per thread

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// SiLU for the bfloat16 path: the result is rounded to 8 bits of mantissa, so the fast
// exponential and reciprocal (about 2 ulp of float32) cost no accuracy that survives.
__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// ---------------------------------------------------------------- epilogue of one row's 16 accumulators
// Normal mode: `row` is a token, columns c0..c0+15 are features.
template <int EPI>
__device__ __forceinline__ void store_normal(const GemmParams& p, int row, int c0, const float (&v)[16], size_t out_row) {
  if (row >= p.rows) return;
  const int n_total = p.cols;
  if (EPI == 3) {
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + out_row * p.ld_out + c0 / 2;
    if (c0 + 16 <= n_total && (p.ld_out % 8 == 0)) {
      uint4 pk;
      uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 t = __floats2bfloat162_rn(silu_f(v[4 * j]) * v[4 * j + 1], silu_f(v[4 * j + 2]) * v[4 * j + 3]);
        w[j] = *reinterpret_cast<uint32_t*>(&t);
      }
      *reinterpret_cast<uint4*>(o) = pk;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (c0 + 2 * j + 1 < n_total) o[j] = __float2bfloat16_rn(silu_f(v[2 * j]) * v[2 * j + 1]);
    }
    return;
  }
  const bool full = c0 + 16 <= n_total;
  if (EPI == 0) {
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + out_row * p.ld_out + c0;
    if (full && p.ld_out % 8 == 0) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint4 pk;
        uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 t = __floats2bfloat162_rn(v[8 * h + 2 * j], v[8 * h + 2 * j + 1]);
          w[j] = *reinterpret_cast<uint32_t*>(&t);
        }
        *reinterpret_cast<uint4*>(o + 8 * h) = pk;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (c0 + j < n_total) o[j] = __float2bfloat16_rn(v[j]);
    }
  } else {   // EPI 1 (store float32) or 2 (add into float32)
    float* o = (float*)p.out + out_row * p.ld_out + c0;
    if (full && p.ld_out % 4 == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float4 t = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        if (EPI == 2) {
          const float4 r = *reinterpret_cast<const float4*>(o + 4 * j);
          t.x += r.x; t.y += r.y; t.z += r.z; t.w += r.w;
        }
        *reinterpret_cast<float4*>(o + 4 * j) = t;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (c0 + j < n_total) o[j] = EPI == 2 ? o[j] + v[j] : v[j];
    }
  }
}

// The sum over the 16 lanes of a half warp (all lanes of the warp take part).
__device__ __forceinline__ float half_warp_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}

// The add epilogue for one feature n and token tok with few tokens; `have` is what the residual
// held if the caller fetched it already.  With p.xs the next norm's input goes out too; every lane of the
// warp must call this, the lanes of a half warp with the same token and 16 consecutive features.
__device__ __forceinline__ void add_and_emit(const GemmParams& p, int n, int tok, float v, bool fetched, float have, int lane,
                                             float norm_w = 0.f) {
  const bool valid = n < p.rows && tok < p.cols;
  float r = 0.f;
  if (valid) {
    float* o = (float*)p.out + (size_t)tok * p.ld_out + n;
    r = (fetched ? have : __ldcg(o)) + v;
    *o = r;
    if (p.xs) p.xs[(size_t)tok * p.xs_ld + n] = __float2bfloat16_rn(r * (fetched ? norm_w : __ldg(p.norm_w + n)));
  }
  if (p.xs) {
    const float sq = half_warp_sum(r * r);
    if ((lane & 15) == 0 && valid) p.sumsq[(size_t)tok * p.sumsq_ld + n / 16] = sq;
  }
}

// Swapped mode: `row` is a feature n, columns c0..c0+15 are tokens.
template <int EPI>
__device__ __forceinline__ void store_swapped(const GemmParams& p, int row, int c0, const float (&v)[16]) {
  const int n = row;
  const bool n_ok = n < p.rows;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int tok = c0 + j;
    if (EPI == 3) {
      const float up = __shfl_down_sync(0xffffffffu, v[j], 1);   // odd rows hold up_j; all lanes take part
      if (n_ok && tok < p.cols && (n & 1) == 0)
        ((__nv_bfloat16*)p.out)[(size_t)tok * p.ld_out + n / 2] = __float2bfloat16_rn(silu_f(v[j]) * up);
    } else if (EPI == 2) {
      add_and_emit(p, n, tok, v[j], false, 0.f, threadIdx.x & 31);
    } else if (n_ok && tok < p.cols) {
      if (EPI == 0) ((__nv_bfloat16*)p.out)[(size_t)tok * p.ld_out + n] = __float2bfloat16_rn(v[j]);
      else ((float*)p.out)[(size_t)tok * p.ld_out + n] = v[j];
    }
  }
}

// One output element of the swapped mode after the cluster reduction: feature n, token tok.
template <int EPI>
__device__ __forceinline__ void store_swapped_one(const GemmParams& p, int n, int tok, float v, float up) {
  if (n >= p.rows || tok >= p.cols) return;
  if (EPI == 0) ((__nv_bfloat16*)p.out)[(size_t)tok * p.ld_out + n] = __float2bfloat16_rn(v);
  else if (EPI == 1) ((float*)p.out)[(size_t)tok * p.ld_out + n] = v;
  else if (EPI == 2) ((float*)p.out)[(size_t)tok * p.ld_out + n] += v;
  else ((__nv_bfloat16*)p.out)[(size_t)tok * p.ld_out + n / 2] = __float2bfloat16_rn(silu_f(v) * up);
}

// 16 columns of this thread's TMEM lane, added over the issuers' accumulators; an issuer that had
// no stage (fewer stages than issuers) left its accumulator unwritten.
template <int BN, int WAYS>
__device__ __forceinline__ void load_ways(uint32_t taddr, int stages, float (&v)[16]) {
  uint32_t r[WAYS][16];
#pragma unroll
  for (int w = 0; w < WAYS; ++w) tmem_load_16_nowait(taddr + w * BN, r[w]);
  tmem_wait_ld();
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < WAYS; ++w) acc += w < stages ? __uint_as_float(r[w][j]) : 0.f;
    v[j] = acc;
  }
}

// (Few tokens: two blocks per SM must fit the register file, 102 registers a thread, and three of
// the 16- and 32-token instances without the add epilogue, 68: measured, 1 % of a decode step.  The
// compiler kept to that by itself until the many-token paths grew; now it is told.)
template <int BN, int EPI, bool PAIR = false>
__global__ void __launch_bounds__(kGemmThreads, BN < 128 ? ((EPI == 2 || BN == 64) ? 2 : 3) : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_row, const __grid_constant__ CUtensorMap map_col,
               const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
  using Cfg = TcCfg<BN, PAIR>;
  const uint32_t pair_rank = PAIR ? cluster_ctarank() : 0;     // 0: the block of a pair that issues the MMAs
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern to start at row 0
  unsigned char* smem = smem_raw;
  if (smem_addr(smem) & 1023u) {                               // never expected (the same in every block): refuse rather than compute garbage
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 99);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  // bars: [0,S) stage full, [S,2S) stage empty, then accumulator full[2], accumulator empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_scale = reinterpret_cast<float*>(smem + Cfg::kStages * Cfg::kStageBytes + 256);   // few tokens: scale of each token

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0 && p.timeline) { timeline_stamp(p.timeline, 0); if (blockIdx.x == 0 && blockIdx.y == 0) p.timeline[0] = p.timeline_kind; }
  const int num_kb = (p.K + kTileK - 1) / kTileK;
  // swapped mode: one tile per block (blockIdx.x = row tile, blockIdx.y = K split);
  // normal mode: the block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (token tiles fastest)
  // a pair walks the tiles two token tiles at a time (the second one may lie beyond the tokens: it reads zeros and stores nothing)
  const int tiles_mp = PAIR ? (p.tiles_m + 1) / 2 : p.tiles_m;
  const int tiles_mn = tiles_mp * p.tiles_n;
  const int total_tiles = p.swapped ? 1 : tiles_mn * p.ksplits;      // work units: (tile, part of the K range)
  const int first_tile = p.swapped ? 0 : (PAIR ? blockIdx.x / 2 : blockIdx.x);
  const int tile_step = p.swapped ? 1 : (PAIR ? gridDim.x / 2 : gridDim.x);
  const int split = p.swapped ? blockIdx.y : 0;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(num_kb, kb0 + p.kb_per_split);
  const int my_kb = max(0, kb1 - kb0);
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar_base = smem_addr(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + 2 + b); };
  auto tile_rows_cols = [&](int tile, int& row_tile, int& col_tile) {
    if (p.swapped) { row_tile = blockIdx.x; col_tile = 0; }
    else { const int t = tile % tiles_mn; row_tile = (t % tiles_mp) * (PAIR ? 2 : 1) + pair_rank; col_tile = t / tiles_mp; }
  };
  // the K blocks of a work unit: first one and how many
  auto unit_k = [&](int tile, int& first_kb, int& n_kb) {
    if (p.swapped || p.ksplits == 1) { first_kb = kb0; n_kb = my_kb; return; }
    first_kb = (tile / tiles_mn) * p.kb_per_split;
    n_kb = max(0, min(num_kb, first_kb + p.kb_per_split) - first_kb);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), p.swapped ? Cfg::kAccWays : 1); mbar_init(acc_empty(b), PAIR ? 16 : 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_row) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_col) : "memory");
    if (EPI == 2 && p.tma_add) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out) : "memory");
  }
  if (warp == 1) {
    if (PAIR) {               // (the same warp in both blocks of the pair, the same place for the address)
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(Cfg::kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(Cfg::kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // a pair: neither block may count bytes on the other's barriers, arrive on them or write its
  // TMEM before both have set theirs up
  if (PAIR) { cluster_arrive(); cluster_wait(); }
  // blocks of a cluster write into each other's shared memory later on; none may do so before all
  // of them run, which the wait that matches this arrival establishes
  if (p.swapped && p.splits > 1) cluster_arrive();

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    // Weights do not depend on earlier kernels of the step: their tiles for the first ring of
    // stages are requested before the wait on the predecessor, the tokens after.
    int it = 0;          // stage uses so far, over all tiles of this block
    int pre = 0;
    int row0 = 0, col0 = 0, kb00 = 0, nkb0 = 0;     // many tokens: this block's first work unit
    if (p.swapped) {
      pre = min(my_kb, Cfg::kStages);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full_bar(i), Cfg::kStageBytes);
        tma_load_2d(smem_base + i * Cfg::kStageBytes, &map_row, full_bar(i), (kb0 + i) * kTileK, blockIdx.x * kTileRows);
      }
    } else if (first_tile < total_tiles) {
      tile_rows_cols(first_tile, row0, col0);
      unit_k(first_tile, kb00, nkb0);
      pre = min(nkb0, Cfg::kStages);
      for (int i = 0; i < pre; ++i) {
        const uint32_t dst = smem_base + i * Cfg::kStageBytes + Cfg::kRowBytes;
        if (PAIR) {
          if (pair_rank == 0) mbar_expect_tx(full_bar(i), 2 * Cfg::kStageBytes);
          tma_load_2d_pair(dst, &map_col, map_to_peer(full_bar(i), 0), (kb00 + i) * kTileK, col0 * BN + (int)pair_rank * (BN / 2));
        } else {
          mbar_expect_tx(full_bar(i), Cfg::kStageBytes);
          tma_load_2d(dst, &map_col, full_bar(i), (kb00 + i) * kTileK, col0 * BN);
        }
      }
    }
    pdl_wait();                // (few tokens: the tokens of those stages are requested by the MMA issuers, each for its own stages)
    pdl_launch_dependents();
    timeline_stamp(p.timeline, 1);
    if (!p.swapped) {
      for (int i = 0; i < pre; ++i) {
        const uint32_t dst = smem_base + i * Cfg::kStageBytes;
        if (i == 0 && p.withhold_first_load) continue;      // (self-test: this stage never fills)
        if (PAIR) tma_load_2d_pair(dst, &map_row, map_to_peer(full_bar(i), 0), (kb00 + i) * kTileK, row0 * kTileRows);
        else tma_load_2d(dst, &map_row, full_bar(i), (kb00 + i) * kTileK, row0 * kTileRows);
      }
    }
    it = pre;
    bool ok = true;
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
      int row_tile, col_tile, ukb0, unkb;
      tile_rows_cols(tile, row_tile, col_tile);
      unit_k(tile, ukb0, unkb);
      for (int i = (tile == first_tile ? pre : 0); i < unkb; ++i, ++it) {
        const int s = it % Cfg::kStages;
        const uint32_t ph = (it / Cfg::kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, 1, p.poll_limit)) { ok = false; break; }
        const uint32_t dst = smem_base + s * Cfg::kStageBytes;
        if (PAIR) {
          // both blocks' tiles are counted on the issuing block's barrier, which expects both (a
          // count that arrives before the expectation is made just runs negative for a while)
          if (pair_rank == 0) mbar_expect_tx(full_bar(s), 2 * Cfg::kStageBytes);
          const uint32_t bar = map_to_peer(full_bar(s), 0);
          tma_load_2d_pair(dst, &map_row, bar, (ukb0 + i) * kTileK, row_tile * kTileRows);
          tma_load_2d_pair(dst + Cfg::kRowBytes, &map_col, bar, (ukb0 + i) * kTileK, col_tile * BN + (int)pair_rank * (BN / 2));
          continue;
        }
        mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
        tma_load_2d(dst, &map_row, full_bar(s), (ukb0 + i) * kTileK, row_tile * kTileRows);
        tma_load_2d(dst + Cfg::kRowBytes, &map_col, full_bar(s), (ukb0 + i) * kTileK, col_tile * BN);
      }
    }
    if (*abort_flag) {
      // leave no copy in flight behind: wait (bounded) for the stages that were requested last
      for (int i = max(0, it - Cfg::kStages); i < it; ++i) {
        const int s = i % Cfg::kStages;
        for (uint32_t t = 0; t < (1u << 16) && !mbar_try_wait(full_bar(s), (i / Cfg::kStages) & 1); ++t) __nanosleep(100);
      }
    }
  } else if (p.swapped && (warp == 1 || (warp >= 6 && warp - 5 < Cfg::kAccWays))) {
    // ------------------------------------------------------------ MMA issuers, few tokens
    pdl_wait();
    pdl_launch_dependents();
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(kTileRows, BN);
      const int issuer = warp == 1 ? 0 : warp - 5;
      const uint32_t acc = tmem_base + issuer * BN;
      // the weights of the first ring of stages are on their way since before the wait; their tokens follow now
      for (int i = issuer; i < min(my_kb, Cfg::kStages); i += Cfg::kAccWays) {
        if (i == 0 && p.withhold_first_load) continue;        // (self-test: this stage never fills)
        tma_load_2d(smem_base + i * Cfg::kStageBytes + Cfg::kRowBytes, &map_col, full_bar(i), (kb0 + i) * kTileK, 0);
      }
      for (int i = issuer; i < my_kb; i += Cfg::kAccWays) {
        const int s = i % Cfg::kStages;
        if (!mbar_wait(full_bar(s), (i / Cfg::kStages) & 1, abort_flag, p.status, 2, p.poll_limit)) break;
        if (i == 0) timeline_stamp(p.timeline, 2);
        tcgen05_fence_after();
        const uint32_t a = smem_base + s * Cfg::kStageBytes;
        const uint32_t b = a + Cfg::kRowBytes;
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k)
          tcgen05_mma_bf16(acc, smem_desc_sw128(a + k * 32), smem_desc_sw128(b + k * 32), idesc, (i >= Cfg::kAccWays || k > 0) ? 1u : 0u);
        tcgen05_commit(empty_bar(s));      // the stage is free once these MMAs have read it
      }
      tcgen05_commit(acc_full(0));         // this issuer's accumulator is complete (also when it had nothing to do)
      if (issuer == 0) timeline_stamp(p.timeline, 3);
    }
  } else if (warp == 1 && lane == 0 && pair_rank == 0) {
    // ------------------------------------------------------------ MMA issuer, many tokens (of a pair: the even block's)
    pdl_wait();
    pdl_launch_dependents();
    constexpr uint32_t idesc = instr_desc_bf16(PAIR ? 2 * kTileRows : kTileRows, BN);
    int it = 0;
    bool ok = true;
    int lt = 0;          // tiles of this block so far
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, ++lt) {
      const int buf = Cfg::kAccBufs == 2 ? (lt & 1) : 0;
      const int use = Cfg::kAccBufs == 2 ? (lt >> 1) : lt;            // how often this buffer was used before
      ok = mbar_wait(acc_empty(buf), (use & 1) ^ 1, abort_flag, p.status, 4, p.poll_limit);    // the epilogue has drained it
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t acc = tmem_base + buf * BN;
      int ukb0, unkb;
      unit_k(tile, ukb0, unkb);
      for (int i = 0; i < unkb; ++i, ++it) {
        const int s = it % Cfg::kStages;
        const uint32_t ph = (it / Cfg::kStages) & 1;
        ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, 2, p.poll_limit);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t a = smem_base + s * Cfg::kStageBytes;
        const uint32_t b = a + Cfg::kRowBytes;
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) {
          if (PAIR) tcgen05_mma_bf16_pair(acc, smem_desc_sw128(a + k * 32), smem_desc_sw128(b + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
          else tcgen05_mma_bf16(acc, smem_desc_sw128(a + k * 32), smem_desc_sw128(b + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        if (PAIR) tcgen05_commit_pair(empty_bar(s));     // the stage is free, in both blocks, once these MMAs have read it
        else tcgen05_commit(empty_bar(s));
      }
      if (PAIR) tcgen05_commit_pair(acc_full(buf));      // the accumulator is complete (also when there was nothing to do)
      else tcgen05_commit(acc_full(buf));
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue
    pdl_wait();               // the epilogue reads and writes memory that earlier kernels touch
    pdl_launch_dependents();
    const int quad = warp & 3;                 // TMEM lanes 32*quad.. belong to this warp
    const int half = (warp - 2) >> 2;          // with many tokens, which half of the tile's columns it handles
    const int row_in_tile = quad * 32 + lane;
    if (BN < 128 && p.swapped && p.scale_sumsq && half == 0) {
      // few tokens: the scale of every token, summed over its slots by 128 / BN threads each
      constexpr int kPer = BN < 128 ? 128 / BN : 1;
      const int tok = row_in_tile / kPer, part = row_in_tile % kPer;
      float sum = 0.f;
      if (tok < p.cols) {
        const float* src = p.scale_sumsq + (size_t)tok * p.scale_ld;
        if (p.scale_ld % 4 == 0 && p.scale_slots % 4 == 0) {
          const float4* src4 = reinterpret_cast<const float4*>(src);
#pragma unroll 4
          for (int k = part; k < p.scale_slots / 4; k += kPer) {
            const float4 q4 = __ldcg(src4 + k);
            sum += (q4.x + q4.y) + (q4.z + q4.w);
          }
        } else {
          for (int k = part; k < p.scale_slots; k += kPer) sum += __ldcg(src + k);
        }
      }
#pragma unroll
      for (int o = kPer / 2; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (part == 0) s_scale[tok] = tok < p.cols ? rsqrtf(sum * p.scale_inv_n + p.scale_eps) : 0.f;
      asm volatile("bar.sync 1, 128;" ::: "memory");           // the four warps that read the table
    }
    int lt = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step, ++lt) {
      int row_tile, col_tile;
      tile_rows_cols(tile, row_tile, col_tile);
      const int buf = Cfg::kAccBufs == 2 ? (lt & 1) : 0;
      const int use = Cfg::kAccBufs == 2 ? (lt >> 1) : lt;
      const int row = row_tile * kTileRows + row_in_tile;
      int ukb0, unkb;
      unit_k(tile, ukb0, unkb);
      const size_t out_row = (size_t)row + (p.swapped ? 0 : (size_t)(tile / tiles_mn) * p.rows);     // partial sums of part s: rows s * rows..
      // the add epilogue fetches what it adds to ahead of time: 32 columns before the accumulator
      // is even complete, then the next 32 while the current ones are being written
      constexpr int kHalfCols = BN / 2 >= 32 ? BN / 2 : 32;
      float4 ahead[8];
      const bool can_prefetch = EPI == 2 && !p.swapped && row < p.rows && p.ld_out % 4 == 0 && p.cols % 32 == 0;
      auto prefetch = [&](int c0) {
        const float4* src = reinterpret_cast<const float4*>((const float*)p.out + (size_t)row * p.ld_out + col_tile * BN + c0);
#pragma unroll
        for (int j = 0; j < 8; ++j) ahead[j] = col_tile * BN + c0 + 4 * j < p.cols ? __ldcg(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
      };
      if (can_prefetch) prefetch(half * kHalfCols);
      float row_scale = 1.f;                   // many tokens: this thread's token
      if (!p.swapped && p.scale_sumsq && row < p.rows) {
        float sum = 0.f;
        for (int k = 0; k < p.scale_slots; ++k) sum += __ldcg(p.scale_sumsq + (size_t)row * p.scale_ld + k);
        row_scale = rsqrtf(sum * p.scale_inv_n + p.scale_eps);
      }
      float ss = 0.f;                          // sum of squares of this thread's share of its row (add epilogue, emitting)
      if (!mbar_wait(acc_full(buf), use & 1, abort_flag, p.status, 3, p.poll_limit)) break;
      if (warp == 2 && lane == 0 && lt == 0) timeline_stamp(p.timeline, 4);
      tcgen05_fence_after();
      const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN;
      if (!p.swapped && row_tile * kTileRows >= p.rows) {
        // the second token tile of a pair, beyond the tokens: nothing to store
      } else if (EPI == 2 && !p.swapped && p.tma_add) {
        // The accumulator goes out through shared memory, 32 columns at a time, and TMA adds it into
        // the residual: nothing of the residual is read here, and global memory sees whole rows of 128 bytes.
        const uint32_t buf = smem_base + Cfg::kStages * Cfg::kStageBytes + 1024 + half * (kTileRows * 128);
        const bool issuer = quad == 0 && lane == 0;
#pragma unroll 1
        for (int c0 = half * kHalfCols; c0 < (half + 1) * kHalfCols && c0 < BN && col_tile * BN + c0 < p.cols; c0 += 32) {
          uint32_t r[32];
          tmem_load_32(acc + c0, r);
          if (issuer) bulk_wait_read_all();                      // the tile sent before has left the buffer
          asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
#pragma unroll
          for (int j = 0; j < 8; ++j)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + row_in_tile * 128 + ((j ^ (row_in_tile & 7)) << 4)),
                         "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync %0, 128;" ::"r"(2 + half) : "memory");
          if (issuer) tma_reduce_add_2d(&map_out, buf, col_tile * BN + c0, row_tile * kTileRows);
        }
      } else if (EPI == 4 && !p.swapped) {
        // q|k|v with rotary encoding and cache write: this thread's token, every second head of the
        // tile's columns (the two warps of a lane quarter take turns; tiles start on head
        // boundaries), 32 pairs (x[j], x[j + d/2]) at a time.  The accumulator is rounded to bfloat16 first and rotated
        // from there, as the separate kernel does with the stored projection: the same bits.
        const int hd = p.rope_d, hh2 = hd / 2;
        int slot = row < p.rows ? __ldcg(p.rope_slots + row) : -1;
        if (slot >= p.rope_num_slots) slot = -1;                                   // never write outside the pool
        const int page = slot >= 0 ? slot / p.rope_page : 0, off = slot >= 0 ? slot % p.rope_page : 0;
        const size_t plane = (size_t)p.rope_nkv * p.rope_page * hd;              // one of k / v inside a page
        __nv_bfloat16* kdst = p.rope_cache + ((size_t)page * 2) * plane + (size_t)off * hd;
        const float2* cs_row = p.rope_table + (size_t)(row < p.rows ? row : 0) * hh2;
#pragma unroll 1
        for (int h0 = half * hd; h0 + hd <= BN; h0 += 2 * hd) {
          const int col = col_tile * BN + h0;                                      // first column of the head
          const int gh = col / hd;                                                 // head number among q, k, v heads
          const bool live = col < p.cols;
          const int kind = gh < p.rope_nq ? 0 : (gh < p.rope_nq + p.rope_nkv ? 1 : 2);
#pragma unroll 1
          for (int c = 0; c < hh2; c += 32) {
            uint32_t a[32], b[32];
            tmem_load_32_nowait(acc + h0 + c, a);
            tmem_load_32_nowait(acc + h0 + c + hh2, b);
            tmem_wait_ld();
            uint32_t pa[16], pb[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float x1a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[j]) * row_scale));
              float x1b = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[j + 1]) * row_scale));
              float x2a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(b[j]) * row_scale));
              float x2b = __bfloat162float(__float2bfloat16_rn(__uint_as_float(b[j + 1]) * row_scale));
              float o1a = x1a, o1b = x1b, o2a = x2a, o2b = x2b;
              if (kind != 2 && live) {
                const float4 cs = __ldg(reinterpret_cast<const float4*>(cs_row + c + j));   // (cos, sin) of two neighbouring frequencies
                rope_rotate(x1a, x2a, cs.x, cs.y, o1a, o2a);
                rope_rotate(x1b, x2b, cs.z, cs.w, o1b, o2b);
              }
              __nv_bfloat162 t1 = __floats2bfloat162_rn(o1a, o1b), t2 = __floats2bfloat162_rn(o2a, o2b);
              pa[j >> 1] = *reinterpret_cast<uint32_t*>(&t1);
              pb[j >> 1] = *reinterpret_cast<uint32_t*>(&t2);
            }
            __nv_bfloat16* dst = nullptr;
            if (live && row < p.rows) {
              if (kind == 0) dst = (__nv_bfloat16*)p.out + (size_t)row * p.ld_out + col + c;
              else if (slot >= 0) dst = kdst + (kind == 2 ? plane : 0) + (size_t)(gh - p.rope_nq - (kind == 2 ? p.rope_nkv : 0)) * p.rope_page * hd + c;
            }
            if (dst) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                *reinterpret_cast<uint4*>(dst + 8 * q4) = make_uint4(pa[4 * q4], pa[4 * q4 + 1], pa[4 * q4 + 2], pa[4 * q4 + 3]);
                *reinterpret_cast<uint4*>(dst + hh2 + 8 * q4) = make_uint4(pb[4 * q4], pb[4 * q4 + 1], pb[4 * q4 + 2], pb[4 * q4 + 3]);
              }
            }
          }
        }
      } else if (!p.swapped) {
#pragma unroll 1
        for (int c0 = half * kHalfCols; c0 < (half + 1) * kHalfCols && c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_load_32(acc + c0, r);
          float v[16];
          if (can_prefetch) {
            float4 cur[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) cur[j] = ahead[j];
            if (c0 + 32 < (half + 1) * kHalfCols) prefetch(c0 + 32);
            float* o = (float*)p.out + (size_t)row * p.ld_out + col_tile * BN + c0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (col_tile * BN + c0 + 4 * j < p.cols) {
                float4 t = cur[j];
                t.x += __uint_as_float(r[4 * j]); t.y += __uint_as_float(r[4 * j + 1]);
                t.z += __uint_as_float(r[4 * j + 2]); t.w += __uint_as_float(r[4 * j + 3]);
                *reinterpret_cast<float4*>(o + 4 * j) = t;
                if (p.xs) {
                  const float4 w4 = __ldg(reinterpret_cast<const float4*>(p.norm_w + col_tile * BN + c0) + j);
                  uint2 pk;
                  __nv_bfloat162 lo = __floats2bfloat162_rn(t.x * w4.x, t.y * w4.y), hi = __floats2bfloat162_rn(t.z * w4.z, t.w * w4.w);
                  pk.x = *reinterpret_cast<uint32_t*>(&lo);
                  pk.y = *reinterpret_cast<uint32_t*>(&hi);
                  *reinterpret_cast<uint2*>(p.xs + (size_t)row * p.xs_ld + col_tile * BN + c0 + 4 * j) = pk;
                  ss += t.x * t.x; ss += t.y * t.y; ss += t.z * t.z; ss += t.w * t.w;
                }
              }
            }
            continue;
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = unkb > 0 ? __uint_as_float(r[16 * h + j]) * row_scale : 0.f;
            store_normal<EPI>(p, row, col_tile * BN + c0 + 16 * h, v, out_row);
          }
        }
        if (can_prefetch && p.xs) p.sumsq[(size_t)row * p.sumsq_ld + col_tile * 2 + half] = ss;
      } else if (half == 1) {
        // few tokens: the tile has at most 64 columns, one warp per lane quarter does it all
        // (warps 6.. issue MMAs instead; a warp that gets here only waits for the tile)
      } else if (p.splits == 1) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16];
          load_ways<BN, Cfg::kAccWays>(acc + c0, my_kb, v);
          if (p.scale_sumsq) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] *= s_scale[c0 + j];
          }
          store_swapped<EPI>(p, row, c0, v);
        }
      } else {
        // K split over the cluster: the tile is sent to the owners of its rows below
      }
      // this warp has read its share of the buffer: one of the eight arrivals that free it
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && pair_rank != 0) mbar_arrive_cluster(map_to_peer(acc_empty(buf), 0));      // the issuing block waits for both blocks' warps
        else mbar_arrive(acc_empty(buf));
      }
    }
    if (EPI == 2 && !p.swapped && p.tma_add && quad == 0 && lane == 0) bulk_wait_all();   // the adds have landed
  }
  if (p.swapped && p.splits > 1) {
    const int row_tile = blockIdx.x;
    const int S = p.splits;
    const int rows_per = kTileRows / S;                    // rows of the tile that each block owns (S is 2, 4 or 8)
    float* recv = reinterpret_cast<float*>(smem + Cfg::kPipeSmem);             // [S sources][BN columns][rows_per]
    cluster_wait();                                        // every block of the cluster runs
    // Both sets of four warps send (a warp reaches the TMEM lanes 32 * (warp % 4)..): they take turns
    // at the groups of 16 columns.  The warps that issued MMAs have not waited for the accumulators yet.
    bool acc_ok = true;
    if (warp >= 6 && BN > 16) {
      acc_ok = mbar_wait(acc_full(0), 0, abort_flag, p.status, 3, p.poll_limit);
      tcgen05_fence_after();
    }
    if (warp >= 2 && (warp < 6 || BN > 16) && acc_ok && !*abort_flag) {
      // this thread's row of the tile goes to the block that owns it (neighbouring lanes write
      // neighbouring words: wider stores of a row's columns would collide in the banks)
      const int rl = (warp & 3) * 32 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
      const uint32_t dst = map_to_peer(smem_addr(recv) + 4u * ((split * BN) * rows_per + rl % rows_per), rl / rows_per);
#pragma unroll 1
      for (int c0 = (BN > 16 ? ((warp - 2) >> 2) * 16 : 0); c0 < BN; c0 += (BN > 16 ? 32 : 16)) {
        float v[16];
        load_ways<BN, Cfg::kAccWays>(acc + c0, my_kb, v);
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) st_peer_f32(dst + 4u * ((c0 + jj) * rows_per), v[jj]);
      }
    }
    tcgen05_fence_before();
    // Two ways to add the partial sums up.  With many columns (tokens) a thread takes four neighbouring rows of
    // one column with 16-byte reads and writes; with few columns that leaves most threads idle, and one result
    // per thread measured faster.
    if constexpr (BN >= kVectorReduceColumns) {
      // The owner's threads each take four neighbouring rows (features) of one column (token): chunk q is
      // rows 4 (q % (rows_per / 4))..+3 of column q / (rows_per / 4).  The partial sums of a chunk are 16
      // bytes in every source's part of `recv`, its four results 8 or 16 contiguous bytes of the output.
      const int r4_per = rows_per / 4;
      const int chunks_total = r4_per * BN;
      const int t = threadIdx.x - 64;                        // 0..255 in the epilogue warps
      const bool worker = warp >= 2;
      cluster_arrive();
      // what the add epilogue adds to and multiplies by, fetched under the barrier: this thread's first chunk
      float4 res0 = make_float4(0.f, 0.f, 0.f, 0.f), nw0 = make_float4(0.f, 0.f, 0.f, 0.f);
      const bool vec_out = p.ld_out % 4 == 0 && p.rows % 4 == 0;      // whole chunks exist and are aligned
      if (EPI == 2 && worker && t < chunks_total && vec_out) {
        const int n = row_tile * kTileRows + split * rows_per + 4 * (t % r4_per), col = t / r4_per;
        if (n < p.rows && col < p.cols) {
          res0 = __ldcg(reinterpret_cast<const float4*>((const float*)p.out + (size_t)col * p.ld_out + n));
          if (p.xs) nw0 = __ldg(reinterpret_cast<const float4*>(p.norm_w + n));
        }
      }
      cluster_wait();                                        // the partial sums of this block's rows have arrived
      if (worker && !*abort_flag) {
#pragma unroll 1
        for (int q = t, i = 0; q < chunks_total; q += 256, ++i) {
          const int r = 4 * (q % r4_per), col = q / r4_per;
          const float* src = recv + col * rows_per + r;
          float4 a[8];
#pragma unroll
          for (int z = 0; z < 8; ++z) a[z] = z < S ? *reinterpret_cast<const float4*>(src + z * BN * rows_per) : make_float4(0.f, 0.f, 0.f, 0.f);
          float v[4] = {a[0].x, a[0].y, a[0].z, a[0].w};
#pragma unroll
          for (int z = 1; z < 8; ++z) { v[0] += a[z].x; v[1] += a[z].y; v[2] += a[z].z; v[3] += a[z].w; }     // in rank order: deterministic
          if (p.scale_sumsq) {
            const float sc = s_scale[col];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] *= sc;
          }
          const int n = row_tile * kTileRows + split * rows_per + r;
          const bool live = n < p.rows && col < p.cols;
          if (EPI == 2) {
            // residual += v; with p.xs the next norm's input and the sum of squares of 16 features (four lanes) go out too
            float rn[4] = {0.f, 0.f, 0.f, 0.f};
            if (live && vec_out) {
              float4* o = reinterpret_cast<float4*>((float*)p.out + (size_t)col * p.ld_out + n);
              const float4 have = i == 0 ? res0 : __ldcg(o);
              rn[0] = have.x + v[0]; rn[1] = have.y + v[1]; rn[2] = have.z + v[2]; rn[3] = have.w + v[3];
              *o = make_float4(rn[0], rn[1], rn[2], rn[3]);
              if (p.xs) {
                const float4 w4 = i == 0 ? nw0 : __ldg(reinterpret_cast<const float4*>(p.norm_w + n));
                uint2 pk;
                pk.x = pack_bf16x2(rn[0] * w4.x, rn[1] * w4.y);
                pk.y = pack_bf16x2(rn[2] * w4.z, rn[3] * w4.w);
                *reinterpret_cast<uint2*>(p.xs + (size_t)col * p.xs_ld + n) = pk;
              }
            } else if (col < p.cols) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (n + j < p.rows) {
                  float* o = (float*)p.out + (size_t)col * p.ld_out + n + j;
                  rn[j] = __ldcg(o) + v[j];
                  *o = rn[j];
                  if (p.xs) p.xs[(size_t)col * p.xs_ld + n + j] = __float2bfloat16_rn(rn[j] * __ldg(p.norm_w + n + j));
                }
              }
            }
            if (p.xs) {
              float sq = (rn[0] * rn[0] + rn[1] * rn[1]) + (rn[2] * rn[2] + rn[3] * rn[3]);
              sq += __shfl_xor_sync(0xffffffffu, sq, 1);       // the four lanes that hold 16 neighbouring features of this token
              sq += __shfl_xor_sync(0xffffffffu, sq, 2);
              if ((lane & 3) == 0 && live) p.sumsq[(size_t)col * p.sumsq_ld + n / 16] = sq;
            }
          } else if (EPI == 3) {
            // rows alternate gate_j, up_j: two results
            if (col < p.cols) {
              __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)col * p.ld_out + n / 2;
              if (n + 3 < p.rows && p.ld_out % 2 == 0) {
                *reinterpret_cast<uint32_t*>(o) = pack_bf16x2(silu_f(v[0]) * v[1], silu_f(v[2]) * v[3]);
              } else {
                if (n + 1 < p.rows) o[0] = __float2bfloat16_rn(silu_f(v[0]) * v[1]);
                if (n + 3 < p.rows) o[1] = __float2bfloat16_rn(silu_f(v[2]) * v[3]);
              }
            }
          } else if (col < p.cols) {
            if (EPI == 0) {
              __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)col * p.ld_out + n;
              if (live && vec_out) {
                uint2 pk;
                pk.x = pack_bf16x2(v[0], v[1]);
                pk.y = pack_bf16x2(v[2], v[3]);
                *reinterpret_cast<uint2*>(o) = pk;
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) if (n + j < p.rows) o[j] = __float2bfloat16_rn(v[j]);
              }
            } else {
              float* o = (float*)p.out + (size_t)col * p.ld_out + n;
              if (live && vec_out) {
                *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) if (n + j < p.rows) o[j] = v[j];
              }
            }
          }
        }
      }
    } else {
      const int group = EPI == 3 ? rows_per / 2 : rows_per;  // items per column: rows, or gate/up pairs
      const int items = group * BN;
      const int t = threadIdx.x - 64;                        // 0..255 in the epilogue warps
      const bool worker = warp >= 2;
      auto item_pos = [&](int idx, int& r, int& col) {
        col = idx / group;
        r = EPI == 3 ? 2 * (idx % group) : idx % group;
      };
      cluster_arrive();
      // what the add epilogue adds to and multiplies by, fetched under the barrier: this thread's first
      // four items (16 to 64 tokens give a thread 1 to 4 of them with eight splits; a fetch inside the
      // loop below costs a trip to L2 each time, 1 us per round at 64 tokens)
      constexpr int kAheadItems = 4;
      float res0[kAheadItems], nw0[kAheadItems];
#pragma unroll
      for (int i = 0; i < kAheadItems; ++i) {
        res0[i] = 0.f;
        nw0[i] = 0.f;
        const int idx = t + 256 * i;
        if (EPI == 2 && worker && idx < items) {
          int r, col;
          item_pos(idx, r, col);
          const int n = row_tile * kTileRows + split * rows_per + r;
          if (n < p.rows && col < p.cols) {
            res0[i] = __ldcg((const float*)p.out + (size_t)col * p.ld_out + n);
            if (p.xs) nw0[i] = __ldg(p.norm_w + n);
          }
        }
      }
      cluster_wait();                                        // the partial sums of this block's rows have arrived
      if (worker && !*abort_flag) {
        auto sum_sources = [&](int r, int col) {
          float a[8];
#pragma unroll
          for (int z = 0; z < 8; ++z) a[z] = z < S ? recv[(z * BN + col) * rows_per + r] : 0.f;
          float v = a[0];
#pragma unroll
          for (int z = 1; z < 8; ++z) v += a[z];
          return v;
        };
#pragma unroll 1
        for (int idx = t, i = 0; idx < items; idx += 256, ++i) {
          int r, col;
          item_pos(idx, r, col);
          const int n = row_tile * kTileRows + split * rows_per + r;
          const float sc = p.scale_sumsq ? s_scale[col] : 1.f;
          const float v = sum_sources(r, col) * sc;
          if (EPI == 2) {
            float have = 0.f, nwv = 0.f;
#pragma unroll
            for (int j = 0; j < kAheadItems; ++j) if (j == i) { have = res0[j]; nwv = nw0[j]; }
            add_and_emit(p, n, col, v, i < kAheadItems, have, lane, nwv);     // (every lane: the sums of squares are added over half warps)
          } else {
            store_swapped_one<EPI>(p, n, col, v, EPI == 3 ? sum_sources(r + 1, col) * sc : 0.f);
          }
        }
      }
    }
  } else {
    tcgen05_fence_before();
    __syncthreads();
  }
  if (warp == 2 && lane == 0) timeline_stamp(p.timeline, 5);
  if (PAIR) { cluster_arrive(); cluster_wait(); }        // neither block frees TMEM or leaves while the other may still reach into it
  if (warp == 1) {
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------- host side
template <int BN, int EPI, bool PAIR = false>
static int launch_tc(const CUtensorMap& mr, const CUtensorMap& mc, const CUtensorMap& mo, const GemmParams& p, dim3 grid,
                     cudaStream_t stream) {
  using Cfg = TcCfg<BN, PAIR>;
  static SmemRaised raised = {};
  if (int rc = raise_shared_memory("gemm_tc", gemm_tc_kernel<BN, EPI, PAIR>, Cfg::kSmem, raised)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = ((p.swapped && p.splits > 1) || p.tma_add) ? Cfg::kSmem : Cfg::kPipeSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (pdl_flag()) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (PAIR || (p.swapped && p.splits > 1)) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = PAIR ? 2 : 1;
    attr[nattr].val.clusterDim.y = PAIR ? 1 : p.splits;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, EPI, PAIR>, mr, mc, mo, p);
  if (e != cudaSuccess) return fail("gemm_tc: launch failed: %s", cudaGetErrorString(e));
  return check_launch("gemm_tc");
}

template <int BN, bool PAIR = false>
static int launch_epi(int epi, const CUtensorMap& mr, const CUtensorMap& mc, const CUtensorMap& mo, const GemmParams& p, dim3 grid,
                      cudaStream_t s) {
  switch (epi) {
    case 0: return launch_tc<BN, 0, PAIR>(mr, mc, mo, p, grid, s);
    case 1: return launch_tc<BN, 1, PAIR>(mr, mc, mo, p, grid, s);
    case 2: return launch_tc<BN, 2, PAIR>(mr, mc, mo, p, grid, s);
    case 3: return launch_tc<BN, 3, PAIR>(mr, mc, mo, p, grid, s);
    case 4:
      if constexpr (BN >= 128) return launch_tc<BN, 4, PAIR>(mr, mc, mo, p, grid, s);
      else break;
  }
  return fail("gemm_tc: unknown epilogue %d", epi);
}

// The three sets of instances, each in a translation unit of its own.
int launch_few_tokens(int bn, int epi, const CUtensorMap& mr, const CUtensorMap& mc, const CUtensorMap& mo, const GemmParams& p, dim3 grid,
                      cudaStream_t s);      // bn 16, 32 or 64 tokens
int launch_many_tokens(int bn, int epi, const CUtensorMap& mr, const CUtensorMap& mc, const CUtensorMap& mo, const GemmParams& p, dim3 grid,
                       cudaStream_t s);     // bn 128, 192 or 256 features
int launch_pair_tiles(int bn, int epi, const CUtensorMap& mr, const CUtensorMap& mc, const CUtensorMap& mo, const GemmParams& p, dim3 grid,
                      cudaStream_t s);      // bn 192 or 256 features, pairs of blocks

}  // namespace ptl
