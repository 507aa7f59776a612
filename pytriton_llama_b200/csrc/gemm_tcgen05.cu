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
};

template <int BN> struct TcCfg {
  static constexpr int kStages = BN >= 256 ? 4 : (BN >= 128 ? 6 : (BN == 64 ? 3 : 4));   // few tokens: small blocks, two or three per SM
  static constexpr int kRowBytes = kTileRows * kTileK * 2;     // 16 KB
  static constexpr int kColBytes = BN * kTileK * 2;
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
  static constexpr int kTmemCols = BN >= 128 ? BN * kAccBufs : (BN == 64 ? 256 : (BN * kAccWays < 32 ? 32 : BN * kAccWays));   // power of two >= 32
  static constexpr int kPipeSmem = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
  // few tokens, K split over a cluster: where the peers' partial sums of this block's rows arrive
  static constexpr int kRecvBytes = BN < 128 ? BN * kTileRows * 4 : 0;
  static constexpr int kSmem = kPipeSmem + kRecvBytes;
};

// SiLU for the bfloat16 path: the result is rounded to 8 bits of mantissa, so the fast
// exponential and reciprocal (about 2 ulp of float32) cost no accuracy that survives.
__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// ---------------------------------------------------------------- epilogue of one row's 16 accumulators
// Normal mode: `row` is a token, columns c0..c0+15 are features.
template <int EPI>
__device__ __forceinline__ void store_normal(const GemmParams& p, int row, int c0, const float (&v)[16]) {
  if (row >= p.rows) return;
  const int n_total = p.cols;
  if (EPI == 3) {
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)row * p.ld_out + c0 / 2;
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
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)row * p.ld_out + c0;
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
    float* o = (float*)p.out + (size_t)row * p.ld_out + c0;
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
    } else if (n_ok && tok < p.cols) {
      if (EPI == 0) ((__nv_bfloat16*)p.out)[(size_t)tok * p.ld_out + n] = __float2bfloat16_rn(v[j]);
      else if (EPI == 1) ((float*)p.out)[(size_t)tok * p.ld_out + n] = v[j];
      else ((float*)p.out)[(size_t)tok * p.ld_out + n] += v[j];
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

template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_row, const __grid_constant__ CUtensorMap map_col, const GemmParams p) {
  using Cfg = TcCfg<BN>;
  extern __shared__ unsigned char smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern to start at row 0
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  // bars: [0,S) stage full, [S,2S) stage empty, then accumulator full[2], accumulator empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + kTileK - 1) / kTileK;
  // swapped mode: one tile per block (blockIdx.x = row tile, blockIdx.y = K split);
  // normal mode: the block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (token tiles fastest)
  const int total_tiles = p.swapped ? 1 : p.tiles_m * p.tiles_n;
  const int first_tile = p.swapped ? 0 : blockIdx.x;
  const int tile_step = p.swapped ? 1 : gridDim.x;
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
    else { row_tile = tile % p.tiles_m; col_tile = tile / p.tiles_m; }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), p.swapped ? Cfg::kAccWays : 1); mbar_init(acc_empty(b), 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_row) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_col) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(Cfg::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // blocks of a cluster write into each other's shared memory later on; none may do so before all
  // of them run, which the wait that matches this arrival establishes
  if (p.swapped && p.splits > 1) cluster_arrive();

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    // Weights do not depend on earlier kernels of the step: with swapped operands their tiles for
    // the first ring of stages are requested before the wait on the predecessor, the tokens after.
    int it = 0;          // stage uses so far, over all tiles of this block
    int pre = 0;
    if (p.swapped) {
      pre = min(my_kb, Cfg::kStages);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full_bar(i), Cfg::kStageBytes);
        tma_load_2d(smem_base + i * Cfg::kStageBytes, &map_row, full_bar(i), (kb0 + i) * kTileK, blockIdx.x * kTileRows);
      }
    }
    pdl_wait();                // (the tokens of those stages are requested by the MMA issuers, each for its own stages)
    pdl_launch_dependents();
    it = pre;
    bool ok = true;
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
      int row_tile, col_tile;
      tile_rows_cols(tile, row_tile, col_tile);
      for (int i = (tile == first_tile ? pre : 0); i < my_kb; ++i, ++it) {
        const int s = it % Cfg::kStages;
        const uint32_t ph = (it / Cfg::kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
        mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
        const uint32_t dst = smem_base + s * Cfg::kStageBytes;
        tma_load_2d(dst, &map_row, full_bar(s), (kb0 + i) * kTileK, row_tile * kTileRows);
        tma_load_2d(dst + Cfg::kRowBytes, &map_col, full_bar(s), (kb0 + i) * kTileK, col_tile * BN);
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
      for (int i = issuer; i < min(my_kb, Cfg::kStages); i += Cfg::kAccWays)
        tma_load_2d(smem_base + i * Cfg::kStageBytes + Cfg::kRowBytes, &map_col, full_bar(i), (kb0 + i) * kTileK, 0);
      for (int i = issuer; i < my_kb; i += Cfg::kAccWays) {
        const int s = i % Cfg::kStages;
        if (!mbar_wait(full_bar(s), (i / Cfg::kStages) & 1, abort_flag, p.status, 2)) break;
        tcgen05_fence_after();
        const uint32_t a = smem_base + s * Cfg::kStageBytes;
        const uint32_t b = a + Cfg::kRowBytes;
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k)
          tcgen05_mma_bf16(acc, smem_desc_sw128(a + k * 32), smem_desc_sw128(b + k * 32), idesc, (i >= Cfg::kAccWays || k > 0) ? 1u : 0u);
        tcgen05_commit(empty_bar(s));      // the stage is free once these MMAs have read it
      }
      tcgen05_commit(acc_full(0));         // this issuer's accumulator is complete (also when it had nothing to do)
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer, many tokens
    pdl_wait();
    pdl_launch_dependents();
    constexpr uint32_t idesc = instr_desc_bf16(kTileRows, BN);
    int it = 0;
    bool ok = true;
    int lt = 0;          // tiles of this block so far
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, ++lt) {
      const int buf = Cfg::kAccBufs == 2 ? (lt & 1) : 0;
      const int use = Cfg::kAccBufs == 2 ? (lt >> 1) : lt;            // how often this buffer was used before
      ok = mbar_wait(acc_empty(buf), (use & 1) ^ 1, abort_flag, p.status, 4);    // the epilogue has drained it
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t acc = tmem_base + buf * BN;
      for (int i = 0; i < my_kb; ++i, ++it) {
        const int s = it % Cfg::kStages;
        const uint32_t ph = (it / Cfg::kStages) & 1;
        ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, 2);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t a = smem_base + s * Cfg::kStageBytes;
        const uint32_t b = a + Cfg::kRowBytes;
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) {
          tcgen05_mma_bf16(acc, smem_desc_sw128(a + k * 32), smem_desc_sw128(b + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        tcgen05_commit(empty_bar(s));      // the stage is free once these MMAs have read it
      }
      tcgen05_commit(acc_full(buf));       // the accumulator is complete (also when there was nothing to do)
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue
    pdl_wait();               // the epilogue reads and writes memory that earlier kernels touch
    pdl_launch_dependents();
    const int quad = warp & 3;                 // TMEM lanes 32*quad.. belong to this warp
    const int half = (warp - 2) >> 2;          // with many tokens, which half of the tile's columns it handles
    const int row_in_tile = quad * 32 + lane;
    int lt = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step, ++lt) {
      int row_tile, col_tile;
      tile_rows_cols(tile, row_tile, col_tile);
      const int buf = Cfg::kAccBufs == 2 ? (lt & 1) : 0;
      const int use = Cfg::kAccBufs == 2 ? (lt >> 1) : lt;
      const int row = row_tile * kTileRows + row_in_tile;
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
      if (!mbar_wait(acc_full(buf), use & 1, abort_flag, p.status, 3)) break;
      tcgen05_fence_after();
      const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN;
      if (!p.swapped) {
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
              }
            }
            continue;
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = my_kb > 0 ? __uint_as_float(r[16 * h + j]) : 0.f;
            store_normal<EPI>(p, row, col_tile * BN + c0 + 16 * h, v);
          }
        }
      } else if (half == 1) {
        // few tokens: the tile has at most 64 columns, one warp per lane quarter does it all
        // (warps 6.. issue MMAs instead; a warp that gets here only waits for the tile)
      } else if (p.splits == 1) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16];
          load_ways<BN, Cfg::kAccWays>(acc + c0, my_kb, v);
          store_swapped<EPI>(p, row, c0, v);
        }
      } else {
        // K split over the cluster: the tile is sent to the owners of its rows below
      }
      // this warp has read its share of the buffer: one of the eight arrivals that free it
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(buf));
    }
  }
  if (p.swapped && p.splits > 1) {
    const int row_tile = blockIdx.x;
    const int S = p.splits;
    const int rows_per = kTileRows / S;                    // rows of the tile that each block owns (S is 2, 4 or 8)
    float* recv = reinterpret_cast<float*>(smem + Cfg::kPipeSmem - 1024);      // [S sources][BN columns][rows_per]
    cluster_wait();                                        // every block of the cluster runs
    if (warp >= 2 && warp < 6 && !*abort_flag) {
      // this thread's row of the tile goes to the block that owns it (neighbouring lanes write
      // neighbouring words: wider stores of a row's columns would collide in the banks)
      const int rl = (warp & 3) * 32 + lane;
      const uint32_t acc = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
      const uint32_t dst = map_to_peer(smem_addr(recv) + 4u * ((split * BN) * rows_per + rl % rows_per), rl / rows_per);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16];
        load_ways<BN, Cfg::kAccWays>(acc + c0, my_kb, v);
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) st_peer_f32(dst + 4u * ((c0 + jj) * rows_per), v[jj]);
      }
    }
    tcgen05_fence_before();
    const int group = EPI == 3 ? rows_per / 2 : rows_per;  // items per column: rows, or gate/up pairs
    const int items = group * BN;
    const int t = threadIdx.x - 64;                        // 0..255 in the epilogue warps
    const bool worker = warp >= 2;
    auto item_pos = [&](int idx, int& r, int& col) {
      col = idx / group;
      r = EPI == 3 ? 2 * (idx % group) : idx % group;
    };
    cluster_arrive();
    float res0 = 0.f;                                      // what the add epilogue adds to, fetched under the barrier
    if (EPI == 2 && worker && t < items) {
      int r, col;
      item_pos(t, r, col);
      const int n = row_tile * kTileRows + split * rows_per + r;
      if (n < p.rows && col < p.cols) res0 = __ldcg((const float*)p.out + (size_t)col * p.ld_out + n);
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
      for (int idx = t; idx < items; idx += 256) {
        int r, col;
        item_pos(idx, r, col);
        const int n = row_tile * kTileRows + split * rows_per + r;
        const float v = sum_sources(r, col);
        if (n >= p.rows || col >= p.cols) continue;
        if (EPI == 2) {
          float* o = (float*)p.out + (size_t)col * p.ld_out + n;
          *o = (idx == t ? res0 : __ldcg(o)) + v;
        } else {
          store_swapped_one<EPI>(p, n, col, v, EPI == 3 ? sum_sources(r + 1, col) : 0.f);
        }
      }
    }
  } else {
    tcgen05_fence_before();
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------- host side
template <int BN, int EPI>
static int launch_tc(const CUtensorMap& mr, const CUtensorMap& mc, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  using Cfg = TcCfg<BN>;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    PTL_REQUIRE(e == cudaSuccess, "gemm_tc: cannot raise shared memory to %d: %s", Cfg::kSmem, cudaGetErrorString(e));
    raised = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = (p.swapped && p.splits > 1) ? Cfg::kSmem : Cfg::kPipeSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (pdl_flag()) {
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (p.swapped && p.splits > 1) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = 1;
    attr[nattr].val.clusterDim.y = p.splits;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = nattr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, EPI>, mr, mc, p);
  if (e != cudaSuccess) return fail("gemm_tc: launch failed: %s", cudaGetErrorString(e));
  return check_launch("gemm_tc");
}

template <int BN>
static int launch_epi(int epi, const CUtensorMap& mr, const CUtensorMap& mc, const GemmParams& p, dim3 grid, cudaStream_t s) {
  switch (epi) {
    case 0: return launch_tc<BN, 0>(mr, mc, p, grid, s);
    case 1: return launch_tc<BN, 1>(mr, mc, p, grid, s);
    case 2: return launch_tc<BN, 2>(mr, mc, p, grid, s);
    case 3: return launch_tc<BN, 3>(mr, mc, p, grid, s);
  }
  return fail("gemm_tc: unknown epilogue %d", epi);
}

}  // namespace ptl

// out: epi 0 bf16 [M,N]; 1 float32 [M,N]; 2 float32 [M,N] added to in place; 3 bf16 [M,N/2].
// Returns -2 when the sizes are not ones this kernel takes (K % 8 != 0 or K < 64), so that the caller
// can use another product.  `splits_hint` > 0 forces the number of K splits when M <= 64 (1, 2, 4 or 8).
PTL_EXPORT int ptl_gemm_tc_bf16(void* out, const void* X, const void* W, int M, int N, int K, int ld_out, int epi,
                                int* status, int splits_hint, void* stream) {
  using namespace ptl;
  PTL_REQUIRE(M >= 0 && N > 0 && K > 0 && ld_out > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
  if (K % 8 != 0 || K < kTileK) return -2;
  PTL_REQUIRE(aligned16(X) && aligned16(W) && aligned16(out), "gemm_tc: operands must be 16-byte aligned");
  PTL_REQUIRE(epi != 3 || N % 2 == 0, "gemm_tc: the SiLU*up epilogue needs an even number of weight rows");
  if (M == 0) return 0;
  GemmParams p{};
  p.out = out; p.status = status;
  p.K = K; p.ld_out = ld_out;
  const int num_kb = (K + kTileK - 1) / kTileK;
  CUtensorMap mr, mc;
  cudaStream_t s = as_stream(stream);
  if (M > 64) {
    p.swapped = 0; p.rows = M; p.cols = N; p.splits = 1; p.kb_per_split = num_kb;
    const bool wide = N % 256 == 0 || N >= 2048;
    int rc = make_map(&mr, X, M, K, kTileRows);
    if (rc) return rc;
    rc = make_map(&mc, W, N, K, wide ? 256 : 128);
    if (rc) return rc;
    const int bn = wide ? 256 : 128;
    p.tiles_m = (M + kTileRows - 1) / kTileRows;
    p.tiles_n = (N + bn - 1) / bn;
    static int sm_count = 0;
    if (!sm_count) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
      if (sm_count <= 0) sm_count = 148;
    }
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    dim3 grid((unsigned)(tiles < sm_count ? tiles : sm_count));
    return wide ? launch_epi<256>(epi, mr, mc, p, grid, s) : launch_epi<128>(epi, mr, mc, p, grid, s);
  }
  // few tokens: swapped operands; the K range is split over a cluster of 1, 2, 4 or 8 blocks so
  // that about two blocks per SM stream the weights
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const int row_tiles = (N + kTileRows - 1) / kTileRows;
  int splits = 1;
  if (splits_hint > 0) {
    splits = splits_hint;
  } else {
    while (splits < 8 && row_tiles * splits * 2 <= 296 && num_kb / (splits * 2) >= 2) splits *= 2;
  }
  PTL_REQUIRE(splits == 1 || splits == 2 || splits == 4 || splits == 8, "gemm_tc: the K range splits 1, 2, 4 or 8 ways, not %d", splits);
  const int kb_per = (num_kb + splits - 1) / splits;
  p.swapped = 1; p.rows = N; p.cols = M; p.splits = splits; p.kb_per_split = kb_per;
  int rc = make_map(&mr, W, N, K, kTileRows);
  if (rc) return rc;
  rc = make_map(&mc, X, M, K, bn);
  if (rc) return rc;
  dim3 grid(row_tiles, splits);
  switch (bn) {
    case 16: return launch_epi<16>(epi, mr, mc, p, grid, s);
    case 32: return launch_epi<32>(epi, mr, mc, p, grid, s);
    default: return launch_epi<64>(epi, mr, mc, p, grid, s);
  }
}
