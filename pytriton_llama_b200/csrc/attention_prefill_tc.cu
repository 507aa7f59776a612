// Attention of prompt portions over the paged cache on the fifth-generation tensor cores
// (head size 64 or 128, bfloat16).  One block per (pair of tiles of up to 128 query tokens each, query
// head); the pair are consecutive rows of one request (tile B continues tile A; B may be absent),
// so both walk the same keys and every key/value tile is fetched once for 256 query rows:
//   S = Q K^T       tcgen05.mma 128 x keys x D into TMEM (float32), per tile of the pair; the K
//                   tile (128 keys with head size 64, 64 keys with 128: 16 KB either way) is
//                   fetched page by page with TMA into 128-byte-swizzled shared memory, 64
//                   values of a row at a time;
//   softmax         a group of four warps per tile of the pair, one thread per query row:
//                   tcgen05.ld of the row's scores, running max and sum in float32 (base-2
//                   exponentials), P rounded to bfloat16 and written to shared memory in the
//                   layout of a K-major MMA operand, the output accumulator in TMEM rescaled by
//                   the change of the maximum;
//   O += P V        tcgen05.mma 128 x D x keys; V stays as the cache has it ([key][dim], the
//                   "MN-major" operand form), so nothing is transposed;
//   epilogue        O / sum -> bfloat16.
// The two tiles of the pair take turns: while group A works on the scores of a key tile, the
// tensor core computes those of group B, then A's P V while B is in its softmax, and so on -- the
// exponentials of one tile run under the matrix products of the other inside one block (one
// block per SM: 193 or 225 KB of shared memory, 384 or 512 TMEM columns).  Queries attend over the pages up to
// their own position (the step's own keys were written before), optionally within a window.
//
// Warp roles.  Head size 128 (352 threads): warp 0 TMA producer, warp 1 TMEM allocation + MMA issue for
// tile A, warps 2..5 softmax and epilogue of tile A, warps 6..9 of tile B (warp w owns TMEM lanes
// 32*(w%4)..+31), warp 10 MMA issue for tile B.
// Head size 64 (640 threads): the two halves of every 128-key tile are chains of their own, four
// chains per block.  A chain has its own score product (128 rows x 64 keys), its own softmax warps
// (one thread per query row and half), its own running maximum and sum, its own P.V product
// into its own accumulator in tensor memory (S of both tiles 256 columns, four accumulators of 64:
// all 512), and its own barriers; nothing in the loop makes one chain wait for another.  A row's two
// chains meet once, at the end: out = (2^(m0-M) O0 + 2^(m1-M) O1) / (2^(m0-M) l0 + 2^(m1-M) l1), the (m, l) pairs
// exchanged through shared memory with release / acquire and a bounded poll.  Warp 0 TMA, warps 1 and
// 2 MMA issue for tiles A and B, warps 4..11 softmax of tile A (4..7 the first 64 keys of a tile, 8..11
// the last 64), warps 12..19 of tile B.
// Waits are bounded as in the matrix product: a wait that gives up records a code in *status and
// the block drains.
//
// tiles[2j], tiles[2j+1] = {request row, first token index, rows, position of the first token};
// the second entry either continues the first (same request, first token and position + 128) or
// has rows == 0.
#include "tcgen05_utils.cuh"

namespace ptl {

constexpr int kTcRows = 128;       // query rows per tile of the pair
constexpr int kTcStagedPages = 264;    // block-table entries kept in shared memory (4,096 + 128 keys with pages of 16)
constexpr int kTcBarBytes = 256;
constexpr int kTcTmemCols = 512;   // S of A and B: columns 0..127, 128..255; O of A and B: 256.., 256 + D..
constexpr int kTcChunk = kTcRows * 128;                      // 128 rows of 64 bfloat16: one swizzled block of an operand

template <int D> struct PfCfg {
  static_assert(D == 64 || D == 128, "head size 64 or 128");
  static constexpr int kKeys = D == 64 ? 128 : 64;           // keys per tile
  static constexpr int kTileBytes = kKeys * D * 2;           // one of K / V: 16 KB
  static constexpr int kQBytes = kTcRows * D * 2;            // per tile of the pair: D / 64 blocks of [128 rows][128 B]
  static constexpr int kPBytes = kTcRows * kKeys * 2;        // per tile of the pair: kKeys / 64 blocks of [128 rows][128 B]
  // P of a tile of the pair lives in one buffer or in two that alternate: with two, the softmax of a
  // key tile does not have to wait for the P V product of the tile before it (which may still
  // stand in the tensor core's queue behind the other group's products), only for the one before that
  // (two where they fit: with head size 64 a P buffer is 32 KB, and two per tile would cost a K/V stage)
  static constexpr int kPBufs = D == 64 ? 1 : 2;
  // Chains per tile of the pair.  With head size 64 a key tile has 128 keys and one thread per row
  // spent 5,000 cycles on it, most of them on dependent chains and waits with two warps per scheduler
  // to hide them; the two halves of the tile as independent chains (see the top of the file) halve the
  // chains and double the warps.  With head size 128 (64 keys per tile; tensor memory and shared
  // memory have no room for more accumulators and the exchange) a tile stays one chain.
  static constexpr int kHalves = D == 64 ? 2 : 1;
  static constexpr int kSoftmaxWarp0 = kHalves == 2 ? 4 : 2;                 // first softmax warp (a multiple of 4 apart from the lane quarters' owners)
  static constexpr int kIssuerB = kHalves == 2 ? 2 : 10;                     // the warp that issues the MMAs of tile B (warp 1: of tile A)
  static constexpr int kThreads = kHalves == 2 ? 640 : 352;
  static constexpr int kStages = 3;                          // K/V tiles in flight
  // where the two chains of a row exchange their (maximum, sum) at the end
  static constexpr int kExchangeBytes = kHalves == 2 ? 2 * 2 * 2 * kTcRows * 8 : 0;   // [tile of the pair][buffer][half][row] x (value, sequence number)
  static constexpr int kSmem = 2 * kQBytes + kStages * 2 * kTileBytes + 2 * kPBufs * kPBytes + kTcBarBytes + kTcStagedPages * 4 + kExchangeBytes;
};

struct PrefillTcParams {
  __nv_bfloat16* out;
  const int* block_table;
  const int* tiles;
  int* status;
  int out_stride, bt_stride, nq, nkv, page_size, window, num_pages;
  float scale_log2;
};

// Barriers (8 bytes each): q_full, per tile of the pair s_full, s_free, p_full and o_done (one of each per P
// buffer), then kv_full[stages], kv_empty[stages].  P buffers have barriers of their own because a wait
// only tells the phases of a barrier apart by their parity: with one p_full for both buffers the softmax
// could hand over two tiles before the issuing thread, held up at a full tensor-core queue, looked
// again, and it would then wait for ever.
enum : int { kBarQ = 0, kBarSFull = 1, kBarSFree = 5, kBarPFull = 9, kBarODone = 13, kBarKvFull = 17 };

// the largest of three (one instruction on sm_100: a row maximum over 64 scores takes 32 of them, not 64)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(PfCfg<D>::kThreads)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const PrefillTcParams p) {
  using Cfg = PfCfg<D>;
  constexpr int kTcStages = Cfg::kStages, kBarKvEmpty = kBarKvFull + kTcStages, kBarCount = kBarKvEmpty + kTcStages;
  static_assert(kBarCount * 8 + 8 <= kTcBarBytes, "barriers, TMEM slot and abort flag fit their region");
  constexpr int kPB = Cfg::kPBufs;
  constexpr int kTcKeys = Cfg::kKeys, kTcD = D, kTcTileBytes = Cfg::kTileBytes, kTcQBytes = Cfg::kQBytes, kTcPBytes = Cfg::kPBytes;
  extern __shared__ __align__(1024) unsigned char smem[];     // swizzled tiles need 1024-byte alignment
  const uint32_t q_smem = smem_addr(smem);
  const uint32_t kv_smem = q_smem + 2 * kTcQBytes;
  const uint32_t p_smem = kv_smem + kTcStages * 2 * kTcTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * kTcQBytes + kTcStages * 2 * kTcTileBytes + 2 * kPB * kTcPBytes);
  const uint32_t bar_base = smem_addr(bars);
  auto bar = [&](int i) { return bar_base + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBarCount);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_pages = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(bars) + kTcBarBytes);
  unsigned long long* s_xchg = reinterpret_cast<unsigned long long*>(s_pages + kTcStagedPages);      // two threads per row: their maxima and sums meet here
  constexpr int kHalves = Cfg::kHalves;
  if (q_smem & 1023u) {                                        // never expected; refuse rather than compute garbage
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 99);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Blocks are handed out with x running fastest: heads along x and pairs along y, last pair
  // first, start the pairs that see the most keys first on every SM (longest work first).
  const int pair = gridDim.y - 1 - blockIdx.y;
  const int* tl = p.tiles + 8 * pair;
  const int req = tl[0], tok0 = tl[1], pos0 = tl[3];
  const int rows_g[2] = {tl[2], tl[6]};                        // rows of tile A and of tile B (0: absent)
  if (rows_g[0] <= 0 && rows_g[1] <= 0) return;                // an empty pair (padding of a captured step): nothing to do, nothing allocated yet
  const int h = blockIdx.x;
  const int kvh = h / (p.nq / p.nkv);
  // Per tile of the pair: first key it may see (window), one past the last, and the range of key
  // tiles it takes part in.  Key tiles are counted from tile A's first page.
  int lo_raw[2], k_end[2], t_first[2], t_last[2], pos_g[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    pos_g[g] = pos0 + g * kTcRows;
    lo_raw[g] = (p.window > 0 && pos_g[g] - p.window + 1 > 0) ? pos_g[g] - p.window + 1 : 0;
    k_end[g] = pos_g[g] + rows_g[g];
  }
  const int k_base = lo_raw[0] / p.page_size * p.page_size;    // tiles start on a page boundary
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    t_first[g] = (lo_raw[g] - k_base) / kTcKeys;
    t_last[g] = rows_g[g] > 0 ? (k_end[g] - k_base + kTcKeys - 1) / kTcKeys : 0;     // one past the last
  }
  const int ntiles = max(t_last[0], t_last[1]);
  const int pages_per_tile = kTcKeys / p.page_size;
  const int* bt_global = p.block_table + (size_t)req * p.bt_stride;
  auto takes_part = [&](int g, int t) { return rows_g[g] > 0 && t >= t_first[g] && t < t_last[g]; };

  if (threadIdx.x == 0) {
    mbar_init(bar(kBarQ), 1);
    for (int s = 0; s < kTcStages; ++s) { mbar_init(bar(kBarKvFull + s), 1); mbar_init(bar(kBarKvEmpty + s), rows_g[1] > 0 ? 2 : 1); }
    for (int g = 0; g < 2; ++g) {
      for (int b = 0; b < 2; ++b) { mbar_init(bar(kBarSFull + 2 * g + b), 1); mbar_init(bar(kBarSFree + 2 * g + b), 4); }
      // (head size 128: b is the P buffer; head size 64: b is the half of the key tile, a chain of its own)
      for (int b = 0; b < 2; ++b) { mbar_init(bar(kBarPFull + 2 * g + b), 4); mbar_init(bar(kBarODone + 2 * g + b), 1); }
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTcTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();                 // everything below reads what earlier kernels of the step wrote
  pdl_launch_dependents();
  // block-table entries of the key range, staged once (the producer thread reads them)
  const int first_block = k_base / p.page_size;
  const int n_blocks = ntiles * pages_per_tile;
  // entries that exist for this request: up to the last key of the tiles that are there (an absent tile B has no
  // keys of its own: counting its would-be range read up to eight entries past the request's, and past the
  // table's row where the table is only as wide as the step needs), and never past the row
  const int last_key = max(rows_g[0] > 0 ? k_end[0] : 0, rows_g[1] > 0 ? k_end[1] : 0) - 1;
  const int have_blocks = min(last_key / p.page_size + 1, p.bt_stride) - first_block;
  const bool staged = n_blocks <= kTcStagedPages;
  if (staged)
    for (int i = threadIdx.x; i < n_blocks; i += Cfg::kThreads) s_pages[i] = i < have_blocks ? bt_global[first_block + i] : -1;
  for (int i = threadIdx.x; i < Cfg::kExchangeBytes / 8; i += Cfg::kThreads) s_xchg[i] = 0ull;      // sequence numbers start at 0
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The two kinds of product, as the issuing threads call them.
  constexpr uint32_t idesc_s = instr_desc_bf16(kTcRows, kTcKeys);                    // Q, K both K-major
  constexpr uint32_t idesc_o = instr_desc_bf16(kTcRows, kTcD) | (1u << 16);          // V is MN-major
  auto stage_of = [&](int t) { return t % kTcStages; };
  auto issue_s = [&](int g, int t) {
    const uint32_t kb = kv_smem + stage_of(t) * 2 * kTcTileBytes;
#pragma unroll
    for (int k = 0; k < kTcD / 16; ++k)       // 16 values of the head per step: block k / 4 of the operands, 32 bytes along its rows
      tcgen05_mma_bf16(tmem_base + g * kTcRows, smem_desc_sw128(q_smem + g * kTcQBytes + (k >> 2) * kTcChunk + (k & 3) * 32),
                       smem_desc_sw128(kb + (k >> 2) * (kTcKeys * 128) + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
    tcgen05_commit(bar(kBarSFull + 2 * g));                       // S of this tile complete
  };
  // Head size 64: the scores of each half of a key tile are a product of their own (64 keys), with
  // barriers of their own, so that the two halves are chains that do not wait for one another.
  constexpr uint32_t idesc_s_half = instr_desc_bf16(kTcRows, 64);
  auto issue_s_half = [&](int g, int hf, int t) {
    const uint32_t kb = kv_smem + stage_of(t) * 2 * kTcTileBytes + hf * (64 * 128);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      tcgen05_mma_bf16(tmem_base + g * kTcRows + hf * 64, smem_desc_sw128(q_smem + g * kTcQBytes + k * 32),
                       smem_desc_sw128(kb + k * 32), idesc_s_half, k > 0 ? 1u : 0u);
    tcgen05_commit(bar(kBarSFull + 2 * g + hf));
  };
  auto issue_pv = [&](int g, int t, int n_pv) {                    // n_pv: how many of the group's products came before
    const uint32_t vb = kv_smem + stage_of(t) * 2 * kTcTileBytes + kTcTileBytes;
#pragma unroll
    for (int k = 0; k < kTcKeys / 16; ++k) {
      // A: P, K-major, 64-key blocks of 16 KB; B: V rows = keys, 16 keys = 2 KB per step, and with
      // head size 128 a second block of 64 values per row, one K/V block further on
      const uint64_t adesc = smem_desc_sw128(p_smem + (g * kPB + n_pv % kPB) * kTcPBytes + (k >> 2) * kTcChunk + (k & 3) * 32);
      const uint64_t bdesc = kTcD == 64 ? smem_desc_sw128(vb + k * 2048) : smem_desc_sw128_mn(vb + k * 2048, kTcKeys * 128);
      tcgen05_mma_bf16(tmem_base + 2 * kTcRows + g * kTcD, adesc, bdesc, idesc_o, (n_pv > 0 || k > 0) ? 1u : 0u);
    }
    tcgen05_commit(bar(kBarODone + 2 * g + n_pv % kPB));          // O of this tile updated, its P buffer free
  };
  // Head size 64: the two halves of a key tile are chains of their own.  Half hf of tile t: P of its
  // 64 keys (block hf of the group's P buffer) times the values of those keys, into the half's own accumulator.
  auto issue_pv_half = [&](int g, int hf, int t, int n_pv) {
    const uint32_t vb = kv_smem + stage_of(t) * 2 * kTcTileBytes + kTcTileBytes + hf * (64 * 128);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      tcgen05_mma_bf16(tmem_base + 2 * kTcRows + (g * 2 + hf) * 64, smem_desc_sw128(p_smem + g * kTcPBytes + hf * kTcChunk + k * 32),
                       smem_desc_sw128(vb + k * 2048), idesc_o, (n_pv > 0 || k > 0) ? 1u : 0u);
    tcgen05_commit(bar(kBarODone + 2 * g + hf));
  };

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    mbar_expect_tx(bar(kBarQ), (rows_g[1] > 0 ? 2 : 1) * kTcQBytes);
#pragma unroll
    for (int c = 0; c < kTcD / 64; ++c) {                          // 64 values of every row at a time
      tma_load_2d(q_smem + c * kTcChunk, &map_q, bar(kBarQ), h * kTcD + c * 64, tok0);     // rows past the step's tokens arrive as zeros
      if (rows_g[1] > 0) tma_load_2d(q_smem + kTcQBytes + c * kTcChunk, &map_q, bar(kBarQ), h * kTcD + c * 64, tok0 + kTcRows);
    }
    const int rows_per_page_group = p.nkv * p.page_size;           // cache rows between the k and v planes of a page
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % kTcStages;
      const uint32_t ph = (t / kTcStages) & 1;
      if (!mbar_wait(bar(kBarKvEmpty + s), ph ^ 1, abort_flag, p.status, 11)) break;
      mbar_expect_tx(bar(kBarKvFull + s), 2 * kTcTileBytes);
      const uint32_t kdst = kv_smem + s * 2 * kTcTileBytes, vdst = kdst + kTcTileBytes;
      for (int i = 0; i < pages_per_tile; ++i) {
        const int bi = t * pages_per_tile + i;
        int page = staged ? s_pages[bi] : (bi < have_blocks ? bt_global[first_block + bi] : -1);
        if (page < 0 || page >= p.num_pages) page = 0;             // beyond the request: any page, its keys get masked
        const int krow = (page * 2 * p.nkv + kvh) * p.page_size;
        const uint32_t off = (uint32_t)i * p.page_size * 128u;
#pragma unroll
        for (int c = 0; c < kTcD / 64; ++c) {
          tma_load_2d(kdst + c * (kTcKeys * 128) + off, &map_kv, bar(kBarKvFull + s), c * 64, krow);
          tma_load_2d(vdst + c * (kTcKeys * 128) + off, &map_kv, bar(kBarKvFull + s), c * 64, krow + rows_per_page_group);
        }
      }
    }
  } else if ((warp == 1 || warp == Cfg::kIssuerB) && lane == 0) {
    // ------------------------------------------------------------ MMA issuers, one per tile of the pair
    // (A thread that issues MMAs is held up by every MMA, about as long as it runs, and by every look
    // at a barrier after one, a couple of hundred cycles: one thread for both tiles was what the
    // softmax groups ended up waiting for.  Four threads, the scores and the P V products of each
    // tile apart, were no faster than two.)
    const int g = warp == 1 ? 0 : 1;
    bool ok = rows_g[g] > 0 && mbar_wait(bar(kBarQ), 0, abort_flag, p.status, 12);
    int n_pv = 0;                                                 // P V products issued so far
    // The scores of the group's next key tile are issued as soon as the group has taken the previous
    // ones out of TMEM (s_free), long before its softmax is done, so that it does not wait for its
    // scores; its P V product follows when it hands over P.  Barriers are tested without suspending.
    // A key tile's stage is given back by both issuers (where both tiles of the pair exist): each
    // arrives once it has seen the tile arrive and has issued its product on it, if it has one --
    // having seen it, it cannot arrive for the stage's next filling too early.
    int next_s = t_first[g], next_pv = t_first[g];
    int pv_half[2] = {0, 0}, s_half[2] = {0, 0};
    int kv_ready = 0, released = 0;
    uint32_t idle = 0;
    while (ok && released < ntiles) {
      bool progress = false;
      if (kv_ready < ntiles && mbar_test_wait(bar(kBarKvFull + stage_of(kv_ready)), (kv_ready / kTcStages) & 1)) {
        ++kv_ready;
        progress = true;
      }
      const int issued = next_s - t_first[g];
      if (kHalves == 2) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int t_next = t_first[g] + s_half[hf];             // the half's next key tile
          if (t_next < t_last[g] && t_next < kv_ready &&
              (s_half[hf] == 0 || mbar_test_wait(bar(kBarSFree + 2 * g + hf), (s_half[hf] - 1) & 1))) {
            tcgen05_fence_after();
            issue_s_half(g, hf, t_next);
            ++s_half[hf];
            progress = true;
          }
        }
        next_s = t_first[g] + min(s_half[0], s_half[1]);
      } else if (next_s < t_last[g] && next_s < kv_ready && (issued == 0 || mbar_test_wait(bar(kBarSFree + 2 * g), (issued - 1) & 1))) {
        tcgen05_fence_after();
        issue_s(g, next_s);
        ++next_s;
        progress = true;
      }
      if (kHalves == 2) {
        // each half hands over its P and gets its product by itself
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int done = pv_half[hf];                           // products of this half so far
          if (done < s_half[hf] && mbar_test_wait(bar(kBarPFull + 2 * g + hf), done & 1)) {
            tcgen05_fence_after();
            issue_pv_half(g, hf, t_first[g] + done, done);
            ++pv_half[hf];
            progress = true;
          }
        }
        next_pv = t_first[g] + min(pv_half[0], pv_half[1]);       // key tiles that both halves are through with
      } else if (next_pv < next_s && mbar_test_wait(bar(kBarPFull + 2 * g + n_pv % kPB), (n_pv / kPB) & 1)) {     // P written, O rescaled
        tcgen05_fence_after();
        issue_pv(g, next_pv, n_pv);
        ++n_pv;
        ++next_pv;
        progress = true;
      }
      while (released < kv_ready && (!takes_part(g, released) || next_pv > released)) {
        tcgen05_commit(bar(kBarKvEmpty + stage_of(released)));
        ++released;
        progress = true;
      }
      if (progress) {
        idle = 0;
      } else if (*abort_flag || ++idle > kPollLimit) {
        if (!*abort_flag) { *abort_flag = 1; if (p.status) atomicExch(p.status, 14); }
        ok = false;
      } else if (idle > 256) {
        __nanosleep(32);
      }
    }
  } else if (warp >= Cfg::kSoftmaxWarp0 && warp < Cfg::kSoftmaxWarp0 + 8 * kHalves) {
    // ------------------------------------------------------------ softmax, correction, epilogue
    const int sw = warp - Cfg::kSoftmaxWarp0;
    const int g = sw / (4 * kHalves);                             // which tile of the pair
    const int hf = kHalves == 2 ? (sw >> 2) & 1 : 0;              // which half of a key tile's columns (two threads per row)
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                               // query row of this thread within its tile
    constexpr int kMyKeys = kTcKeys / kHalves;                    // keys of a tile that this thread takes
    constexpr int kMyD = kTcD / kHalves;                          // columns of the output that it writes
    const int col0 = hf * kMyKeys, d0 = hf * kMyD;
    // With two threads per row each is a chain of its own: its own running maximum and sum, its
    // own accumulator in tensor memory (its half's P times its half's values), its own hand-over
    // barriers (slot b of the P barriers = the half); the two meet once, at the end.
    const int pb = kHalves == 2 ? hf : 0;                         // this thread's P / O barrier pair when the halves are chains
    // The two threads of a row exchange a value through shared memory: each stores (value, sequence
    // number) with release semantics and polls the other's slot until it carries the same number
    // (bounded, and it gives up when the block aborts: no barrier that a drained partner would miss).
    // Every exchange has a buffer and a sequence number of its own.
    const uint32_t xchg = smem_addr(s_xchg + g * (2 * 2 * kTcRows));          // [buffer][half][row]
    auto exchange = [&](int buf, float mine, uint32_t seq, float& theirs) -> bool {
      const uint32_t my_slot = xchg + 8u * ((buf * 2 + hf) * kTcRows + r), other = xchg + 8u * ((buf * 2 + (hf ^ 1)) * kTcRows + r);
      const unsigned long long word = ((unsigned long long)seq << 32) | __float_as_uint(mine);
      asm volatile("st.release.cta.shared.b64 [%0], %1;" ::"r"(my_slot), "l"(word) : "memory");
      for (uint32_t i = 0; i < kPollLimit; ++i) {
        unsigned long long got;
        asm volatile("ld.acquire.cta.shared.b64 %0, [%1];" : "=l"(got) : "r"(other) : "memory");
        if ((uint32_t)(got >> 32) == seq) { theirs = __uint_as_float((uint32_t)got); return true; }
        if (*abort_flag) return false;
      }
      *abort_flag = 1;
      if (p.status) atomicExch(p.status, 19);
      return false;
    };
    const int rows = rows_g[g];
    const int tile_pos0 = pos_g[g];
    const int qpos = tile_pos0 + r;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t tmem_s = tmem_base + g * kTcRows;
    const uint32_t tmem_o = tmem_base + 2 * kTcRows + (kHalves == 2 ? (g * 2 + hf) * 64 : g * kTcD);
    const uint32_t my_p0 = p_smem + g * kPB * kTcPBytes;
    // the P V product of this group's i-th key tile is complete (barrier of the P buffer it read, that buffer's (i / kPB)-th use)
    auto wait_pv = [&](int i, int code) {
      if (kHalves == 2) return mbar_wait(bar(kBarODone + 2 * g + pb), i & 1, abort_flag, p.status, code);
      return mbar_wait(bar(kBarODone + 2 * g + i % kPB), (i / kPB) & 1, abort_flag, p.status, code);
    };
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    int n = 0;                                                    // key tiles taken so far
    for (int t = t_first[g]; t < t_last[g] && ok; ++t, ++n) {
      ok = mbar_wait(bar(kBarSFull + 2 * g + pb), n & 1, abort_flag, p.status, 15);
      if (!ok) break;
      tcgen05_fence_after();
      const int key0 = k_base + t * kTcKeys;
      const bool need_mask = key0 + kTcKeys - 1 > tile_pos0 || key0 < lo_raw[g] ||
                             (p.window > 0 && key0 < tile_pos0 + kTcRows - 1 - p.window + 1);
      // the row's scores come out of TMEM once and stay in registers
      uint32_t v[kMyKeys];
#pragma unroll
      for (int c0 = 0; c0 < kMyKeys; c0 += 32) tmem_load_32_nowait(tmem_s + lane_addr + col0 + c0, v + c0);
      tmem_wait_ld();
      // the scores are in registers: the next key tile's may be written
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarSFree + 2 * g + pb));
      // the row maximum over eight running maxima: one chain of dependent comparisons over all keys
      // of the tile was a fifth of this thread's time per tile
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < kMyKeys; ++j) {
          const int key = key0 + col0 + j;
          float x = __uint_as_float(v[j]);
          if (key > qpos || (p.window > 0 && key < qpos - p.window + 1)) x = -INFINITY;
          v[j] = __float_as_uint(x);
          mx8[j & 7] = fmaxf(mx8[j & 7], x);
        }
      } else {
#pragma unroll
        for (int j = 0; j < kMyKeys; j += 2) mx8[(j >> 1) & 7] = max3(mx8[(j >> 1) & 7], __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
      }
      float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      mx *= p.scale_log2;                                       // the scale is positive: max and scaling commute
      // The reference maximum only moves when the row's maximum has grown by more than 8 (a factor of
      // 256 in P, which bfloat16 and the float32 sums take): rescaling the accumulator becomes rare.
      const float m_top = fmaxf(m_run, mx);
      const bool moved = m_top > m_run + 8.0f;
      const float m_new = moved ? m_top : m_run;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = moved ? ex2_approx(m_run - m_use) : 1.0f;
      // the P V product that read this P buffer last must be complete before it is overwritten
      if (n >= kPB) {
        ok = wait_pv(n - kPB, 16);
        if (!ok) break;
        tcgen05_fence_after();
      }
      const uint32_t my_p = my_p0 + (n % kPB) * kTcPBytes;
      // P = 2^(s * scale - m) as bfloat16 into shared memory (K-major operand layout), row sum
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c0 = 0; c0 < kMyKeys; c0 += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(v[c0 + j]), p.scale_log2, -m_use));
          const float p1 = ex2_approx(fmaf(__uint_as_float(v[c0 + j + 1]), p.scale_log2, -m_use));
          sum4[j >> 1] += p0 + p1;
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          packed[j >> 1] = *reinterpret_cast<uint32_t*>(&pk);
        }
        // keys kc..kc+7 of the tile are 16-byte chunk (kc % 64) / 8 of this row inside 64-key block kc / 64
        const int kc = col0 + c0;
        const uint32_t dst = my_p + (kc >> 6) * kTcChunk + r * 128 + (((((kc & 63) >> 3)) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(packed[0]), "r"(packed[1]), "r"(packed[2]),
                     "r"(packed[3]) : "memory");
      }
      l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      m_run = m_new;
      // rescale the output accumulator where the maximum moved (never on the first tile: O is overwritten there)
      if (n > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
        if (kPB > 1) {                                              // (every P V product so far must have landed in O)
          ok = wait_pv(n - 1, 18);
          if (!ok) break;
          tcgen05_fence_after();
        }
#pragma unroll 1
        for (int c0 = 0; c0 < kTcD; c0 += 32) {                  // (with two chains per row: the chain's own 64 columns)
          uint32_t o[32];
          tmem_load_32(tmem_o + lane_addr + c0, o);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_store_32(tmem_o + lane_addr + c0, o);
        }
      }
      // make the generic-proxy writes of P visible to the tensor core, then hand over
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPFull + 2 * g + (kHalves == 2 ? pb : n % kPB)));
    }
    // epilogue: wait for the last P V product, then O / sum
    if (ok && n > 0) ok = wait_pv(n - 1, 17);
    if (kHalves == 2) {
      // The row's two chains meet: with M the larger of their reference maxima,
      // out = (2^(m0 - M) O0 + 2^(m1 - M) O1) / (2^(m0 - M) l0 + 2^(m1 - M) l1).  Each thread sends its
      // (m, l), takes the other's, waits for the other chain's last product and writes 32 of the 64 columns.
      float m_other = -INFINITY, l_other = 0.f;
      if (ok) ok = exchange(0, m_run, 0x80000001u, m_other);
      if (ok) ok = exchange(1, l_run, 0x80000002u, l_other);
      if (ok && n > 0) ok = mbar_wait(bar(kBarODone + 2 * g + (hf ^ 1)), (n - 1) & 1, abort_flag, p.status, 21);
      if (ok && n > 0) {
        tcgen05_fence_after();
        const float m_all = fmaxf(m_run, m_other);
        const float w_mine = m_run == -INFINITY ? 0.f : ex2_approx(m_run - m_all);
        const float w_other = m_other == -INFINITY ? 0.f : ex2_approx(m_other - m_all);
        const float w0 = hf == 0 ? w_mine : w_other, w1 = hf == 0 ? w_other : w_mine;       // of chain 0 and chain 1, the same in both threads
        const float l0 = hf == 0 ? l_run : l_other, l1 = hf == 0 ? l_other : l_run;
        const float l_all = w0 * l0 + w1 * l1;
        const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
        const float f0 = w0 * inv, f1 = w1 * inv;
        const uint32_t acc0 = tmem_base + 2 * kTcRows + (g * 2) * 64 + lane_addr + d0;
        uint32_t a[32], b[32];
        tmem_load_32_nowait(acc0, a);
        tmem_load_32_nowait(acc0 + 64, b);
        tmem_wait_ld();
        if (r < rows) {
          __nv_bfloat16* dst = p.out + (size_t)(tok0 + g * kTcRows + r) * p.out_stride + (size_t)h * kTcD + d0;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 pk;
            uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int e = 8 * q4 + 2 * j;
              __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(a[e]) * f0 + __uint_as_float(b[e]) * f1,
                                                        __uint_as_float(a[e + 1]) * f0 + __uint_as_float(b[e + 1]) * f1);
              w[j] = *reinterpret_cast<uint32_t*>(&t2);
            }
            *reinterpret_cast<uint4*>(dst + 8 * q4) = pk;
          }
        }
      }
    } else if (ok && n > 0) {
      tcgen05_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kTcD; c0 += 32) {
        uint32_t v[32];
        tmem_load_32(tmem_o + lane_addr + c0, v);
        if (r < rows) {
          __nv_bfloat16* dst = p.out + (size_t)(tok0 + g * kTcRows + r) * p.out_stride + (size_t)h * kTcD + c0;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 pk;
            uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[8 * q4 + 2 * j]) * inv, __uint_as_float(v[8 * q4 + 2 * j + 1]) * inv);
              w[j] = *reinterpret_cast<uint32_t*>(&t2);
            }
            *reinterpret_cast<uint4*>(dst + 8 * q4) = pk;
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTcTmemCols) : "memory");
  }
}

}  // namespace ptl

namespace ptl {

template <int D>
static int launch_prefill_tc(const void* q, const void* cache, int n_tiles, int n_tokens, int q_stride, int nq, int nkv,
                             int page_size, int num_pages, const PrefillTcParams& p, cudaStream_t stream) {
  using Cfg = PfCfg<D>;
  static SmemRaised raised = {};
  if (int rc = raise_shared_memory("prefill_attention_tc", prefill_attention_tc_kernel<D>, Cfg::kSmem, raised)) return rc;
  CUtensorMap mq, mkv;
  int rc = make_map(&mq, q, n_tokens, q_stride, kTcRows);                 // whole step: [tokens, q_stride], boxes of 64 x 128
  if (rc) return rc;
  rc = make_map(&mkv, cache, num_pages * 2 * nkv * page_size, D, page_size);     // cache as rows of one head's D values, boxes of 64 x page
  if (rc) return rc;
  return launch_kernel("prefill_attention_tc", prefill_attention_tc_kernel<D>, dim3(nq, n_tiles / 2), dim3(Cfg::kThreads), Cfg::kSmem,
                       stream, mq, mkv, p);
}

}  // namespace ptl

// Returns 0 on success; -2 if this kernel does not take the sizes (the caller then uses the
// warp-level kernel): head size 64 or 128 only, pages of 8 keys or more that divide the key tile
// (128 keys with head size 64, 64 with 128), 16-byte aligned rows; -1 on an error.  `tiles` holds
// n_tiles entries in pairs (n_tiles is even): see the top of the file.
PTL_EXPORT int ptl_prefill_attention_tc_bf16(void* out, const void* q, const void* cache, const int* block_table,
                                             const int* tiles, int n_tiles, int n_tokens, int q_stride, int out_stride,
                                             int bt_stride, int nq, int nkv, int d, int page_size, float scale,
                                             int window, int num_pages, int* status, void* stream) {
  using namespace ptl;
  PTL_REQUIRE(n_tiles >= 0 && nq > 0 && nkv > 0 && page_size > 0 && num_pages > 0, "prefill_attention_tc: bad sizes");
  PTL_REQUIRE(n_tiles % 2 == 0, "prefill_attention_tc: tiles come in pairs, %d is odd", n_tiles);
  PTL_REQUIRE(nq % nkv == 0, "prefill_attention_tc: %d query heads are no multiple of %d kv heads", nq, nkv);
  if (d != 64 && d != 128) return -2;
  const int keys = d == 64 ? PfCfg<64>::kKeys : PfCfg<128>::kKeys;
  if (page_size < 8 || page_size > keys || keys % page_size != 0 || q_stride % 8 != 0 || out_stride % 8 != 0 || n_tiles / 2 > 65535)
    return -2;
  PTL_REQUIRE(aligned16(q) && aligned16(cache) && aligned16(out), "prefill_attention_tc: q, cache and out must be 16-byte aligned");
  if (n_tiles == 0) return 0;
  PrefillTcParams p{};
  p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.tiles = tiles; p.status = status;
  p.out_stride = out_stride; p.bt_stride = bt_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size;
  p.window = window; p.num_pages = num_pages; p.scale_log2 = scale * 1.4426950408889634f;
  if (d == 64) return launch_prefill_tc<64>(q, cache, n_tiles, n_tokens, q_stride, nq, nkv, page_size, num_pages, p, as_stream(stream));
  return launch_prefill_tc<128>(q, cache, n_tiles, n_tokens, q_stride, nq, nkv, page_size, num_pages, p, as_stream(stream));
}
