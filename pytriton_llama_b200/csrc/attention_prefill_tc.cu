// Attention of prompt portions over the paged cache on the fifth-generation tensor cores
// (head size 64, bfloat16).  One block per (tile of up to 128 query tokens of one request, query
// head):
//   S = Q K^T       tcgen05.mma 128 x 128 x 64 into TMEM (float32), K tile fetched page by page
//                   with TMA into 128-byte-swizzled shared memory;
//   softmax         four warps, one thread per query row: tcgen05.ld of the row's 128 scores,
//                   running max and sum in float32 (base-2 exponentials), P rounded to bfloat16
//                   and written to shared memory in the layout of a K-major MMA operand, the
//                   output accumulator in TMEM rescaled by the change of the maximum;
//   O += P V        tcgen05.mma 128 x 64 x 128; V stays as the cache has it ([key][dim], the
//                   "MN-major" operand form), so nothing is transposed;
//   epilogue        O / sum -> bfloat16.
// Two blocks fit on an SM (112 KB of shared memory, 256 TMEM columns each), so one block's
// softmax runs under the other's MMAs.  Queries attend over the pages up to their own position
// (the step's own keys were written before), optionally within a window.
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 TMEM allocation + MMA issue, warps 2..5
// softmax and epilogue (warp w owns TMEM lanes 32*(w%4)..+31).  Waits are bounded as in the
// matrix product: a wait that gives up records a code in *status and the block drains.
#include "tcgen05_utils.cuh"

namespace ptl {

constexpr int kTcRows = 128;       // query rows per block
constexpr int kTcKeys = 128;       // keys per tile
constexpr int kTcD = 64;           // head size
constexpr int kTcThreads = 192;
constexpr int kTcStages = 2;
constexpr int kTcTileBytes = kTcKeys * kTcD * 2;           // one of K / V: 16 KB
constexpr int kTcQBytes = kTcRows * kTcD * 2;              // 16 KB
constexpr int kTcPBytes = kTcRows * kTcKeys * 2;           // 32 KB: two 64-key blocks of [128 rows][128 B]
constexpr int kTcStagedPages = 128;    // block-table entries kept in shared memory (2,048 keys with pages of 16)
// Two blocks per SM need each to stay below ~113 KB: tiles, 128 bytes of barriers, the staged table.
constexpr int kTcSmem = kTcQBytes + kTcStages * 2 * kTcTileBytes + kTcPBytes + 128 + kTcStagedPages * 4;
constexpr int kTcTmemCols = 256;   // S: columns 0..127, O: columns 128..191

struct PrefillTcParams {
  __nv_bfloat16* out;
  const int* block_table;
  const int* tiles;          // {request row, first token, rows, first position} per block
  int* status;
  int out_stride, bt_stride, nq, nkv, page_size, window, num_pages;
  float scale_log2;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kTcThreads)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const PrefillTcParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];     // swizzled tiles need 1024-byte alignment
  const uint32_t q_smem = smem_addr(smem);
  const uint32_t kv_smem = q_smem + kTcQBytes;
  const uint32_t p_smem = kv_smem + kTcStages * 2 * kTcTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTcQBytes + kTcStages * 2 * kTcTileBytes + kTcPBytes);
  // bars: 0 q_full | 1,2 kv_full | 3,4 kv_empty | 5 s_full | 6 p_full | 7 o_done
  const uint32_t bar_base = smem_addr(bars);
  auto bar = [&](int i) { return bar_base + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_pages = reinterpret_cast<int*>(bars + 16);
  if (q_smem & 1023u) {                                        // never expected; refuse rather than compute garbage
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 99);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* tl = p.tiles + 4 * (gridDim.x - 1 - blockIdx.x);     // later tiles see more keys: start them first
  const int req = tl[0], tok0 = tl[1], rows = tl[2], pos0 = tl[3];
  const int h = blockIdx.y;
  const int kvh = h / (p.nq / p.nkv);
  const int k_lo_raw = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int k_lo = k_lo_raw / p.page_size * p.page_size;        // tiles start on a page boundary
  const int k_end = pos0 + rows;
  const int ntiles = (k_end - k_lo + kTcKeys - 1) / kTcKeys;
  const int pages_per_tile = kTcKeys / p.page_size;
  const int* bt_global = p.block_table + (size_t)req * p.bt_stride;

  if (threadIdx.x == 0) {
    mbar_init(bar(0), 1);
    for (int s = 0; s < kTcStages; ++s) { mbar_init(bar(1 + s), 1); mbar_init(bar(3 + s), 1); }
    mbar_init(bar(5), 1);
    mbar_init(bar(6), 4);
    mbar_init(bar(7), 1);
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
  const int first_block = k_lo / p.page_size;
  const int n_blocks = ntiles * pages_per_tile;
  const int have_blocks = (k_end - 1) / p.page_size - first_block + 1;     // entries that exist for this request
  const bool staged = n_blocks <= kTcStagedPages;
  if (staged)
    for (int i = threadIdx.x; i < n_blocks; i += kTcThreads) s_pages[i] = i < have_blocks ? bt_global[first_block + i] : -1;
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    mbar_expect_tx(bar(0), kTcQBytes);
    tma_load_2d(q_smem, &map_q, bar(0), h * kTcD, tok0);           // rows past the step's tokens arrive as zeros
    const int rows_per_page_group = p.nkv * p.page_size;           // cache rows between the k and v planes of a page
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % kTcStages;
      const uint32_t ph = (t / kTcStages) & 1;
      if (!mbar_wait(bar(3 + s), ph ^ 1, abort_flag, p.status, 11)) break;
      mbar_expect_tx(bar(1 + s), 2 * kTcTileBytes);
      const uint32_t kdst = kv_smem + s * 2 * kTcTileBytes, vdst = kdst + kTcTileBytes;
      for (int i = 0; i < pages_per_tile; ++i) {
        const int bi = t * pages_per_tile + i;
        int page = staged ? s_pages[bi] : (bi < have_blocks ? bt_global[first_block + bi] : -1);
        if (page < 0 || page >= p.num_pages) page = 0;             // beyond the request: any page, its keys get masked
        const int krow = (page * 2 * p.nkv + kvh) * p.page_size;
        const uint32_t off = (uint32_t)i * p.page_size * 128u;
        tma_load_2d(kdst + off, &map_kv, bar(1 + s), 0, krow);
        tma_load_2d(vdst + off, &map_kv, bar(1 + s), 0, krow + rows_per_page_group);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = instr_desc_bf16(kTcRows, kTcKeys);                    // Q, K both K-major
    constexpr uint32_t idesc_o = instr_desc_bf16(kTcRows, kTcD) | (1u << 16);          // V is MN-major
    bool ok = mbar_wait(bar(0), 0, abort_flag, p.status, 12);
    for (int t = 0; t < ntiles && ok; ++t) {
      const int s = t % kTcStages;
      const uint32_t ph = (t / kTcStages) & 1;
      ok = mbar_wait(bar(1 + s), ph, abort_flag, p.status, 13);
      if (!ok) break;
      // the previous tile's softmax has read S (it arrives on p_full only after that), so S is free
      tcgen05_fence_after();
      const uint32_t kb = kv_smem + s * 2 * kTcTileBytes, vb = kb + kTcTileBytes;
#pragma unroll
      for (int k = 0; k < kTcD / 16; ++k)
        tcgen05_mma_bf16(tmem_s, smem_desc_sw128(q_smem + k * 32), smem_desc_sw128(kb + k * 32), idesc_s, k > 0 ? 1u : 0u);
      tcgen05_commit(bar(5));                                     // S complete
      ok = mbar_wait(bar(6), t & 1, abort_flag, p.status, 14);   // P written, O rescaled
      if (!ok) break;
      tcgen05_fence_after();
#pragma unroll
      for (int k = 0; k < kTcKeys / 16; ++k) {
        // A: P, K-major, 64-key blocks of 16 KB; B: V rows = keys, 16 keys = 2 KB per step
        const uint64_t adesc = smem_desc_sw128(p_smem + (k >> 2) * (kTcRows * 128) + (k & 3) * 32);
        const uint64_t bdesc = smem_desc_sw128(vb + k * 2048);
        tcgen05_mma_bf16(tmem_o, adesc, bdesc, idesc_o, (t > 0 || k > 0) ? 1u : 0u);
      }
      tcgen05_commit(bar(3 + s));                                 // K/V stage free
      tcgen05_commit(bar(7));                                     // O updated, P free
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ softmax, correction, epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                               // query row of this thread
    const int qpos = pos0 + r;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
      ok = mbar_wait(bar(5), t & 1, abort_flag, p.status, 15);
      if (!ok) break;
      tcgen05_fence_after();
      const int key0 = k_lo + t * kTcKeys;
      const bool need_mask = key0 + kTcKeys - 1 > pos0 || key0 < k_lo_raw ||
                             (p.window > 0 && key0 < pos0 + kTcRows - 1 - p.window + 1);
      // the row's 128 scores come out of TMEM once and stay in registers
      uint32_t v[kTcKeys];
#pragma unroll
      for (int c0 = 0; c0 < kTcKeys; c0 += 32) tmem_load_32_nowait(tmem_s + lane_addr + c0, v + c0);
      tmem_wait_ld();
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < kTcKeys; ++j) {
          const int key = key0 + j;
          float x = __uint_as_float(v[j]);
          if (key > qpos || (p.window > 0 && key < qpos - p.window + 1)) x = -INFINITY;
          v[j] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      } else {
#pragma unroll
        for (int j = 0; j < kTcKeys; ++j) mx = fmaxf(mx, __uint_as_float(v[j]));
      }
      mx *= p.scale_log2;                                       // the scale is positive: max and scaling commute
      const float m_new = fmaxf(m_run, mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = ex2_approx(m_run - m_use);
      // the previous P V product must be complete before P is overwritten and O rescaled
      if (t > 0) {
        ok = mbar_wait(bar(7), (t - 1) & 1, abort_flag, p.status, 16);
        if (!ok) break;
        tcgen05_fence_after();
      }
      // P = 2^(s * scale - m) as bfloat16 into shared memory (K-major operand layout), row sum
      float sum = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < kTcKeys; c0 += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(v[c0 + j]), p.scale_log2, -m_use));
          const float p1 = ex2_approx(fmaf(__uint_as_float(v[c0 + j + 1]), p.scale_log2, -m_use));
          sum += p0 + p1;
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          packed[j >> 1] = *reinterpret_cast<uint32_t*>(&pk);
        }
        // keys c0..c0+7 are 16-byte chunk (c0 % 64) / 8 of this row inside 64-key block c0 / 64
        const uint32_t dst = p_smem + (c0 >> 6) * (kTcRows * 128) + r * 128 + (((((c0 & 63) >> 3)) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(packed[0]), "r"(packed[1]), "r"(packed[2]),
                     "r"(packed[3]) : "memory");
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      // rescale the output accumulator where the maximum moved (never on the first tile: O is overwritten there)
      if (t > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
        for (int c0 = 0; c0 < kTcD; c0 += 32) {
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
      if (lane == 0) mbar_arrive(bar(6));
    }
    // epilogue: wait for the last P V product, then O / sum
    if (ok && ntiles > 0) ok = mbar_wait(bar(7), (ntiles - 1) & 1, abort_flag, p.status, 17);
    if (ok) {
      tcgen05_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kTcD; c0 += 32) {
        uint32_t v[32];
        tmem_load_32(tmem_o + lane_addr + c0, v);
        if (r < rows) {
          __nv_bfloat16* dst = p.out + (size_t)(tok0 + r) * p.out_stride + (size_t)h * kTcD + c0;
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

// Returns 0 on success; -2 if this kernel does not take the sizes (the caller then uses the
// warp-level kernel): head size 64 only, pages of 8..128 keys that divide 128, 16-byte aligned
// rows; -1 on an error.
PTL_EXPORT int ptl_prefill_attention_tc_bf16(void* out, const void* q, const void* cache, const int* block_table,
                                             const int* tiles, int n_tiles, int n_tokens, int q_stride, int out_stride,
                                             int bt_stride, int nq, int nkv, int d, int page_size, float scale,
                                             int window, int num_pages, int* status, void* stream) {
  using namespace ptl;
  PTL_REQUIRE(n_tiles >= 0 && nq > 0 && nkv > 0 && page_size > 0 && num_pages > 0, "prefill_attention_tc: bad sizes");
  PTL_REQUIRE(nq % nkv == 0, "prefill_attention_tc: %d query heads are no multiple of %d kv heads", nq, nkv);
  if (d != kTcD || page_size < 8 || page_size > kTcKeys || kTcKeys % page_size != 0 || q_stride % 8 != 0 ||
      out_stride % 8 != 0 || nq > 65535)
    return -2;
  PTL_REQUIRE(aligned16(q) && aligned16(cache) && aligned16(out), "prefill_attention_tc: q, cache and out must be 16-byte aligned");
  if (n_tiles == 0) return 0;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem);
    PTL_REQUIRE(e == cudaSuccess, "prefill_attention_tc: cannot raise shared memory: %s", cudaGetErrorString(e));
    raised = true;
  }
  CUtensorMap mq, mkv;
  int rc = make_map(&mq, q, n_tokens, q_stride, kTcRows);                 // whole step: [tokens, q_stride], boxes of 64 x 128
  if (rc) return rc;
  rc = make_map(&mkv, cache, num_pages * 2 * nkv * page_size, kTcD, page_size);   // cache as rows of one head's 64 values
  if (rc) return rc;
  PrefillTcParams p{};
  p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.tiles = tiles; p.status = status;
  p.out_stride = out_stride; p.bt_stride = bt_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size;
  p.window = window; p.num_pages = num_pages; p.scale_log2 = scale * 1.4426950408889634f;
  return launch_kernel("prefill_attention_tc", prefill_attention_tc_kernel, dim3(n_tiles, nq), dim3(kTcThreads), kTcSmem,
                       as_stream(stream), mq, mkv, p);
}
