// The tcgen05 matrix product's host side: the plan (tile width, parts of the K range, pairs of
// blocks), tensor maps, and the exported entry points.  The kernel lives in gemm_tcgen05.cuh.
#include "gemm_tcgen05.cuh"

namespace ptl {

static int sm_count_of_device() {
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  return sm_count;
}

// The plan for a product with many tokens: features per tile (256, 192 where N is a multiple of
// it, or 128) and, where the caller can add partial sums up, into how many parts the K range is cut.
// The cost of a candidate is the number of rounds its work units (tiles x parts) take on the SMs times
// the length of a unit: K blocks per part x 4 MMAs x the cycles of an MMA of that width as one
// thread gets them through (129, 115, 92 per 128 x width x 16: measured; narrow MMAs are bound by
// the rate at which one thread can issue them).  16 x 12 tiles of 256 take two rounds of 148 SMs,
// 16 x 16 of 192 take two cheaper ones; a few hundred tokens make too few wide tiles to fill the
// SMs once.  A narrower tile has to win by a tenth.
struct TilePlan { int bn, parts; };
static TilePlan plan_tiles(int M, int N, int K, bool with_parts, int whole_heads = 0) {
  const int sm_count = sm_count_of_device();
  const long long tm = (M + kTileRows - 1) / kTileRows;
  const int num_kb = (K + kTileK - 1) / kTileK;
  const int widths[3] = {256, 192, 128}, cycles[3] = {129, 115, 92};
  static const int forced = [] { const char* e = getenv("PTL_GEMM_TILE_FEATURES"); return e ? atoi(e) : 0; }();   // (for measurements)
  TilePlan best{128, 1};
  long long best_cost = -1;
  for (int i = 0; i < 3; ++i) {
    const int bn = widths[i];
    if (bn == 192 && N % 192 != 0) continue;
    if (bn == 256 && N % 256 != 0 && N < 2048) continue;        // a narrow product with a ragged edge: 128
    if (forced && forced != bn) continue;
    if (whole_heads && bn % whole_heads != 0) continue;         // the rotary epilogue: a tile's columns hold whole heads
    const long long tiles = tm * ((N + bn - 1) / bn);
    long long parts = 1;
    if (with_parts && tiles * 2 <= sm_count) {
      parts = sm_count / tiles;
      if (parts > 8) parts = 8;
      if (parts > num_kb / 8) parts = num_kb / 8;                // at least 8 K blocks (512 values) per part
      if (parts < 1) parts = 1;
    }
    const long long kb_per = (num_kb + parts - 1) / parts;
    const long long cost = (tiles * parts + sm_count - 1) / sm_count * kb_per * cycles[i];
    if (best_cost < 0 || cost * 100 < best_cost * 90) { best = TilePlan{bn, (int)parts}; best_cost = cost; }
  }
  return best;
}

}  // namespace ptl

// With more than 64 tokens but few of them (or a narrow product) the tiles fill only some of the SMs,
// and each walks the whole K range.  Returns into how many parts the K range is best cut so that the
// work units fill the SMs (1: leave it whole): the caller then asks for float32 partial sums
// (epi 1, `splits_hint` = parts, out [parts, M, N]) and adds them up in order.
PTL_EXPORT int ptl_gemm_tc_k_parts(int M, int N, int K) {
  using namespace ptl;
  if (M <= 64 || K % 8 != 0 || K < kTileK) return 1;
  return plan_tiles(M, N, K, true).parts;
}

// out: epi 0 bf16 [M,N]; 1 float32 [M,N]; 2 float32 [M,N] added to in place; 3 bf16 [M,N/2].
// Returns -2 when the sizes are not ones this kernel takes (K % 8 != 0 or K < 64), so that the caller
// can use another product.  `splits_hint` > 0 forces the number of K splits when M <= 64 (1, 2, 4 or 8);
// when M > 64 it asks for that many parts of the K range, whose partial sums are stored one after
// another (epi 1 only: out is [splits_hint, M, N] float32).
//
// Around an RMS norm: with `xs` (bf16 [M,N]), `norm_w` (float32 [N]) and `sumsq` (float32 [M, sumsq_ld],
// sumsq_ld >= ceil(N/16)) the add epilogue also writes the next norm's input, xs = bfloat16(new
// residual * norm_w), and sums of squares of the new residual over slices of each row; *slots_out
// says how many slots a row got.  A later product that takes this xs as X and is given `scale_sumsq`
// (that array), `scale_slots`, `scale_ld` and `scale_eps` multiplies every output row by
// rsqrt(sum of the row's slots / K + eps), which completes the norm (epi 0, 1 and 3).  -2 is also
// returned when what was asked for around the norm cannot be done for these sizes.
static int gemm_tc_impl(void* out, const void* X, const void* W, int M, int N, int K, int ld_out, int epi,
                        int* status, int splits_hint, void* xs, const float* norm_w, float* sumsq,
                        int sumsq_ld, int* slots_out, const float* scale_sumsq, int scale_slots,
                        int scale_ld, float scale_eps, const ptl::GemmParams* rope, void* stream,
                        unsigned poll_limit = ptl::kPollLimit, int withhold_first_load = 0) {
  using namespace ptl;
  PTL_REQUIRE(M >= 0 && N > 0 && K > 0 && ld_out > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
  if (K % 8 != 0 || K < kTileK) return -2;
  PTL_REQUIRE(aligned16(X) && aligned16(W) && aligned16(out), "gemm_tc: operands must be 16-byte aligned");
  PTL_REQUIRE(epi != 3 || N % 2 == 0, "gemm_tc: the SiLU*up epilogue needs an even number of weight rows");
  if (M == 0) return 0;
  GemmParams p{};
  p.out = out; p.status = status;
  p.K = K; p.ld_out = ld_out;
  p.poll_limit = poll_limit; p.withhold_first_load = withhold_first_load;
  p.timeline = M <= 64 ? timeline_slot() : nullptr;      // (measurements of the decode step)
  p.timeline_kind = 10 + epi;
  if (xs) {
    if (epi != 2 || N % 32 != 0 || ld_out % 4 != 0) return -2;
    PTL_REQUIRE(norm_w && sumsq && slots_out, "gemm_tc: the next norm's input needs its weight, the sums and a place for their count");
    PTL_REQUIRE(aligned16(xs) && aligned16(norm_w) && sumsq_ld >= (N + 15) / 16, "gemm_tc: xs and norm_w must be 16-byte aligned, sumsq_ld >= N/16");
    p.xs = (__nv_bfloat16*)xs; p.norm_w = norm_w; p.sumsq = sumsq; p.xs_ld = N; p.sumsq_ld = sumsq_ld;
  }
  if (scale_sumsq) {
    if (epi == 2) return -2;
    PTL_REQUIRE(scale_slots > 0 && scale_ld >= scale_slots && scale_eps > 0.f, "gemm_tc: bad row scale arguments");
    p.scale_sumsq = scale_sumsq; p.scale_slots = scale_slots; p.scale_ld = scale_ld; p.scale_eps = scale_eps;
    p.scale_inv_n = 1.0f / (float)K;
  }
  const int num_kb = (K + kTileK - 1) / kTileK;
  CUtensorMap mr, mc;
  cudaStream_t s = as_stream(stream);
  if (M > 64) {
    p.swapped = 0; p.rows = M; p.cols = N; p.splits = 1; p.kb_per_split = num_kb;
    const int sm_count = sm_count_of_device();
    int parts = 1;
    const int bn = plan_tiles(M, N, K, splits_hint > 1, rope ? rope->rope_d : 0).bn;
    if (rope) {
      if (epi != 4 || bn % rope->rope_d != 0) return -2;
      p.rope_table = rope->rope_table; p.rope_slots = rope->rope_slots; p.rope_cache = rope->rope_cache;
      p.rope_nq = rope->rope_nq; p.rope_nkv = rope->rope_nkv; p.rope_d = rope->rope_d; p.rope_page = rope->rope_page;
      p.rope_num_slots = rope->rope_num_slots;
    }
    if (splits_hint > 1) {
      PTL_REQUIRE(epi == 1 && !scale_sumsq && splits_hint <= 64 && splits_hint <= num_kb,
                  "gemm_tc: with more than 64 tokens the K range is cut only for plain float32 partial sums, into at most 64 parts");
      parts = splits_hint;
    }
    p.ksplits = parts;
    p.kb_per_split = (num_kb + parts - 1) / parts;
    // wide tiles over at least two token tiles go to pairs of blocks (one MMA of 256 rows, W fetched once per pair)
    static const bool pairs_allowed = [] { const char* e = getenv("PTL_GEMM_PAIRS"); return !(e && e[0] == '0'); }();
    // (not the 128-wide tiles of a few hundred tokens: measured, pairs made them 5 % slower: there the
    // issuing thread's wait for each stage bounds the loop, 160 cycles per MMA of 256 x 128 x 16)
    const bool pair = pairs_allowed && bn >= 192 && parts == 1 && M > kTileRows && sm_count >= 2;
    int rc = make_map(&mr, X, M, K, kTileRows);
    if (rc) return rc;
    rc = make_map(&mc, W, N, K, pair ? bn / 2 : bn);
    if (rc) return rc;
    p.tiles_m = (M + kTileRows - 1) / kTileRows;
    p.tiles_n = (N + bn - 1) / bn;
    if (slots_out) *slots_out = p.tiles_n * 2;
    const long long tiles = pair ? (long long)((p.tiles_m + 1) / 2) * p.tiles_n * 2 : (long long)p.tiles_m * p.tiles_n * parts;
    const long long most = pair ? sm_count / 2 * 2 : sm_count;
    dim3 grid((unsigned)(tiles < most ? tiles : most));
    // the add epilogue hands its tiles to TMA, which adds them into the residual (unless the next norm's input is wanted too)
    CUtensorMap mo = mr;
    if (epi == 2 && !xs && N % 32 == 0 && ld_out % 4 == 0) {
      rc = make_map(&mo, out, M, N, kTileRows, ld_out);
      if (rc) return rc;
      p.tma_add = 1;
    }
    if (pair) return launch_pair_tiles(bn, epi, mr, mc, mo, p, grid, s);
    return launch_many_tokens(bn, epi, mr, mc, mo, p, grid, s);
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
  p.swapped = 1; p.rows = N; p.cols = M; p.splits = splits; p.kb_per_split = kb_per; p.ksplits = 1;
  int rc = make_map(&mr, W, N, K, kTileRows);
  if (rc) return rc;
  rc = make_map(&mc, X, M, K, bn);
  if (rc) return rc;
  dim3 grid(row_tiles, splits);
  if (slots_out) *slots_out = (N + 15) / 16;
  return launch_few_tokens(bn, epi, mr, mc, mr, p, grid, s);
}

PTL_EXPORT int ptl_gemm_tc_bf16_norm(void* out, const void* X, const void* W, int M, int N, int K, int ld_out, int epi,
                                     int* status, int splits_hint, void* xs, const float* norm_w, float* sumsq,
                                     int sumsq_ld, int* slots_out, const float* scale_sumsq, int scale_slots,
                                     int scale_ld, float scale_eps, void* stream) {
  PTL_REQUIRE(epi >= 0 && epi <= 3, "gemm_tc: unknown epilogue %d", epi);
  return gemm_tc_impl(out, X, W, M, N, K, ld_out, epi, status, splits_hint, xs, norm_w, sumsq, sumsq_ld, slots_out, scale_sumsq,
                      scale_slots, scale_ld, scale_eps, nullptr, stream);
}

// The q|k|v projection of a step with more than 64 tokens, with rotary position encoding and the
// cache write in its epilogue: out [M, N] bfloat16 gets the rotated q columns (its k and v columns
// are not written), cache slot slots[t] gets token t's rotated k and plain v.  table [M, d/2] holds
// (cos, sin) of every token's angles (ptl_rope_table).  N = (nq + 2 nkv) d, d 64 or 128, the whole
// head rotated.  Returns -2 where this is not possible (the caller then runs the steps apart).
PTL_EXPORT int ptl_gemm_tc_bf16_qkv_rope(void* out, const void* X, const void* W, int M, int N, int K, int* status,
                                         const void* table, const int* slots, void* cache, int nq, int nkv, int d,
                                         int page_size, long long num_slots, void* stream) {
  using namespace ptl;
  PTL_REQUIRE(nq > 0 && nkv > 0 && d > 0 && page_size > 0 && num_slots > 0, "qkv_rope: bad sizes");
  if (M <= 64 || (d != 64 && d != 128) || N != (nq + 2 * nkv) * d) return -2;
  PTL_REQUIRE(table && slots && cache && aligned16(table) && aligned16(cache), "qkv_rope: needs the angle table, slots and an aligned cache");
  GemmParams rope{};
  rope.rope_table = (const float2*)table; rope.rope_slots = slots; rope.rope_cache = (__nv_bfloat16*)cache;
  rope.rope_nq = nq; rope.rope_nkv = nkv; rope.rope_d = d; rope.rope_page = page_size; rope.rope_num_slots = num_slots;
  return gemm_tc_impl(out, X, W, M, N, K, N, 4, status, 0, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0.f, &rope, stream);
}

PTL_EXPORT int ptl_gemm_tc_bf16(void* out, const void* X, const void* W, int M, int N, int K, int ld_out, int epi,
                                int* status, int splits_hint, void* stream) {
  return ptl_gemm_tc_bf16_norm(out, X, W, M, N, K, ld_out, epi, status, splits_hint, nullptr, nullptr, nullptr, 0, nullptr,
                               nullptr, 0, 0, 0.f, stream);
}

// Self-test of the bounded waits: the product out[M,N] = X W^T (bfloat16 store) as ONE block whose
// first stage is never filled (the load of its token tile is left out) and whose waits give up
// after `poll_limit` polls.  The kernel must then write `*status` (code 2: a wait for a full
// stage ran out), let every role drain, free its tensor memory and return; `out` holds nothing of
// value.  Only sizes that make a single block without a cluster are taken (M <= 128 and N <= 128;
// with M <= 64 also K <= 192), so that no other block or kernel can be left waiting.
PTL_EXPORT int ptl_gemm_tc_wait_selftest(void* out, const void* X, const void* W, int M, int N, int K, int* status,
                                         unsigned poll_limit, void* stream) {
  PTL_REQUIRE(status != nullptr, "gemm_tc_wait_selftest: needs a status word");
  PTL_REQUIRE(M >= 1 && M <= 128 && N >= 1 && N <= 128 && K >= 64 && K % 8 == 0 && (M > 64 || K <= 192),
              "gemm_tc_wait_selftest: one block only (M <= 128, N <= 128, K >= 64; K <= 192 with M <= 64), got M=%d N=%d K=%d", M, N, K);
  PTL_REQUIRE(poll_limit >= 1 && poll_limit <= (1u << 16), "gemm_tc_wait_selftest: between 1 and 65536 polls");
  return gemm_tc_impl(out, X, W, M, N, K, N, 0, status, M <= 64 ? 1 : 0, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0, 0.f,
                      nullptr, stream, poll_limit, 1);
}
