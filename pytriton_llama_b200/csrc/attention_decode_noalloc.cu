// The allocation-free variant of the split-key decode attention: see noalloc.h for who needs it
// and what it costs.  The kernels are the ones the engine uses (attention_decode.cu); only the
// place of the partial results differs: a file-scope device array instead of caller memory.
#include "common.cuh"
#include "noalloc.h"

// The regular entry point, which takes the scratch buffers from its caller.
extern "C" int ptl_decode_attention_bf16(void* out, float* part_acc, float* part_ml, const void* q, const void* cache,
                                         const int* block_table, const int* items, const int* tok_req,
                                         const int* positions, int n_items, int q_stride, int out_stride,
                                         int bt_stride, int nq, int nkv, int d, int page_size, float scale, int window,
                                         int splits, int num_pages, int* counters, void* stream);

namespace {

constexpr size_t kScratchFloats = PTL_NOALLOC_SCRATCH_BYTES / sizeof(float);

// Part of the library image on every device that loads it.  In host code this name is only a
// handle for cudaGetSymbolAddress, never a pointer to hand to a kernel.
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {nullptr};   // device address of the array, per device

// Looks the array up once per device, with that device current.
int scratch_for_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return ptl::fail("decode_attention_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return ptl::fail("decode_attention_noalloc: device %d is beyond the %d this table holds", dev, kMaxDevices);
  if (!g_scratch_address[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return ptl::fail("decode_attention_noalloc: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
    g_scratch_address[dev] = static_cast<float*>(p);
  }
  *ptr = g_scratch_address[dev];
  return 0;
}

}  // namespace

PTL_EXPORT unsigned long long ptl_noalloc_scratch_bytes(void) { return PTL_NOALLOC_SCRATCH_BYTES; }

PTL_EXPORT int ptl_noalloc_scratch_address(void** address) {
  PTL_REQUIRE(address != nullptr, "noalloc_scratch_address: nowhere to put the address");
  float* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc) return rc;
  *address = base;
  return 0;
}

PTL_EXPORT int ptl_decode_attention_bf16_noalloc(void* out, const void* q, const void* cache, const int* block_table,
                                                 const int* items, const int* tok_req, const int* positions,
                                                 int n_items, int q_stride, int out_stride, int bt_stride, int nq,
                                                 int nkv, int d, int page_size, float scale, int window, int splits,
                                                 int num_pages, void* stream) {
  PTL_REQUIRE(n_items >= 0 && nq > 0 && nkv > 0 && d > 0 && splits >= 1, "decode_attention_noalloc: bad sizes");
  float* part_acc = nullptr;
  float* part_ml = nullptr;
  if (splits > 1) {
    // Partial accumulators [token row][nq][splits][d], then the (max, sum) pairs [token row][nq][splits][2].
    // The kernels index both by the token's row in q, so the array is laid out for rows 0..n_items-1.
    const unsigned long long acc = (unsigned long long)n_items * nq * splits * d;
    const unsigned long long ml = (unsigned long long)n_items * nq * splits * 2;
    PTL_REQUIRE(acc + ml <= kScratchFloats,
                "decode_attention_noalloc: %d tokens x %d heads x %d splits x (%d + 2) floats = %llu bytes exceed the "
                "built-in scratch of %u bytes; use fewer splits or tokens, or the entry point that takes scratch buffers",
                n_items, nq, splits, d, (acc + ml) * 4ull, PTL_NOALLOC_SCRATCH_BYTES);
    PTL_REQUIRE(items == nullptr, "decode_attention_noalloc: with splits > 1 the tokens must be rows 0..n_items-1 (items == nullptr)");
    float* base = nullptr;
    int rc = scratch_for_current_device(&base);
    if (rc) return rc;
    part_acc = base;
    part_ml = base + ((acc + 63ull) & ~63ull);
    PTL_REQUIRE(((acc + 63ull) & ~63ull) + ml <= kScratchFloats, "decode_attention_noalloc: scratch too small after alignment");
  }
  return ptl_decode_attention_bf16(out, part_acc, part_ml, q, cache, block_table, items, tok_req, positions, n_items,
                                   q_stride, out_stride, bt_stride, nq, nkv, d, page_size, scale, window, splits,
                                   num_pages, /*counters=*/nullptr, stream);
}
