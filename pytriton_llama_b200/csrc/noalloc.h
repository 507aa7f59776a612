// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in lite_llama.  It exists for hosts that embed the kernel
// library where cudaMalloc is off limits: code that runs between two captured regions of someone
// else's stream, real-time loops that may not take the allocator's lock, plugins that were handed
// a fixed memory budget by their host program and are not allowed to grow it.  Such a caller still
// passes its inputs and its output buffer; what the split-key decode kernel needs in between (the
// per-split partial sums that a second kernel merges) lives in an array that is part of the
// library image instead of being allocated per call.
//
// Cost and limits, so that nobody is surprised:
//   * The array is PTL_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory on EVERY GPU on which the
//     library is loaded, from load until the process exits, used or not.
//   * A call needs n_items * nq * splits * (d + 2) floats of it.  A call that needs more is
//     refused with an error message; nothing is launched.  splits == 1 needs none.
//   * With splits > 1 the tokens must be rows 0..n_items-1 of q and out (items == NULL): the
//     partial results are laid out by row.
//   * The first call with splits > 1 on a device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current) and raises the kernels' shared-memory limit.  Make that first call
//     before any stream capture begins; later calls only launch kernels.
//   * All calls on a device share the one array.  It keeps whatever the last call left there;
//     that is harmless because every call overwrites each partial result it later reads, so
//     nothing has to be cleared.  Two calls whose kernels overlap on the GPU (different streams,
//     no dependency between them) would write the same words: do not do that, order them.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on the first call or later.
//
// Arguments are those of ptl_decode_attention_bf16 (attention_decode.cu) without the two scratch
// pointers.  Returns 0 on success, -2 if the head size or group size is not one this kernel takes,
// -1 on an error (ptl_last_error() has the message).
#pragma once

#define PTL_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int ptl_decode_attention_bf16_noalloc(void* out, const void* q, const void* cache, const int* block_table,
                                      const int* items, const int* tok_req, const int* positions, int n_items,
                                      int q_stride, int out_stride, int bt_stride, int nq, int nkv, int d,
                                      int page_size, float scale, int window, int splits, int num_pages,
                                      void* stream);

/* Bytes of the built-in scratch array (for callers that want to check a size beforehand). */
unsigned long long ptl_noalloc_scratch_bytes(void);

/* Device address of the built-in scratch array on the current device (the same look-up the first
   call with splits > 1 does; allocates nothing).  For diagnostics: a host can overwrite the array
   between calls to convince itself that no call depends on what an earlier one left there.
   Returns 0, or -1 with a message in ptl_last_error(). */
int ptl_noalloc_scratch_address(void** address);

#ifdef __cplusplus
}
#endif
