// Shared helpers of the sm_100a kernel library: element conversion, warp/block reductions,
// error reporting.  Every exported launcher is `extern "C" int ptl_*(...)`: it checks its
// sizes, launches on the caller's stream and returns 0, or a non-zero code after storing a
// message that `ptl_last_error()` hands back.  No launcher allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>

#define PTL_EXPORT extern "C" __attribute__((visibility("default")))

namespace ptl {

// ---------------------------------------------------------------- errors (host)
inline char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
inline int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return -1;
}
inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
  return 0;
}
#define PTL_REQUIRE(cond, ...) do { if (!(cond)) return ptl::fail(__VA_ARGS__); } while (0)

// ---------------------------------------------------------------- element types
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A 16-byte packet of T: 4 floats or 8 bfloat16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ float get(int i) const { return (&raw.x)[i]; }
  __device__ __forceinline__ void set(int i, float v) { (&raw.x)[i] = v; }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(&raw);
    return __bfloat162float(p[i]);
  }
  __device__ __forceinline__ void set(int i, float v) {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(&raw);
    p[i] = __float2bfloat16_rn(v);
  }
};
template <typename T> __device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> v;
  v.raw = *reinterpret_cast<const decltype(v.raw)*>(p);
  return v;
}
template <typename T> __device__ __forceinline__ void store16(T* p, const Vec16<T>& v) {
  *reinterpret_cast<decltype(v.raw)*>(p) = v.raw;
}

// ---------------------------------------------------------------- reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---------------------------------------------------------------- programmatic dependent launch
// Kernels of one step run back to back on one stream.  Launched with the attribute below, a kernel
// may start while its predecessor is still running: its blocks get scheduled and do whatever does
// not depend on earlier kernels (set-up, fetching weights), then `pdl_wait()` holds each thread
// until every earlier kernel has finished and its writes are visible.  `pdl_launch_dependents()`
// lets the successor start likewise.  Rule: no access to memory that another kernel of the step
// writes, and no global write at all, before `pdl_wait()`.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline int& pdl_flag() {
  static int enabled = 1;
  return enabled;
}

// ---------------------------------------------------------------- timeline of a step (measurements only)
// Between ptl_timeline_begin(buffer, slots) and ptl_timeline_end() the launchers of the decode
// step's kernels hand every launch a slot of 16 words of `buffer` (device memory), and the first and
// the last block of the grid write %globaltimer there at fixed points: word 0 the kind of kernel,
// words 1..7 the first block's stamps, 8..14 the last block's.  Stamps: 0 block entered, 1 the wait on
// the predecessor returned, 2 first operands arrived, 3 main loop done, 4 accumulators / partial
// results complete, 5 block done.  Outside such a bracket the slot is null and the kernels skip it.
struct TimelineState { unsigned long long* buf; int capacity; int next; };
inline TimelineState& timeline_state() {
  static TimelineState s = {nullptr, 0, 0};
  return s;
}
inline unsigned long long* timeline_slot() {
  TimelineState& s = timeline_state();
  if (!s.buf || s.next >= s.capacity) return nullptr;
  return s.buf + 16 * (size_t)s.next++;
}
__device__ __forceinline__ void timeline_stamp(unsigned long long* slot, int idx) {
  if (!slot) return;
  const unsigned block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const unsigned last = gridDim.x * gridDim.y * gridDim.z - 1;
  if (block != 0 && block != last) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  slot[1 + (block == 0 ? 0 : 7) + idx] = t;
}

// One rotary pair: (x1, x2) turned by the angle whose cosine and sine are given.  Products and sums
// are rounded one by one (no fused multiply-add), so that every kernel that rotates gets the same bits.
__device__ __forceinline__ void rope_rotate(float x1, float x2, float c, float s, float& o1, float& o2) {
  o1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
  o2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
}

// ---------------------------------------------------------------- thread-block clusters
// Arrive and wait of the cluster barrier (every thread of every block takes part), the address of
// a peer block's shared memory, and stores into it.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_peer(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_peer_f32(uint32_t remote_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_peer_f32x2(uint32_t remote_addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote_addr), "f"(a), "f"(b) : "memory");
}

// Launches `kernel` on `stream`, as a programmatic dependent of the kernel before it when enabled.
// `cluster_x` > 1 groups that many consecutive blocks (along x) into a thread-block cluster.
template <typename... Params, typename... Args>
inline int launch_kernel_cluster(const char* what, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_flag()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
  if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
}

template <typename... Params, typename... Args>
inline int launch_kernel(const char* what, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                         cudaStream_t stream, Args&&... args) {
  return launch_kernel_cluster(what, kernel, grid, block, smem, stream, 1, static_cast<Args&&>(args)...);
}

// The dynamic shared-memory limit of a kernel is a property of (kernel, device).  A launcher keeps
// one `SmemRaised` per kernel instance (static, zero-initialised) and calls this before launching:
// the limit is raised on the current device the first time `level` is asked for there.
constexpr int kMaxDevices = 64;
struct SmemRaised { unsigned char level[kMaxDevices]; };
template <typename Kernel>
inline int raise_shared_memory(const char* what, Kernel kernel, int bytes, SmemRaised& table, int level = 1) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail("%s: no current device below %d", what, kMaxDevices);
  if (table.level[dev] >= level) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail("%s: cannot raise shared memory to %d bytes: %s", what, bytes, cudaGetErrorString(e));
  table.level[dev] = (unsigned char)level;
  return 0;
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace ptl
