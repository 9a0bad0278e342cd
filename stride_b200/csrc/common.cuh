// Shared helpers of the sm_100a kernels: error reporting through the C ABI,
// bfloat16 widening and rounding, fixed-order block reductions.
//
// Every exported function returns 0 on success. On a refused argument or a CUDA
// error it returns non-zero and leaves a message that `sb_last_error()` of the
// same library returns; nothing is launched after a refused argument.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <set>
#include <utility>

#define SB_EXPORT extern "C" __attribute__((visibility("default")))

namespace sb {

inline char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

inline int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return 1;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
  return 0;
}

// Programmatic dependent launch: a kernel launched with `launch_pdl` may start while its predecessor
// in the stream still runs. `grid_dependency_wait()` returns once the predecessor has finished and its
// writes are visible; every kernel calls it before its first read of data another kernel wrote and
// before its first global write, so completion of a kernel implies completion of all before it.
// `grid_launch_dependents()` lets the successor's blocks be scheduled (they then sit in their own wait).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Every kernel asks for the largest shared-memory carve-out, so that consecutive kernels of a step do not
// make the SMs switch their L1 / shared split (which would keep a successor from becoming resident early).
inline void prefer_max_shared(const void* kernel) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;     // a kernel's attributes are kept per device
  int device = 0;
  cudaGetDevice(&device);
  std::lock_guard<std::mutex> lock(mu);
  if (done.insert({kernel, device}).second)
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// The number of SMs of the current device (148 on a B200), asked once per device: what grids of persistent CTAs and
// "does everything run at once" decisions are sized by.
inline int sm_count() {
  static std::atomic<int> cached[64];
  int d = 0;
  cudaGetDevice(&d);
  int n = cached[d & 63].load(std::memory_order_relaxed);
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 148;
    cached[d & 63].store(n, std::memory_order_relaxed);
  }
  return n;
}

// A kernel's attributes (its shared-memory limit among them) are kept per device: `DeviceOnce` remembers on which
// devices a call site has set them. Usage: static DeviceOnce once; if (once.needed()) { set ...; once.done(); }
struct DeviceOnce {
  std::atomic<unsigned long long> mask{0};
  bool needed() {
    int d = 0;
    cudaGetDevice(&d);
    return !((mask.load(std::memory_order_acquire) >> (d & 63)) & 1ull);
  }
  void done() {
    int d = 0;
    cudaGetDevice(&d);
    mask.fetch_or(1ull << (d & 63), std::memory_order_release);
  }
};

template <class... KArgs, class... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);   // errors surface through check_launch()
}

// The same with the grid cut into thread-block clusters of `cluster` CTAs.
template <class... KArgs, class... Args>
inline void launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster,
                               Args&&... args) {
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster.x;
  attr[1].val.clusterDim.y = cluster.y;
  attr[1].val.clusterDim.z = cluster.z;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);   // errors surface through check_launch()
}

// Thread-block clusters: this CTA's rank, and a barrier over all threads of the cluster (release / acquire).
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The address, in the cluster's shared-memory window, of the same variable in the CTA of rank `rank`; and loads from it.
__device__ __forceinline__ uint32_t cluster_peer_address(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))), "r"(rank));
  return out;
}
__device__ __forceinline__ float2 cluster_load_float2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
  return v;
}

__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class T>
__device__ __forceinline__ T narrow(float v);
template <>
__device__ __forceinline__ float narrow<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sum over the block in an order that depends only on blockDim: lanes by xor
// shuffles, then the warps' sums left to right. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  float total = smem32[0];
  for (int i = 1; i < nwarps; ++i) total += smem32[i];
  return total;
}

__device__ __forceinline__ float block_max(float v, float* smem32) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  float total = smem32[0];
  for (int i = 1; i < nwarps; ++i) total = fmaxf(total, smem32[i]);
  return total;
}

}  // namespace sb

#define SB_DEFINE_LAST_ERROR() \
  SB_EXPORT const char* sb_last_error() { return sb::error_buffer(); }
