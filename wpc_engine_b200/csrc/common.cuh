// Shared helpers of the kernels: element types, conversions, reductions, launch checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define WPC_DTYPE_F32 0
#define WPC_DTYPE_BF16 1

// error codes returned by the launchers (besides cudaError_t values, which are < 1000)
#define WPC_ERR_BAD_ARGUMENT 1001
#define WPC_ERR_UNSUPPORTED 1002
#define WPC_ERR_TOO_LARGE 1003
#define WPC_ERR_DEVICE_WAIT 1004

#define WPC_PAGE 64

namespace wpc {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

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

// Sum over a block of up to 1024 threads; `red` is shared memory of 32 floats.  All threads
// get the result.  Fixed order, so a row's result does not depend on its neighbours.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = (lane < nwarps) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = (lane < nwarps) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// ---- thread-block clusters: a barrier over all threads of all CTAs, and stores into a peer's shared memory ----
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in the cluster's shared window, of this CTA's shared address `addr` in CTA `rank`
__device__ __forceinline__ uint32_t peer_smem(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// (a peer may be written once it runs: after a cluster barrier at the start of the kernel; every
// store is a packet between two SMs, so the wide forms are the ones to use)
__device__ __forceinline__ void st_peer_f32x2(uint32_t addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void st_peer_f32x4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// The barrier in two halves: what a thread wrote before it arrived, peers see after their wait.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// Every kernel of this library starts with pdl_trigger() and calls pdl_wait() before it touches
// memory that an earlier kernel of the stream may have written.  Launched with the attribute
// below, a kernel may then become resident, set itself up and (where it says so) fetch model
// weights while the kernel before it is still finishing; pdl_wait() returns once that kernel
// has completed and its writes are visible.  Without the attribute both calls do nothing.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline int& pdl_enabled() {
  static int on = 1;
  return on;
}
// Set to 1 before a launch that should not start ahead of the kernel before it; cleared by the launch.
inline int& pdl_skip_next() {
  static thread_local int skip = 0;
  return skip;
}
inline int& last_launch_error() {
  static thread_local int rc = 0;
  return rc;
}

template <typename... KArgs, typename... Args>
inline void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_enabled() && !pdl_skip_next()) ? 1 : 0;
  pdl_skip_next() = 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) last_launch_error() = (int)e;
}

// The same with thread-block clusters of `cluster_x` CTAs along x (gridDim.x a multiple of it).
template <typename... KArgs, typename... Args>
inline void launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_enabled() && !pdl_skip_next()) ? 2 : 1;
  pdl_skip_next() = 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) last_launch_error() = (int)e;
}

inline int launch_status() {
  int rc = last_launch_error();
  last_launch_error() = 0;
  const int e = (int)cudaGetLastError();
  return rc ? rc : e;
}

}  // namespace wpc

// Runs the statement given last with `T` bound to the element type that `code` names.
#define WPC_DISPATCH_DTYPE(code, T, ...)                   \
  do {                                                     \
    if ((code) == WPC_DTYPE_F32) {                         \
      using T = float;                                     \
      __VA_ARGS__;                                         \
    } else if ((code) == WPC_DTYPE_BF16) {                 \
      using T = __nv_bfloat16;                             \
      __VA_ARGS__;                                         \
    } else {                                               \
      return WPC_ERR_BAD_ARGUMENT;                         \
    }                                                      \
  } while (0)
