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

// ---- the activation of a gated feed-forward: out = act(gate) * up ---------------------------------
#define WPC_ACT_SILU 1          // g / (1 + exp(-g))  (wpc-runtime/src/model.rs:527-531)
#define WPC_ACT_GELU_TANH 2     // g/2 (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))
// FAST: the quotient of SiLU by __fdividef (2 units in the last place of float32), for
// epilogues whose results become bfloat16 at once and where the exact division's slow path
// would be a branch per element.
template <bool FAST, int ACT>
__device__ __forceinline__ float gate_act(float g) {
  if (ACT == WPC_ACT_GELU_TANH) {
    const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    return 0.5f * g * (1.0f + t);
  }
  return FAST ? __fdividef(g, 1.0f + expf(-g)) : g / (1.0f + expf(-g));
}
// Runs the statement given last once, with ACT a compile-time copy of `act`: a loop over many
// elements then has no test inside it (a test per element would turn independent chains of exp
// and division into branches that run one after the other).
#define WPC_WITH_ACT(act, ACT, ...)                 \
  do {                                              \
    if ((act) == WPC_ACT_GELU_TANH) {               \
      constexpr int ACT = WPC_ACT_GELU_TANH;        \
      __VA_ARGS__;                                  \
    } else {                                        \
      constexpr int ACT = WPC_ACT_SILU;             \
      __VA_ARGS__;                                  \
    }                                               \
  } while (0)

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
__device__ __forceinline__ void st_peer_b32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
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

// ---- bounded waits ------------------------------------------------------------------------------
// Every wait of a kernel on an mbarrier gives up after `limit_ns`; the kernel then records
// WPC_ERR_DEVICE_WAIT in the device status word and returns.  `starve` is a switch for tests of
// that path: the warp that starts a kernel's TMA copies starts none, so that the barriers that
// wait for data are never signalled and the waits run out (nothing is in flight then, nothing
// traps, and the kernel leaves as it would after a real loss).  Both are copied into a
// kernel's arguments at launch.
struct WaitPolicy {
  unsigned long long limit_ns;
  int starve;
};
inline WaitPolicy& wait_policy() {
  static WaitPolicy p = {2000000000ull, 0};      // 2 s
  return p;
}

// ---- the current device ---------------------------------------------------------------------------
constexpr int MAX_DEVICES = 64;
inline int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 0;
  return dev;
}
// SMs of the current device (asked once per device).
inline int sm_count() {
  static int n[MAX_DEVICES] = {0};
  const int dev = current_device();
  if (n[dev] <= 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per device and kernel: `done` is the
// kernel's own table of the sizes set so far (zero-initialised static).  Returns 0 or a cudaError_t.
template <typename K>
inline int allow_smem(K kernel, int bytes, int (&done)[MAX_DEVICES]) {
  const int dev = current_device();
  if (done[dev] >= bytes && done[dev] > 0) return 0;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return (int)e;
  done[dev] = bytes > 0 ? bytes : 1;
  return 0;
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
