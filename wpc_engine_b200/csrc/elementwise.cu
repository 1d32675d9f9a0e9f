// Row-wise and element-wise kernels: embedding rows, RMS norm, SiLU*up, residual add, row
// gather, rotation angles, rotation + cache append, normal fill.  Each works for float32
// and bfloat16 storage with float32 arithmetic, for any width.
#include "api.h"
#include "common.cuh"

namespace wpc {

// ---- embedding: out[t, :] = table[tokens[t], :] as float32 (wpc-runtime/src/weights.rs:101-105)
template <typename Tw>
__global__ void embed_kernel(const int* __restrict__ tokens, const Tw* __restrict__ table,
                             float* __restrict__ out, int H, int V) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = tokens[t];
  if (id < 0 || id >= V) id = 0;                 // the host checks ids; never read outside
  const Tw* row = table + (size_t)id * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

// ---- RMS norm: out = x * rsqrt(mean(x^2) + eps) * gain (wpc-runtime/src/norm.rs:4-13)
template <typename To>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                               float eps, To* __restrict__ out, int H, const int* __restrict__ rows, int T) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  int src = rows ? rows[blockIdx.x] : (int)blockIdx.x;
  if (src < 0 || src >= T) src = 0;
  const float* row = x + (size_t)src * H;
  To* o = out + (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = row[i];
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float scale = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<To>(row[i] * scale * gain[i]);
}

__device__ __forceinline__ void store4(float* o, float4 v) { *(float4*)o = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* o, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *(uint32_t*)&a;
  u.y = *(uint32_t*)&b;
  *(uint2*)o = u;
}

// The same for widths that are multiples of 4 and at most 4 * VPT * blockDim: the row is read
// once, 16 bytes at a time, and stays in registers between the sum and the scaling.
// `rows` (or null): output row i is the norm of input row rows[i] (the rows whose logits are wanted),
// which the host wrote before the step began; T: rows of x, to keep a bad index inside it.
template <typename To, int VPT>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                   float eps, To* __restrict__ out, int H, const int* __restrict__ rows, int T) {
  pdl_trigger();
  __shared__ float red[32];
  int src = rows ? rows[blockIdx.x] : (int)blockIdx.x;
  if (src < 0 || src >= T) src = 0;
  const float4* row = (const float4*)(x + (size_t)src * H);
  const float4* g4 = (const float4*)gain;
  To* o = out + (size_t)blockIdx.x * H;
  const int n4 = H / 4;
  float4 v[VPT], g[VPT];
  float ss = 0.f;
  // the gain is a model parameter: it is fetched while the kernel ahead is still finishing
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < n4) g[k] = g4[i];
  }
  pdl_wait();
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < n4) {
      v[k] = row[i];
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = block_sum(ss, red);
  const float scale = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < n4)
      store4(o + 4 * i, make_float4(v[k].x * scale * g[k].x, v[k].y * scale * g[k].y, v[k].z * scale * g[k].z,
                                    v[k].w * scale * g[k].w));
  }
}

// ---- act(gate) * up, act = SiLU for the reference's model (wpc-runtime/src/model.rs:527-531).
//      gu rows hold gate and up interleaved in blocks of G features: [G gate | G up | G gate | ...];
//      G = I is "all gates, then all ups".
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int G, size_t n, int act) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / I;
    const int c = (int)(i - t * I);
    const size_t base = t * 2 * I + (size_t)(c / G) * 2 * G + c % G;
    const float g = to_float(gu[base]);
    const float u = to_float(gu[base + G]);
    WPC_WITH_ACT(act, ACT, out[i] = from_float<T>(gate_act<false, ACT>(g) * u));
  }
}

// bfloat16, 8 features a thread (G a multiple of 8, rows 16-byte aligned)
__global__ void silu_mul_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I,
                                    int G, size_t n8, int act) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    const size_t e = i * 8;
    const size_t t = e / I;
    const int c = (int)(e - t * I);
    const size_t base = t * 2 * I + (size_t)(c / G) * 2 * G + c % G;
    const uint4 gv = *(const uint4*)(gu + base), uv = *(const uint4*)(gu + base + G);
    const __nv_bfloat162* g2 = (const __nv_bfloat162*)&gv;
    const __nv_bfloat162* u2 = (const __nv_bfloat162*)&uv;
    uint4 ov;
    __nv_bfloat162* o2 = (__nv_bfloat162*)&ov;
    WPC_WITH_ACT(act, ACT, {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        o2[k] = __floats2bfloat162_rn(gate_act<false, ACT>(g.x) * u.x, gate_act<false, ACT>(g.y) * u.y);
      }
    });
    *(uint4*)(out + e) = ov;
  }
}

template <typename T>
__global__ void add_kernel(float* __restrict__ x, const T* __restrict__ y, size_t n) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] += to_float(y[i]);
}

__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ idx,
                                   float* __restrict__ out, int H, int T) {
  pdl_trigger();
  pdl_wait();
  int r = idx[blockIdx.x];
  if (r < 0 || r >= T) r = 0;
  const float* row = x + (size_t)r * H;
  float* o = out + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = row[i];
}

template <typename Ti, typename To>
__global__ void convert_kernel(const Ti* __restrict__ in, To* __restrict__ out, size_t n) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<To>(to_float(in[i]));
}

// ---- rotation angles in float64, as wpc-runtime/src/rope.rs:30-33 computes them
__global__ void rope_angles_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                   float* __restrict__ cosv, float* __restrict__ sinv, int R, int n) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int t = i / R, r = i - t * R;
  const double a = (double)positions[t] * inv_freq[r];
  double s, c;
  sincos(a, &s, &c);
  cosv[i] = (float)c;
  sinv[i] = (float)s;
}

// rotates the pair (r, r + half) of one head vector (wpc-runtime/src/rope.rs:34-37)
template <typename T>
__device__ __forceinline__ void rotate_pair(const T* v, int r, int half, float c, float s, float& o1, float& o2) {
  const float x1 = to_float(v[r]), x2 = to_float(v[r + half]);
  o1 = x1 * c - x2 * s;
  o2 = x2 * c + x1 * s;
}

// Rotates pair r of every head in place.  interleaved = 0: the pair is (r, r + hd/2), the
// reference's pairing (rope.rs:34-37); 1: the pair is (2r, 2r + 1).
template <typename T>
__global__ void rope_inplace_kernel(T* __restrict__ x, int row_stride, int n_heads, int hd, int R,
                                    const float* __restrict__ cosv, const float* __restrict__ sinv, int interleaved) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, half = hd / 2;
  T* row = x + (size_t)t * row_stride;
  for (int i = threadIdx.x; i < n_heads * R; i += blockDim.x) {
    const int h = i / R, r = i - h * R;
    const float c = cosv[(size_t)t * R + r], s = sinv[(size_t)t * R + r];
    T* a = row + h * hd + (interleaved ? 2 * r : r);
    T* b = interleaved ? a + 1 : a + half;
    const float x1 = to_float(*a), x2 = to_float(*b);
    *a = from_float<T>(x1 * c - x2 * s);
    *b = from_float<T>(x2 * c + x1 * s);
  }
}

// ---- RMS norm of every head of a row, in place: a warp to a (token, head); the same arithmetic
//      as rmsnorm_kernel over hd elements (wpc-runtime/src/model.rs:447-462 applies norm.rs:4-13
//      to each head's slice)
template <typename T>
__global__ void head_rmsnorm_kernel(T* __restrict__ x, int row_stride, int n_heads, int hd,
                                    const float* __restrict__ gain, float eps, int T_rows) {
  pdl_trigger();
  pdl_wait();
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (warp >= T_rows * n_heads) return;
  const int t = warp / n_heads, h = warp - t * n_heads;
  T* v = x + (size_t)t * row_stride + (size_t)h * hd;
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) {
    const float f = to_float(v[i]);
    ss += f * f;
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
  for (int i = lane; i < hd; i += 32) v[i] = from_float<T>(to_float(v[i]) * scale * gain[i]);
}

// ---- q and k rotated (q in place), k and v appended to the pages of their sequence
//      (wpc-runtime/src/model.rs:464-475: keys are stored after rotation, values as they are).
//      Row layout of qkv: nh query heads, then nkv key heads, then nkv value heads.
//      One warp per (token, head of the row), eight heads to a block.
constexpr int ROPE_HEADS_PER_BLOCK = 8;
template <typename T>
__global__ void qk_rope_kv_store_kernel(T* __restrict__ qkv, int row_stride, int nh, int nkv, int hd, int R,
                                        const float* __restrict__ cosv, const float* __restrict__ sinv,
                                        T* __restrict__ k_pages, T* __restrict__ v_pages,
                                        const int* __restrict__ page_table, int table_width,
                                        const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                                        int n_pages, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, half = hd / 2, lane = threadIdx.x & 31;
  const int head = blockIdx.y * ROPE_HEADS_PER_BLOCK + (threadIdx.x >> 5);
  if (head >= nh + 2 * nkv) return;
  T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
  const float* ct = cosv ? cosv + (size_t)t * R : nullptr;
  const float* st = sinv ? sinv + (size_t)t * R : nullptr;
  if (head < nh) {
    for (int r = lane; r < R; r += 32) {
      float o1, o2;
      rotate_pair(src, r, half, ct[r], st[r], o1, o2);
      src[r] = from_float<T>(o1);
      src[r + half] = from_float<T>(o2);
    }
    return;
  }
  const int pos = positions[t];
  const int b = seq_of_token[t];
  const int block = pos / WPC_PAGE;
  const int page = (block < table_width) ? page_table[(size_t)b * table_width + block] : -1;
  if (page < 0 || page >= n_pages) {
    if (lane == 0 && status) atomicExch(status, WPC_ERR_BAD_ARGUMENT);
    return;
  }
  const int in_page = pos % WPC_PAGE;
  if (head < nh + nkv) {
    const int h = head - nh;
    T* dst = k_pages + (((size_t)page * nkv + h) * WPC_PAGE + in_page) * hd;
    for (int r = lane; r < half; r += 32) {
      if (r < R) {
        float o1, o2;
        rotate_pair(src, r, half, ct[r], st[r], o1, o2);
        dst[r] = from_float<T>(o1);
        dst[r + half] = from_float<T>(o2);
      } else {
        dst[r] = src[r];
        dst[r + half] = src[r + half];
      }
    }
  } else {
    const int h = head - nh - nkv;
    T* dst = v_pages + (((size_t)page * nkv + h) * WPC_PAGE + in_page) * hd;
    for (int d = lane; d < hd; d += 32) dst[d] = src[d];
  }
}

// ---- N(mean, std) fill from a counter-based generator: element i of a tensor with key k
//      draws from mix64(k ^ mix64(i)); Box-Muller on two 24-bit uniforms
template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, size_t n, uint64_t key, float mean, float std) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t z = mix64(key ^ mix64((uint64_t)i));
    const float u1 = ((float)((z >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
    const float u2 = (float)((z >> 16) & 0xFFFFFF) * (1.0f / 16777216.0f);            // [0, 1)
    const float r = sqrtf(-2.0f * logf(u1));
    out[i] = from_float<T>(mean + std * r * cospif(2.0f * u2));
  }
}

static inline int grid_for(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace wpc

using namespace wpc;

extern "C" {

int wpc_set_pdl(int on) {
  const int was = pdl_enabled();
  pdl_enabled() = on ? 1 : 0;
  return was;
}

int wpc_set_wait_policy(unsigned long long limit_ns, int starve) {
  if (limit_ns == 0) return WPC_ERR_BAD_ARGUMENT;
  wait_policy().limit_ns = limit_ns;
  wait_policy().starve = starve ? 1 : 0;
  return 0;
}

int wpc_embed(const int* tokens, const void* table, int table_dtype, float* out, int T, int H, int V,
              cudaStream_t stream) {
  if (T <= 0) return 0;
  WPC_DISPATCH_DTYPE(table_dtype, Tw,
                     (wpc::launch(embed_kernel<Tw>, T, 256, 0, stream, tokens, (const Tw*)table, out, H, V)));
  return launch_status();
}

// rows == null: out [T, H] = norm of x [T, H].  Else out [n_rows, H]: row i is the norm of x[rows[i]].
int wpc_rmsnorm(const float* x, const float* gain, float eps, void* out, int out_dtype, int T, int H,
                const int* rows, int n_rows, cudaStream_t stream) {
  const int n = rows ? n_rows : T;
  if (n <= 0 || T <= 0) return 0;
  const bool aligned = H % 4 == 0 && (((uintptr_t)x | (uintptr_t)gain | (uintptr_t)out) & 15) == 0;
  if (aligned && H <= 1024) {
    WPC_DISPATCH_DTYPE(out_dtype, To, (wpc::launch(rmsnorm_vec_kernel<To, 2>, n, 128, 0, stream, x, gain, eps, (To*)out, H, rows, T)));
  } else if (aligned && H <= 4096) {
    WPC_DISPATCH_DTYPE(out_dtype, To, (wpc::launch(rmsnorm_vec_kernel<To, 4>, n, 256, 0, stream, x, gain, eps, (To*)out, H, rows, T)));
  } else if (aligned && H <= 16384) {
    WPC_DISPATCH_DTYPE(out_dtype, To, (wpc::launch(rmsnorm_vec_kernel<To, 8>, n, 512, 0, stream, x, gain, eps, (To*)out, H, rows, T)));
  } else {
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    WPC_DISPATCH_DTYPE(out_dtype, To, (wpc::launch(rmsnorm_kernel<To>, n, threads, 0, stream, x, gain, eps, (To*)out, H, rows, T)));
  }
  return launch_status();
}

int wpc_gate_mul(const void* gu, void* out, int dtype, int T, int I, int group, int act, cudaStream_t stream) {
  const size_t n = (size_t)T * I;
  if (n == 0) return 0;
  if (group < 1 || I % group || (act != WPC_ACT_SILU && act != WPC_ACT_GELU_TANH)) return WPC_ERR_BAD_ARGUMENT;
  if (dtype == WPC_DTYPE_BF16 && group % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
    wpc::launch(silu_mul_vec_kernel, grid_for(n / 8, 256), 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I,
                                                                 group, n / 8, act);
    return launch_status();
  }
  WPC_DISPATCH_DTYPE(dtype, Tt, (wpc::launch(silu_mul_kernel<Tt>, grid_for(n, 256), 256, 0, stream, (const Tt*)gu, (Tt*)out,
                                                                                          I, group, n, act)));
  return launch_status();
}

int wpc_add(float* x, const void* y, int y_dtype, size_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  WPC_DISPATCH_DTYPE(y_dtype, Tt, (wpc::launch(add_kernel<Tt>, grid_for(n, 256), 256, 0, stream, x, (const Tt*)y, n)));
  return launch_status();
}

int wpc_gather_rows(const float* x, const int* idx, float* out, int n_rows, int H, int T, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  wpc::launch(gather_rows_kernel, n_rows, 256, 0, stream, x, idx, out, H, T);
  return launch_status();
}

int wpc_convert(const void* in, int in_dtype, void* out, int out_dtype, size_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  const int g = grid_for(n, 256);
  if (in_dtype == WPC_DTYPE_F32 && out_dtype == WPC_DTYPE_BF16)
    wpc::launch(convert_kernel<float, __nv_bfloat16>, g, 256, 0, stream, (const float*)in, (__nv_bfloat16*)out, n);
  else if (in_dtype == WPC_DTYPE_BF16 && out_dtype == WPC_DTYPE_F32)
    wpc::launch(convert_kernel<__nv_bfloat16, float>, g, 256, 0, stream, (const __nv_bfloat16*)in, (float*)out, n);
  else
    return WPC_ERR_BAD_ARGUMENT;
  return launch_status();
}

int wpc_rope_angles(const int* positions, const double* inv_freq, float* cosv, float* sinv, int T, int R,
                    cudaStream_t stream) {
  const int n = T * R;
  if (n <= 0) return 0;
  wpc::launch(rope_angles_kernel, (n + 127) / 128, 128, 0, stream, positions, inv_freq, cosv, sinv, R, n);
  return launch_status();
}

int wpc_rope_inplace(void* x, int dtype, int row_stride, int T, int n_heads, int hd, int R, const float* cosv,
                     const float* sinv, int interleaved, cudaStream_t stream) {
  if (T <= 0 || R <= 0) return 0;
  if (hd % 2 || R > hd / 2) return WPC_ERR_BAD_ARGUMENT;
  WPC_DISPATCH_DTYPE(dtype, Tt, (wpc::launch(rope_inplace_kernel<Tt>, T, 256, 0, stream, (Tt*)x, row_stride, n_heads, hd,
                                                                               R, cosv, sinv, interleaved ? 1 : 0)));
  return launch_status();
}

int wpc_head_rmsnorm(void* x, int dtype, int row_stride, int T, int n_heads, int hd, const float* gain, float eps,
                     cudaStream_t stream) {
  if (T <= 0 || n_heads <= 0) return 0;
  if (hd < 1 || !gain) return WPC_ERR_BAD_ARGUMENT;
  const long warps = (long)T * n_heads;
  WPC_DISPATCH_DTYPE(dtype, Tt, (wpc::launch(head_rmsnorm_kernel<Tt>, (unsigned)((warps + 7) / 8), 256, 0, stream, (Tt*)x,
                                             row_stride, n_heads, hd, gain, eps, T)));
  return launch_status();
}

int wpc_qk_rope_kv_store(void* qkv, int dtype, int row_stride, int T, int nh, int nkv, int hd, int R,
                         const float* cosv, const float* sinv, void* k_pages, void* v_pages,
                         const int* page_table, int table_width, const int* seq_of_token, const int* positions,
                         int n_pages, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd % 2 || R > hd / 2 || (R > 0 && (!cosv || !sinv))) return WPC_ERR_BAD_ARGUMENT;
  WPC_DISPATCH_DTYPE(dtype, Tt,
                     (wpc::launch(qk_rope_kv_store_kernel<Tt>, dim3(T, (nh + 2 * nkv + ROPE_HEADS_PER_BLOCK - 1) / ROPE_HEADS_PER_BLOCK),
                                 32 * ROPE_HEADS_PER_BLOCK, 0, stream, 
                         (Tt*)qkv, row_stride, nh, nkv, hd, R, cosv, sinv, (Tt*)k_pages, (Tt*)v_pages, page_table,
                         table_width, seq_of_token, positions, n_pages, status)));
  return launch_status();
}

int wpc_fill_normal(void* out, int dtype, size_t n, uint64_t key, float mean, float std, cudaStream_t stream) {
  if (n == 0) return 0;
  WPC_DISPATCH_DTYPE(dtype, Tt, (wpc::launch(fill_normal_kernel<Tt>, grid_for(n, 256), 256, 0, stream, (Tt*)out, n, key,
                                                                                             mean, std)));
  return launch_status();
}

}  // extern "C"
