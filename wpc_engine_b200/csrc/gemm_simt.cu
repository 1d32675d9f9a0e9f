// C[M,N] = A[M,K] . W[N,K]^T (+ bias), float32 multiply-add on the CUDA cores only: the
// matrix product of the true 32-bit path, and the plain twin of the tensor-core product.
// Each output is one dot product (wpc-runtime/src/weights.rs:59-78) accumulated in float32 in a
// fixed order that depends on the shape alone, so a row's result does not depend on the other
// rows: in ascending k in the tile kernel, a lane's elements in ascending k and then a fixed
// tree over the lanes in the kernel for few rows.
#include "api.h"
#include "common.cuh"

namespace wpc {

constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16, SG_THREADS = 256;

// mode 0: C (type To) = acc + bias;  mode 1: C (float32) += acc + bias
template <typename Ta, typename Tw, typename To, int MODE>
__global__ void __launch_bounds__(SG_THREADS)
gemm_simt_kernel(const Ta* __restrict__ A, int lda, const Tw* __restrict__ W, int ldw,
                 const float* __restrict__ bias, To* __restrict__ C, int ldc, int M, int N, int K) {
  pdl_trigger();
  pdl_wait();
  __shared__ float As[SG_BK][SG_BM + 4];
  __shared__ float Ws[SG_BK][SG_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
  const int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
    for (int e = tid; e < SG_BM * SG_BK; e += SG_THREADS) {
      const int r = e / SG_BK, c = e % SG_BK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
    }
#pragma unroll
    for (int e = tid; e < SG_BN * SG_BK; e += SG_THREADS) {
      const int r = e / SG_BK, c = e % SG_BK;
      const int gn = n0 + r, gk = k0 + c;
      Ws[c][r] = (gn < N && gk < K) ? to_float(W[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SG_BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      To* dst = C + (size_t)gm * ldc + gn;
      if (MODE == 1) *dst = from_float<To>(to_float(*dst) + v);
      else *dst = from_float<To>(v);
    }
  }
}

// ---- few rows (tokens): a product that streams the weights once ----------------------------------
// With up to 16 rows of A the tile kernel above would spend a 64 x 64 tile on them and read the
// weights through shared memory at a fraction of the memory bandwidth.  Here a warp takes FPW
// features (four, or one when the features are so few that blocks of 32 features would leave
// SMs idle) and walks their weight rows with 16-byte loads, each lane its own elements of k, all rows of A against them; the rows of A pass through
// shared memory in chunks of k that the eight warps share.  A lane adds its elements in ascending
// k, then the 32 lanes are added in a fixed tree: float32 multiply-add only, the same order for a
// row whatever the other rows are.
constexpr int GV_WARPS = 8;
// k elements of every row of A in shared memory at a time (32 KiB at most)
__host__ __device__ constexpr int gv_chunk(int mt) { return mt <= 8 ? 1024 : 512; }

template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 t = __ldg((const float4*)p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = __ldg((const uint2*)p);
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&t.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&t.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
};

// MT: rows of A handled at once (1, 2, 4, 8 or 16; M <= MT).  VEC: K and both row strides are
// multiples of 4 elements and both bases 16-byte aligned, so that four elements load at once.
template <typename Ta, typename Tw, typename To, int MODE, int MT, bool VEC, int GV_FPW>
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_simt_kernel(const Ta* __restrict__ A, int lda, const Tw* __restrict__ W, int ldw, const float* __restrict__ bias,
                 To* __restrict__ C, int ldc, int M, int N, int K) {
  pdl_trigger();
  constexpr int GV_CHUNK = gv_chunk(MT);
  __shared__ __align__(16) float xs[MT][GV_CHUNK];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int f0 = (blockIdx.x * GV_WARPS + warp) * GV_FPW;           // this warp's first feature
  float acc[GV_FPW][MT];
#pragma unroll
  for (int f = 0; f < GV_FPW; ++f)
#pragma unroll
    for (int t = 0; t < MT; ++t) acc[f][t] = 0.f;
  const Tw* wrow[GV_FPW];
#pragma unroll
  for (int f = 0; f < GV_FPW; ++f) wrow[f] = W + (size_t)min(f0 + f, N - 1) * ldw;     // rows past N repeat the last (not stored)
  pdl_wait();
  for (int k0 = 0; k0 < K; k0 += GV_CHUNK) {
    const int kc = min(GV_CHUNK, K - k0);
    __syncthreads();                                   // the chunk before has been used
    for (int e = tid; e < MT * GV_CHUNK; e += GV_WARPS * 32) {
      const int t = e / GV_CHUNK, k = e - t * GV_CHUNK;
      xs[t][k] = (t < M && k < kc) ? to_float(A[(size_t)t * lda + k0 + k]) : 0.f;
    }
    __syncthreads();
    if (VEC) {
#pragma unroll(GV_FPW == 1 ? 4 : 2)
      for (int k = lane * 4; k < kc; k += 128) {
        float w[GV_FPW][4];
#pragma unroll
        for (int f = 0; f < GV_FPW; ++f) Vec4<Tw>::load(wrow[f] + k0 + k, w[f]);
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const float4 x = *(const float4*)&xs[t][k];
#pragma unroll
          for (int f = 0; f < GV_FPW; ++f) {
            acc[f][t] = fmaf(x.x, w[f][0], acc[f][t]);
            acc[f][t] = fmaf(x.y, w[f][1], acc[f][t]);
            acc[f][t] = fmaf(x.z, w[f][2], acc[f][t]);
            acc[f][t] = fmaf(x.w, w[f][3], acc[f][t]);
          }
        }
      }
    } else {
      for (int k = lane; k < kc; k += 32) {
#pragma unroll
        for (int f = 0; f < GV_FPW; ++f) {
          const float w = to_float(wrow[f][k0 + k]);
#pragma unroll
          for (int t = 0; t < MT; ++t) acc[f][t] = fmaf(xs[t][k], w, acc[f][t]);
        }
      }
    }
  }
#pragma unroll
  for (int f = 0; f < GV_FPW; ++f)
#pragma unroll
    for (int t = 0; t < MT; ++t) acc[f][t] = warp_sum(acc[f][t]);
  if (lane == 0) {
#pragma unroll
    for (int f = 0; f < GV_FPW; ++f) {
      const int n = f0 + f;
      if (n >= N) continue;
      const float b = bias ? bias[n] : 0.f;
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        if (t >= M) continue;
        To* dst = C + (size_t)t * ldc + n;
        const float v = acc[f][t] + b;
        if (MODE == 1) *dst = from_float<To>(to_float(*dst) + v);
        else *dst = from_float<To>(v);
      }
    }
  }
}

template <typename Ta, typename Tw, typename To, int MODE>
static void launch_gemv_rows(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M,
                             int N, int K, cudaStream_t stream) {
  const bool vec = K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0;
  // four features to a warp unless that leaves fewer than two blocks to an SM
  const bool wide = (N + GV_WARPS * 4 - 1) / (GV_WARPS * 4) >= 2 * sm_count();
  const int fpw = wide ? 4 : 1;
  const unsigned grid = (unsigned)((N + GV_WARPS * fpw - 1) / (GV_WARPS * fpw));
#define WPC_GEMV(MT_, VEC_)                                                                                        \
  do {                                                                                                             \
    if (wide)                                                                                                      \
      wpc::launch(gemv_simt_kernel<Ta, Tw, To, MODE, MT_, VEC_, 4>, grid, GV_WARPS * 32, 0, stream, (const Ta*)A,  \
                  lda, (const Tw*)W, ldw, bias, (To*)C, ldc, M, N, K);                                             \
    else                                                                                                           \
      wpc::launch(gemv_simt_kernel<Ta, Tw, To, MODE, MT_, VEC_, 1>, grid, GV_WARPS * 32, 0, stream, (const Ta*)A,  \
                  lda, (const Tw*)W, ldw, bias, (To*)C, ldc, M, N, K);                                             \
  } while (0)
  if (vec) {
    if (M <= 1) WPC_GEMV(1, true); else if (M <= 2) WPC_GEMV(2, true); else if (M <= 4) WPC_GEMV(4, true);
    else if (M <= 8) WPC_GEMV(8, true); else WPC_GEMV(16, true);
  } else {
    if (M <= 1) WPC_GEMV(1, false); else if (M <= 2) WPC_GEMV(2, false); else if (M <= 4) WPC_GEMV(4, false);
    else if (M <= 8) WPC_GEMV(8, false); else WPC_GEMV(16, false);
  }
#undef WPC_GEMV
}

constexpr int GV_MAX_ROWS = 16;

template <typename Ta, typename Tw>
static int launch_simt(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc,
                       int out_dtype, int accumulate, int M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
  if (accumulate && out_dtype != WPC_DTYPE_F32) return WPC_ERR_BAD_ARGUMENT;
  if (M <= GV_MAX_ROWS) {            // few rows: stream the weights once (see gemv_simt_kernel)
    if (accumulate) launch_gemv_rows<Ta, Tw, float, 1>(A, lda, W, ldw, bias, C, ldc, M, N, K, stream);
    else if (out_dtype == WPC_DTYPE_F32) launch_gemv_rows<Ta, Tw, float, 0>(A, lda, W, ldw, bias, C, ldc, M, N, K, stream);
    else if (out_dtype == WPC_DTYPE_BF16) launch_gemv_rows<Ta, Tw, __nv_bfloat16, 0>(A, lda, W, ldw, bias, C, ldc, M, N, K, stream);
    else return WPC_ERR_BAD_ARGUMENT;
    return launch_status();
  }
  if (accumulate) {
    wpc::launch(gemm_simt_kernel<Ta, Tw, float, 1>, grid, SG_THREADS, 0, stream, (const Ta*)A, lda, (const Tw*)W, ldw, bias,
                                                                       (float*)C, ldc, M, N, K);
  } else if (out_dtype == WPC_DTYPE_F32) {
    wpc::launch(gemm_simt_kernel<Ta, Tw, float, 0>, grid, SG_THREADS, 0, stream, (const Ta*)A, lda, (const Tw*)W, ldw, bias,
                                                                       (float*)C, ldc, M, N, K);
  } else if (out_dtype == WPC_DTYPE_BF16) {
    wpc::launch(gemm_simt_kernel<Ta, Tw, __nv_bfloat16, 0>, grid, SG_THREADS, 0, stream, 
        (const Ta*)A, lda, (const Tw*)W, ldw, bias, (__nv_bfloat16*)C, ldc, M, N, K);
  } else {
    return WPC_ERR_BAD_ARGUMENT;
  }
  return launch_status();
}

}  // namespace wpc

using namespace wpc;

extern "C" int wpc_gemm_simt(const void* A, int a_dtype, int lda, const void* W, int w_dtype, int ldw,
                             const float* bias, void* C, int out_dtype, int ldc, int accumulate, int M, int N,
                             int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return WPC_ERR_BAD_ARGUMENT;
  if (a_dtype == WPC_DTYPE_F32 && w_dtype == WPC_DTYPE_F32)
    return launch_simt<float, float>(A, lda, W, ldw, bias, C, ldc, out_dtype, accumulate, M, N, K, stream);
  if (a_dtype == WPC_DTYPE_BF16 && w_dtype == WPC_DTYPE_BF16)
    return launch_simt<__nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, bias, C, ldc, out_dtype, accumulate, M, N, K,
                                                     stream);
  if (a_dtype == WPC_DTYPE_F32 && w_dtype == WPC_DTYPE_BF16)
    return launch_simt<float, __nv_bfloat16>(A, lda, W, ldw, bias, C, ldc, out_dtype, accumulate, M, N, K, stream);
  if (a_dtype == WPC_DTYPE_BF16 && w_dtype == WPC_DTYPE_F32)
    return launch_simt<__nv_bfloat16, float>(A, lda, W, ldw, bias, C, ldc, out_dtype, accumulate, M, N, K, stream);
  return WPC_ERR_BAD_ARGUMENT;
}
