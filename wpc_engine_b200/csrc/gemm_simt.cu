// C[M,N] = A[M,K] . W[N,K]^T (+ bias), float32 multiply-add on the CUDA cores only: the
// matrix product of the true 32-bit path, and the plain twin of the tensor-core product.
// Each output is one dot product accumulated in float32 in ascending k
// (wpc-runtime/src/weights.rs:59-78), so a row's result does not depend on the other rows.
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

template <typename Ta, typename Tw>
static int launch_simt(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc,
                       int out_dtype, int accumulate, int M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
  if (accumulate) {
    if (out_dtype != WPC_DTYPE_F32) return WPC_ERR_BAD_ARGUMENT;
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
