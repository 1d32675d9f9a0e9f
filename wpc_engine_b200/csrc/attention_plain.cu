// Attention over the paged cache, the plain way: one block per (query token, query head),
// any head size, any context length, float32 arithmetic with an online softmax over chunks
// of keys.  It is the attention of the true 32-bit path and the plain twin of the fast
// kernels (wpc-runtime/src/model.rs:476-510).  When the queries are few and their contexts
// long (a decode step of the 32-bit path), the keys of a query are divided evenly among
// several blocks, whose partial results a second kernel adds up in order.
#include "api.h"
#include "common.cuh"

namespace wpc {

constexpr int AP_THREADS = 128;

// four consecutive elements of a key row as floats (the row starts 16-byte aligned when hd is a multiple of 4)
__device__ __forceinline__ float4 load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 t = *(const uint2*)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&t.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&t.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
constexpr int AP_CHUNK = 512;        // keys per chunk; their scores live in shared memory

template <typename T>
__global__ void __launch_bounds__(AP_THREADS)
attention_plain_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                       const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                       const int* __restrict__ page_table, int table_width,
                       const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                       int nh, int nkv, int hd, float scale, int window, float* __restrict__ part) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float smem[];
  float* qs = smem;                    // [hd]
  float* ps = smem + hd;               // [AP_CHUNK]
  __shared__ float red[32];
  const int t = blockIdx.x, h = blockIdx.y;
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int b = seq_of_token[t];
  const int* table = page_table + (size_t)b * table_width;
  // this block's share of the keys that the query sees (all of them with one block to a query)
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_splits = gridDim.z, per = (pos - first + 1 + n_splits - 1) / n_splits;
  const int lo = first + (int)blockIdx.z * per;
  const int n_keys = max(min(pos + 1, lo + per) - lo, 0);

  const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int d = threadIdx.x; d < hd; d += AP_THREADS) qs[d] = to_float(qrow[d]);
  __syncthreads();

  float m_run = -INFINITY, l_run = 0.f;
  float acc[2] = {0.f, 0.f};           // outputs d = tid and d = tid + AP_THREADS (hd <= 256)

  for (int c0 = 0; c0 < n_keys; c0 += AP_CHUNK) {
    const int cn = min(AP_CHUNK, n_keys - c0);
    float m_loc = -INFINITY;
    for (int j = threadIdx.x; j < cn; j += AP_THREADS) {
      const int p = lo + c0 + j;
      const int page = table[p / WPC_PAGE];
      const T* kr = k_pages + (((size_t)page * nkv + kvh) * WPC_PAGE + p % WPC_PAGE) * hd;
      float dot = 0.f;
      if ((hd & 3) == 0) {                              // the same order of additions, four elements a load
        for (int d = 0; d < hd; d += 4) {
          const float4 kv = load4(kr + d);
          dot = fmaf(qs[d], kv.x, dot);
          dot = fmaf(qs[d + 1], kv.y, dot);
          dot = fmaf(qs[d + 2], kv.z, dot);
          dot = fmaf(qs[d + 3], kv.w, dot);
        }
      } else {
        for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_float(kr[d]), dot);
      }
      dot *= scale;
      ps[j] = dot;
      m_loc = fmaxf(m_loc, dot);
    }
    m_loc = block_max(m_loc, red);
    const float m_new = fmaxf(m_run, m_loc);
    const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    float l_loc = 0.f;
    for (int j = threadIdx.x; j < cn; j += AP_THREADS) {
      const float e = expf(ps[j] - m_new);
      ps[j] = e;
      l_loc += e;
    }
    l_loc = block_sum(l_loc, red);       // also orders the writes of ps before the reads below
    l_run = l_run * corr + l_loc;
    m_run = m_new;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int d = threadIdx.x + u * AP_THREADS;
      if (d < hd) {
        float a = acc[u] * corr;
        for (int j = 0; j < cn;) {                       // page by page: one look-up for up to 64 keys
          const int p = lo + c0 + j;
          const int in_page = p % WPC_PAGE, n = min(cn - j, WPC_PAGE - in_page);
          const T* vr = v_pages + (((size_t)table[p / WPC_PAGE] * nkv + kvh) * WPC_PAGE + in_page) * hd + d;
          for (int i = 0; i < n; ++i) a = fmaf(ps[j + i], to_float(vr[(size_t)i * hd]), a);
          j += n;
        }
        acc[u] = a;
      }
    }
    __syncthreads();
  }
  if (n_splits > 1) {
    // unnormalised outputs, then the running maximum and sum: [token][head][split][hd + 2]
    float* prow = part + (((size_t)t * nh + h) * n_splits + blockIdx.z) * (hd + 2);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int d = threadIdx.x + u * AP_THREADS;
      if (d < hd) prow[d] = acc[u];
    }
    if (threadIdx.x == 0) {
      prow[hd] = m_run;
      prow[hd + 1] = l_run;
    }
    return;
  }
  T* orow = out + (size_t)t * out_stride + (size_t)h * hd;
  const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int d = threadIdx.x + u * AP_THREADS;
    if (d < hd) orow[d] = from_float<T>(acc[u] * inv);
  }
}

// Adds up the partial results of a query's blocks, in block order.
template <typename T>
__global__ void attention_plain_combine_kernel(const float* __restrict__ part, T* __restrict__ out, int out_stride, int nh,
                                               int hd, int n_splits) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* prow = part + ((size_t)t * nh + h) * n_splits * (hd + 2);
  float m = -INFINITY;
  for (int z = 0; z < n_splits; ++z) m = fmaxf(m, prow[(size_t)z * (hd + 2) + hd]);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int z = 0; z < n_splits; ++z) {
      const float* pz = prow + (size_t)z * (hd + 2);
      const float f = pz[hd] == -INFINITY ? 0.f : expf(pz[hd] - m);
      num = fmaf(f, pz[d], num);
      den = fmaf(f, pz[hd + 1], den);
    }
    out[(size_t)t * out_stride + (size_t)h * hd + d] = from_float<T>(den > 0.f ? num / den : 0.f);
  }
}

}  // namespace wpc

using namespace wpc;

extern "C" int wpc_attention_plain(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                   const void* k_pages, const void* v_pages, const int* page_table,
                                   int table_width, const int* seq_of_token, const int* positions, int T, int nh,
                                   int nkv, int hd, float scale, int window, int n_splits, float* part,
                                   cudaStream_t stream) {
  // n_splits > 1: that many blocks share the keys of each query; part: float32 scratch of
  // T * nh * n_splits * (hd + 2) elements for their partial results
  if (T <= 0) return 0;
  if (hd < 1 || hd > 2 * AP_THREADS || nkv < 1 || nh % nkv) return WPC_ERR_UNSUPPORTED;
  if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && !part)) return WPC_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)(hd + AP_CHUNK) * sizeof(float);
  dim3 grid(T, nh, n_splits);
  WPC_DISPATCH_DTYPE(dtype, Tt,
                     wpc::launch(attention_plain_kernel<Tt>, grid, AP_THREADS, smem, stream, 
                         (const Tt*)q, q_stride, (Tt*)out, out_stride, (const Tt*)k_pages, (const Tt*)v_pages,
                         page_table, table_width, seq_of_token, positions, nh, nkv, hd, scale, window, part));
  int rc = launch_status();
  if (rc || n_splits == 1) return rc;
  WPC_DISPATCH_DTYPE(dtype, Tt,
                     wpc::launch(attention_plain_combine_kernel<Tt>, dim3(T, nh), 128, 0, stream, (const float*)part,
                                 (Tt*)out, out_stride, nh, hd, n_splits));
  return launch_status();
}
