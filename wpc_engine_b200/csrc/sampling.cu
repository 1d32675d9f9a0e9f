// Picking the next token from float32 logits: greedy (the first strictly greatest value,
// banned ids skipped; wpc-runtime/src/sampling.rs:3-13, 35-51) or, with a temperature, a
// draw from softmax(logits / T) by inverse CDF in index order with one counter-based uniform
// number per draw.  One block per row.  The maximum is found with coalesced strided reads; for
// a draw each thread then owns a contiguous range of the vocabulary, so that the cumulative
// sums run in index order.
#include "api.h"
#include "common.cuh"

namespace wpc {

constexpr int SP_THREADS = 1024;

__device__ __forceinline__ bool is_banned(int i, const int* banned, int n_banned) {
  for (int j = 0; j < n_banned; ++j)
    if (banned[j] == i) return true;
  return false;
}

// seq_state rows: [position, seed, request number, tokens drawn]
__global__ void __launch_bounds__(SP_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const int* __restrict__ slots,
              long long* __restrict__ seq_state, float temperature, const int* __restrict__ banned,
              int n_banned, int* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  __shared__ float s_val[SP_THREADS];
  __shared__ int s_idx[SP_THREADS];
  __shared__ float s_scan[SP_THREADS];
  __shared__ int s_pick;
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* z = logits + (size_t)row * V;
  const int chunk = (V + SP_THREADS - 1) / SP_THREADS;
  const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);

  // the first strictly greatest value: threads stride over the row (coalesced); among equal
  // values the lowest index wins, within a thread by order and between threads by comparison
  float best = -INFINITY;
  int best_i = -1;
  for (int i = tid; i < V; i += SP_THREADS) {
    const float v = z[i];
    if (v > best && !(n_banned && is_banned(i, banned, n_banned))) {
      best = v;
      best_i = i;
    }
  }
  s_val[tid] = best;
  s_idx[tid] = best_i;
  __syncthreads();
  for (int s = SP_THREADS / 2; s > 0; s >>= 1) {
    if (tid < s) {
      const float ov = s_val[tid + s];
      const int oi = s_idx[tid + s];
      const bool take = oi >= 0 && (s_idx[tid] < 0 || ov > s_val[tid] || (ov == s_val[tid] && oi < s_idx[tid]));
      if (take) {
        s_val[tid] = ov;
        s_idx[tid] = oi;
      }
    }
    __syncthreads();
  }
  const float vmax = s_val[0];
  const int arg = s_idx[0] < 0 ? 0 : s_idx[0];     // nothing comparable: 0, as sampling.rs:4 starts
  long long* st = seq_state + (size_t)slots[row] * 4;

  if (!(temperature > 0.f) || s_idx[0] < 0) {
    if (tid == 0) {
      out[row] = arg;
      st[3] += 1;
    }
    return;
  }

  const float inv_t = 1.0f / temperature;
  float sum = 0.f;
  for (int i = lo; i < hi; ++i)
    if (!(n_banned && is_banned(i, banned, n_banned))) sum += expf((z[i] - vmax) * inv_t);
  // inclusive scan of the per-thread sums, in thread (= index) order
  s_scan[tid] = sum;
  __syncthreads();
  for (int off = 1; off < SP_THREADS; off <<= 1) {
    const float add = tid >= off ? s_scan[tid - off] : 0.f;
    __syncthreads();
    s_scan[tid] += add;
    __syncthreads();
  }
  const float total = s_scan[SP_THREADS - 1];
  uint64_t r = mix64((uint64_t)st[1]);
  r = mix64(r ^ (uint64_t)st[2]);
  r = mix64(r ^ (uint64_t)st[3]);
  const float u = (float)(r >> 40) * (1.0f / 16777216.0f);
  const float target = u * total;
  if (tid == 0) s_pick = -1;
  __syncthreads();
  const float before = s_scan[tid] - sum;
  if (hi > lo && target >= before && target < s_scan[tid]) {
    // the first index of this range whose cumulative sum exceeds the target
    float c = before;
    int pick = -1;
    for (int i = lo; i < hi; ++i) {
      if (n_banned && is_banned(i, banned, n_banned)) continue;
      c += expf((z[i] - vmax) * inv_t);
      pick = i;
      if (c > target) break;
    }
    if (pick >= 0) atomicMax(&s_pick, pick);
  }
  __syncthreads();
  if (tid == 0) {
    out[row] = s_pick >= 0 ? s_pick : arg;       // rounding left no range: the most likely token
    st[3] += 1;
  }
  (void)red;
}

}  // namespace wpc

extern "C" int wpc_sample(const float* logits, int n_rows, int V, const int* slots, long long* seq_state,
                          float temperature, const int* banned, int n_banned, int* out, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0) return WPC_ERR_BAD_ARGUMENT;
  wpc::launch(wpc::sample_kernel, n_rows, wpc::SP_THREADS, 0, stream, logits, V, slots, seq_state, temperature, banned,
                                                            n_banned, out);
  return wpc::launch_status();
}
