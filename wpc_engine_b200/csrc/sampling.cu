// Picking the next token from float32 logits: greedy (the first strictly greatest value,
// banned ids skipped; wpc-runtime/src/sampling.rs:3-13, 35-51) or, with a temperature, a
// draw from softmax(logits / T) by inverse CDF in index order with one counter-based uniform
// number per draw.  A thread-block cluster of up to 8 CTAs takes a row (a row of 152,064 logits
// is 608 KB: one CTA would read it at a fraction of the memory bandwidth); rank r owns the r-th
// contiguous part of the vocabulary and, for a draw, each of its threads a contiguous range of
// that, so that the cumulative sums run in index order.  The ranks exchange their maxima, their
// sums and their picks through one another's shared memory.
#include "api.h"
#include "common.cuh"

namespace wpc {

constexpr int SP_THREADS = 512;
constexpr int SP_MAX_RANKS = 8;

__device__ __forceinline__ bool is_banned(int i, const int* banned, int n_banned) {
  for (int j = 0; j < n_banned; ++j)
    if (banned[j] == i) return true;
  return false;
}

// seq_state rows: [position, seed, request number, tokens drawn]
__global__ void __launch_bounds__(SP_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const int* __restrict__ slots,
              long long* __restrict__ seq_state, float temperature, const int* __restrict__ banned,
              int n_banned, int* __restrict__ out, int C) {
  pdl_trigger();
  __shared__ float s_val[SP_THREADS];
  __shared__ int s_idx[SP_THREADS];
  __shared__ float s_scan[SP_THREADS];
  __shared__ float r_val[SP_MAX_RANKS];        // every rank's maximum, its index, its sum and its pick,
  __shared__ int r_idx[SP_MAX_RANKS];          // written by the ranks themselves
  __shared__ float r_sum[SP_MAX_RANKS];
  __shared__ int r_pick[SP_MAX_RANKS];
  const int row = blockIdx.x / C, tid = threadIdx.x;
  const int rank = (int)cluster_rank();
  const float* z = logits + (size_t)row * V;
  // this rank's part of the vocabulary (multiples of 4 elements, so that parts start aligned alike)
  const int part = (((V + C - 1) / C) + 3) & ~3;
  const int p_lo = min(V, rank * part), p_hi = min(V, p_lo + part);
  const int chunk = (p_hi - p_lo + SP_THREADS - 1) / SP_THREADS;
  const int lo = min(p_hi, p_lo + tid * chunk), hi = min(p_hi, lo + chunk);
  cluster_sync_all();                          // every rank runs: its shared memory may be written
  pdl_wait();

  // the first strictly greatest value: threads stride over the part (coalesced); among equal
  // values the lowest index wins, within a thread by order and between threads by comparison
  float best = -INFINITY;
  int best_i = -1;
  for (int i = p_lo + tid; i < p_hi; i += SP_THREADS) {
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
  if (tid < C) {                               // this rank's best goes to every rank
    st_peer_b32(peer_smem((uint32_t)__cvta_generic_to_shared(r_val + rank), (uint32_t)tid), __float_as_uint(s_val[0]));
    st_peer_b32(peer_smem((uint32_t)__cvta_generic_to_shared(r_idx + rank), (uint32_t)tid), (uint32_t)s_idx[0]);
  }
  cluster_sync_all();
  float vmax = -INFINITY;
  int arg = -1;
  for (int r = 0; r < C; ++r)                  // parts ascend with the rank: the first of equal values wins
    if (r_idx[r] >= 0 && (arg < 0 || r_val[r] > vmax)) {
      vmax = r_val[r];
      arg = r_idx[r];
    }
  const bool nothing = arg < 0;                // nothing comparable: 0, as sampling.rs:4 starts
  if (nothing) arg = 0;
  long long* st = seq_state + (size_t)slots[row] * 4;

  if (!(temperature > 0.f) || nothing) {
    if (tid == 0 && rank == 0) {
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
  if (tid < C)
    st_peer_b32(peer_smem((uint32_t)__cvta_generic_to_shared(r_sum + rank), (uint32_t)tid),
                __float_as_uint(s_scan[SP_THREADS - 1]));
  cluster_sync_all();
  float total = 0.f, ahead = 0.f;              // the sums of all parts, and of the parts before this one, in rank order
  for (int r = 0; r < C; ++r) {
    if (r == rank) ahead = total;
    total += r_sum[r];
  }
  uint64_t r64 = mix64((uint64_t)st[1]);
  r64 = mix64(r64 ^ (uint64_t)st[2]);
  r64 = mix64(r64 ^ (uint64_t)st[3]);
  const float u = (float)(r64 >> 40) * (1.0f / 16777216.0f);
  const float target = u * total;
  if (tid == 0) s_idx[0] = -1;                 // this rank's pick
  __syncthreads();
  const float before = ahead + s_scan[tid] - sum;
  if (hi > lo && target >= before && target < ahead + s_scan[tid]) {
    // the first index of this range whose cumulative sum exceeds the target
    float c = before;
    int pick = -1;
    for (int i = lo; i < hi; ++i) {
      if (n_banned && is_banned(i, banned, n_banned)) continue;
      c += expf((z[i] - vmax) * inv_t);
      pick = i;
      if (c > target) break;
    }
    if (pick >= 0) atomicMax(&s_idx[0], pick);
  }
  __syncthreads();
  if (tid == 0) st_peer_b32(peer_smem((uint32_t)__cvta_generic_to_shared(r_pick + rank), 0u), (uint32_t)s_idx[0]);
  cluster_sync_all();
  if (tid == 0 && rank == 0) {
    int pick = -1;
    for (int r = 0; r < C; ++r) pick = max(pick, r_pick[r]);
    out[row] = pick >= 0 ? pick : arg;         // rounding left no range: the most likely token
    st[3] += 1;
  }
}

}  // namespace wpc

extern "C" int wpc_sample(const float* logits, int n_rows, int V, const int* slots, long long* seq_state,
                          float temperature, const int* banned, int n_banned, int* out, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0) return WPC_ERR_BAD_ARGUMENT;
  // a rank for every 16 Ki logits, 8 at most; few rows of a small vocabulary need no cluster
  int ranks = V / 16384;
  ranks = ranks < 1 ? 1 : (ranks > wpc::SP_MAX_RANKS ? wpc::SP_MAX_RANKS : ranks);
  wpc::launch_clusters(wpc::sample_kernel, dim3((unsigned)(n_rows * ranks)), wpc::SP_THREADS, 0, stream, (unsigned)ranks,
                       logits, V, slots, seq_state, temperature, banned, n_banned, out, ranks);
  return wpc::launch_status();
}
