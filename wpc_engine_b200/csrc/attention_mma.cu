// bfloat16 attention over the paged cache on the tensor cores, with an online softmax in
// float32 (wpc-runtime/src/model.rs:476-510 is the arithmetic: scaled scores of a query
// against the visible keys, softmax, weighted values).
//
// The query heads that share a KV head are stacked along the MMA's row dimension, so a page
// of keys and values is read once for the whole group.
//
//   decode   one query token per sequence.  A fixed grid of CTAs shares all (sequence, kv
//            head, page) work evenly; the 16 MMA rows hold the group's query heads; the four
//            warps of a CTA take the four 16-key quarters of each 64-key page and are merged
//            at the end; partial results of a pair that spans CTAs are combined by the last
//            of them to finish.  With few pairs of about equal lengths, one or several
//            thread-block clusters take a pair instead and add up through one another's shared
//            memory (see decode_cluster_kernel).
//   prefill  any number of new tokens per sequence.  grid = (row tiles, kv heads,
//            sequences); a tile is 64 rows of (token, head-in-group), 16 per warp; every warp
//            walks the pages up to the tile's last visible key.
//
// Keys and values of a page ([64, head_dim], contiguous) are copied to shared memory with
// cp.async, a ring of pages in flight (3 when two CTAs share an SM, 6 when one has it alone),
// rows padded by 16 bytes so that ldmatrix is free of bank
// conflicts.  head_dim: multiples of 16 up to 128 (other sizes take the plain kernel).
#include "api.h"
#include "common.cuh"

namespace wpc {
namespace fa {

constexpr int PAGE = WPC_PAGE;
constexpr int THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x in one instruction (x <= 0 here; results below the normal range are zero)
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

template <int HD>
struct Cfg {
  static constexpr int STRIDE = HD + 8;                   // elements per padded row
  static constexpr int PAGE_ELEMS = PAGE * STRIDE;
  static constexpr int SMEM_BYTES = 4 * PAGE_ELEMS * 2;   // K and V, two buffers each
};

// Copies one page ([64, HD], contiguous) into padded shared memory rows.
template <int HD>
__device__ __forceinline__ void load_page(__nv_bfloat16* dst, const __nv_bfloat16* src, int tid) {
  constexpr int CPR = HD / 8;                    // 16-byte chunks per row
  for (int c = tid; c < PAGE * CPR; c += THREADS) {
    const int row = c / CPR, col = c - row * CPR;
    cp_async16(dst + row * Cfg<HD>::STRIDE + col * 8, src + row * HD + col * 8);
  }
}

// s[nt] (16 rows x 8 keys each) = q (16 x HD) . K[key0 + 8 nt + .., :]^T for NT key tiles.
template <int HD, int NT>
__device__ __forceinline__ void scores(const uint32_t (&qf)[HD / 16][4], const __nv_bfloat16* ks, int key0,
                                       float (&s)[NT][4], int lane) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      const int key = key0 + np * 16 + (mat >> 1) * 8 + r;
      const int dim = kk * 16 + (mat & 1) * 8;
      ldmatrix_x4(b, ks + key * Cfg<HD>::STRIDE + dim);
      mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
      mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
    }
  }
}

// o (16 x HD) += p (16 x 8 NT keys, bf16 fragments) . V[key0 .., :]
template <int HD, int NT>
__device__ __forceinline__ void weighted_values(const uint32_t (&pf)[NT / 2][4], const __nv_bfloat16* vs, int key0,
                                                float (&o)[HD / 8][4], int lane) {
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kc = 0; kc < NT / 2; ++kc) {
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      uint32_t b[4];
      const int key = key0 + kc * 16 + (mat & 1) * 8 + r;
      const int dim = dp * 16 + (mat >> 1) * 8;
      ldmatrix_x4_trans(b, vs + key * Cfg<HD>::STRIDE + dim);
      mma_bf16(o[2 * dp], pf[kc], b[0], b[1]);
      mma_bf16(o[2 * dp + 1], pf[kc], b[2], b[3]);
    }
  }
}

// One online-softmax step for the two rows that a thread holds (lane/4 and lane/4 + 8).
// `s` holds scaled scores (log2 domain) with -inf where masked; on return it holds the
// probabilities' numerators; m, l, o are updated (l is a per-thread partial sum).
template <int HD, int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[HD / 8][4]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * h], s[nt][2 * h + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[h], mx);
    const bool none = m_new == -INFINITY;
    // (one instruction an exponential: the arguments are at most 0, and exp2f's care for results
    // below the normal range costs four more for each score of every page)
    const float alpha = none ? 1.f : ex2_fast(m[h] - m_new);
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float p0 = none ? 0.f : ex2_fast(s[nt][2 * h] - m_new);
      const float p1 = none ? 0.f : ex2_fast(s[nt][2 * h + 1] - m_new);
      s[nt][2 * h] = p0;
      s[nt][2 * h + 1] = p1;
      sum += p0 + p1;
    }
    l[h] = l[h] * alpha + sum;
    m[h] = m_new;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      o[d][2 * h] *= alpha;
      o[d][2 * h + 1] *= alpha;
    }
  }
}

template <int NT>
__device__ __forceinline__ void to_fragments(const float (&s)[NT][4], uint32_t (&pf)[NT / 2][4]) {
#pragma unroll
  for (int kc = 0; kc < NT / 2; ++kc) {
    pf[kc][0] = pack_bf16(s[2 * kc][0], s[2 * kc][1]);
    pf[kc][1] = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
    pf[kc][2] = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]);
    pf[kc][3] = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
  }
}

// Query fragments of the two rows (row_lo, row_hi) of this thread, straight from global memory;
// a null pointer gives a zero row.
template <int HD>
__device__ __forceinline__ void load_q(uint32_t (&qf)[HD / 16][4], const __nv_bfloat16* row_lo,
                                       const __nv_bfloat16* row_hi, int lane) {
  const int c = (lane & 3) * 2;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    qf[kk][0] = row_lo ? *(const uint32_t*)(row_lo + kk * 16 + c) : 0u;
    qf[kk][1] = row_hi ? *(const uint32_t*)(row_hi + kk * 16 + c) : 0u;
    qf[kk][2] = row_lo ? *(const uint32_t*)(row_lo + kk * 16 + c + 8) : 0u;
    qf[kk][3] = row_hi ? *(const uint32_t*)(row_hi + kk * 16 + c + 8) : 0u;
  }
}

// ---- decode -------------------------------------------------------------------------------------
// The work of a decode step is the list of (sequence, kv head, page) triples that the queries
// see, in that order.  A fixed grid of CTAs divides the list evenly, so that every SM streams
// about the same number of pages whatever the sequences' lengths are.  A CTA walks its share
// as segments of one (sequence, kv head) pair each.  A pair that lies inside one CTA is
// finished there; a pair that spans several CTAs gets one partial result (unnormalised output,
// running maximum, running sum) from each, and the CTA that draws the pair's last ticket
// combines them in CTA order, so the result does not depend on who came last.  Nobody waits.
//
// part_o: [(CTAs + pairs), 16, HD] float32; part_ml: [(CTAs + pairs), 16, 2]; the partial of CTA
// c for pair k lives at slot c + k (consecutive pairs share at most one CTA, so slots are unique).
constexpr int MAX_DECODE_SEQS = 1024;
// Whether the decode kernels start the copies of earlier pages ahead of their dependency wait.
inline int& early_pages() {
  static int on = 1;
  return on;
}
// Pages in the ring of a decode CTA: 3 with two CTAs to an SM; 6 when there are so few CTAs that
// each has an SM to itself (few sequences), so that all of a CTA's pages are on their way at once.
constexpr int DECODE_STAGES_SHARED = 3;
constexpr int DECODE_STAGES_ALONE = 6;
constexpr int MAX_SEGMENT_PAGES = 512;

template <int HD, int DECODE_STAGES>
__global__ void __launch_bounds__(THREADS)
decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out, int out_stride,
              const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
              const int* __restrict__ page_table, int table_width, const int* __restrict__ ctx_lens, int B,
              int nh, int nkv, float scale_log2, int window, float* __restrict__ part_o,
              float* __restrict__ part_ml, int* __restrict__ counters, int smem_bytes, int early_pages) {
  pdl_trigger();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* ks = (__nv_bfloat16*)smem_raw;                       // [DECODE_STAGES][PAGE][STRIDE]
  __nv_bfloat16* vs = ks + DECODE_STAGES * Cfg<HD>::PAGE_ELEMS;
  __shared__ int s_cum[MAX_DECODE_SEQS + 1];                          // units before each sequence
  __shared__ int s_pages[MAX_SEGMENT_PAGES];                          // page numbers of the current segment
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rep = nh / nkv;
  const size_t page_elems = (size_t)nkv * PAGE * HD;

  // ---- units of each sequence, and their running sum ----
  for (int b = tid; b < B; b += THREADS) {
    const int pos = ctx_lens[b] - 1;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    s_cum[b + 1] = pos >= 0 ? (pos / PAGE - lo / PAGE + 1) * nkv : 0;
  }
  if (tid == 0) s_cum[0] = 0;
  __syncthreads();
  if (warp == 0) {
    // inclusive scan of s_cum[1..B]: each lane a contiguous chunk, then a scan of the chunk sums
    const int chunk = (B + 31) / 32;
    const int lo_i = 1 + lane * chunk, hi_i = min(B + 1, lo_i + chunk);
    int sum = 0;
    for (int i = lo_i; i < hi_i; ++i) sum += s_cum[i];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    int run = incl - sum;
    for (int i = lo_i; i < hi_i; ++i) {
      run += s_cum[i];
      s_cum[i] = run;
    }
  }
  __syncthreads();
  const int U = s_cum[B];
  const int per = (U + (int)gridDim.x - 1) / (int)gridDim.x;
  const int u0 = blockIdx.x * per, u1 = min(U, u0 + per);
  if (per == 0 || u0 >= u1) return;

  // the sequence that holds unit u0
  int b = 0;
  {
    int lo_b = 0, hi_b = B;                     // s_cum[lo_b] <= u0 < s_cum[hi_b]
    while (hi_b - lo_b > 1) {
      const int mid = (lo_b + hi_b) >> 1;
      if (s_cum[mid] <= u0) lo_b = mid; else hi_b = mid;
    }
    b = lo_b;
  }

  const int r_lo = lane >> 2, r_hi = r_lo + 8;                        // rows = heads of the group
  float* so = (float*)smem_raw;                         // merge area [4][16][HD] (after the pages are done)
  float* sm = so + 4 * 16 * HD;                         // [4][16]
  float* sl = sm + 4 * 16;                              // [4][16]

  for (int u = u0; u < u1;) {
    while (s_cum[b + 1] <= u) ++b;
    const int nb = (s_cum[b + 1] - s_cum[b]) / nkv;                   // pages that sequence b's query sees
    const int within = u - s_cum[b];
    const int g = within / nb, pg = within - g * nb;
    const int pair_start = s_cum[b] + g * nb, pair_end = pair_start + nb;
    const int seg_end = min(u1, pair_end);
    const int L = ctx_lens[b];
    const int pos = L - 1;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int blk0 = lo / PAGE + pg, blk1 = blk0 + (seg_end - u);
    // the segment's page numbers go to shared memory at once: a lookup per page in the loop
    // would put a trip to L2 before every copy
    const int* gtable = page_table + (size_t)b * table_width + blk0;
    const int n_seg = blk1 - blk0;
    for (int i = tid; i < min(n_seg, MAX_SEGMENT_PAGES); i += THREADS) s_pages[i] = gtable[i];
    __syncthreads();                                     // the page numbers are in shared memory for every thread
    auto page_of = [&](int blk) { const int i = blk - blk0; return i < MAX_SEGMENT_PAGES ? s_pages[i] : gtable[i]; };

    // A ring of DECODE_STAGES pages: two are in flight while one is computed.  Up to here only
    // the step's lengths and page numbers were read, which the host wrote before the step's
    // first kernel started.  The queries come from the kernel ahead, and so do the key and the
    // value of this step's token, which lie in the sequence's last page: those are read after
    // the dependency wait.  Every earlier page holds positions of earlier steps only, finished
    // long before this step began: a CTA's first segment fetches such pages while the kernel
    // ahead is still running (one commit a stage, in order, so that the counting of the loop
    // below holds whichever side of the wait a page was started on).
    const int last_blk = pos / PAGE;
    const bool early = u == u0;          // (later segments of a CTA begin after the wait anyway)
    int filled = 0;
    if (early) {
#pragma unroll
      for (; early_pages && filled < DECODE_STAGES - 1; ++filled) {
        if (blk0 + filled < blk1) {
          if (blk0 + filled == last_blk) break;
          const size_t src = (size_t)max(page_of(blk0 + filled), 0) * page_elems + (size_t)g * PAGE * HD;
          load_page<HD>(ks + filled * Cfg<HD>::PAGE_ELEMS, k_pages + src, tid);
          load_page<HD>(vs + filled * Cfg<HD>::PAGE_ELEMS, v_pages + src, tid);
        }
        cp_async_commit();
      }
      pdl_wait();
    }
    for (int i = filled; i < DECODE_STAGES - 1; ++i) {
      if (blk0 + i < blk1) {
        const size_t src = (size_t)max(page_of(blk0 + i), 0) * page_elems + (size_t)g * PAGE * HD;
        load_page<HD>(ks + i * Cfg<HD>::PAGE_ELEMS, k_pages + src, tid);
        load_page<HD>(vs + i * Cfg<HD>::PAGE_ELEMS, v_pages + src, tid);
      }
      cp_async_commit();
    }
    const __nv_bfloat16* qtok = q + (size_t)b * q_stride + (size_t)g * n_rep * HD;
    uint32_t qf[HD / 16][4];
    load_q<HD>(qf, r_lo < n_rep ? qtok + r_lo * HD : nullptr, r_hi < n_rep ? qtok + r_hi * HD : nullptr, lane);
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[d][i] = 0.f;
    for (int blk = blk0; blk < blk1; ++blk) {
      const int buf = (blk - blk0) % DECODE_STAGES;
      if (blk + DECODE_STAGES - 1 < blk1) {
        const int nbuf = (buf + DECODE_STAGES - 1) % DECODE_STAGES;
        const size_t src = (size_t)max(page_of(blk + DECODE_STAGES - 1), 0) * page_elems + (size_t)g * PAGE * HD;
        load_page<HD>(ks + nbuf * Cfg<HD>::PAGE_ELEMS, k_pages + src, tid);
        load_page<HD>(vs + nbuf * Cfg<HD>::PAGE_ELEMS, v_pages + src, tid);
      }
      cp_async_commit();
      cp_async_wait<DECODE_STAGES - 1>();
      __syncthreads();
      const int key0 = warp * 16;                                       // this warp's quarter of the page
      const int abs0 = blk * PAGE + key0;
      if (abs0 <= pos && abs0 + 15 >= lo) {
        float s[2][4];
        scores<HD, 2>(qf, ks + buf * Cfg<HD>::PAGE_ELEMS, key0, s, lane);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int kabs = abs0 + nt * 8 + (lane & 3) * 2 + (i & 1);
            s[nt][i] = (kabs >= lo && kabs <= pos) ? s[nt][i] * scale_log2 : -INFINITY;
          }
        softmax_step<HD, 2>(s, m, l, o);
        uint32_t pf[1][4];
        to_fragments<2>(s, pf);
        weighted_values<HD, 2>(pf, vs + buf * Cfg<HD>::PAGE_ELEMS, key0, o, lane);
      }
      __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the four warps (each saw a quarter of every page) through shared memory ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      const int c = d * 8 + (lane & 3) * 2;
      *(float2*)(so + (warp * 16 + r_lo) * HD + c) = make_float2(o[d][0], o[d][1]);
      *(float2*)(so + (warp * 16 + r_hi) * HD + c) = make_float2(o[d][2], o[d][3]);
    }
    if ((lane & 3) == 0) {
      sm[warp * 16 + r_lo] = m[0];
      sm[warp * 16 + r_hi] = m[1];
      sl[warp * 16 + r_lo] = l[0];
      sl[warp * 16 + r_hi] = l[1];
    }
    __syncthreads();
    const int pair = b * nkv + g;
    const int c_first = pair_start / per, c_last = (pair_end - 1) / per;
    const bool whole = c_first == c_last;                 // the pair lies inside this CTA
    const size_t slot = (size_t)blockIdx.x + pair;
    for (int e = tid; e < n_rep * HD; e += THREADS) {
      const int row = e / HD, d = e - row * HD;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, sm[w * 16 + row]);
      float acc = 0.f, Lsum = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = sm[w * 16 + row];
        const float f = (mw == -INFINITY) ? 0.f : ex2_fast(mw - M);
        acc += f * so[(w * 16 + row) * HD + d];
        Lsum += f * sl[w * 16 + row];
      }
      if (whole) {
        out[(size_t)b * out_stride + (size_t)(g * n_rep + row) * HD + d] =
            __float2bfloat16_rn(Lsum > 0.f ? __fdividef(acc, Lsum) : 0.f);
      } else {
        part_o[(slot * 16 + row) * HD + d] = acc;
        if (d == 0) {
          part_ml[(slot * 16 + row) * 2] = M;
          part_ml[(slot * 16 + row) * 2 + 1] = Lsum;
        }
      }
    }
    if (!whole) {
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int ticket = atomicAdd(counters + pair, 1);
        s_last = ticket == c_last - c_first;
        if (s_last) counters[pair] = 0;                    // ready for the next launch
      }
      __syncthreads();
      if (s_last) {
        // (every writer fenced its partial results before it took its ticket, and the copies below
        // read through L2, where those results are: no fence is needed on this side)
        // All partial results of the pair come into shared memory with one burst of cp.async
        // (loads through registers would go a few at a time, each batch a trip to L2), in
        // chunks of as many parts as fit; a warp per row turns maxima and sums into weights.
        const int n_parts = c_last - c_first + 1;
        const size_t slot0 = (size_t)c_first + pair;
        float* wm = (float*)smem_raw;                      // [16][n_parts] maximum, then the weight
        float* wl = wm + 16 * n_parts;                     // [16][n_parts] sum
        float* winv = wl + 16 * n_parts;                   // [16] 1 / total
        float* po_s = winv + 16;                           // [chunk][n_rep][HD] partial outputs
        const int chunk = max(1, min(n_parts, (smem_bytes - (2 * 16 * n_parts + 16) * 4) / (n_rep * HD * 4)));
        float acc[(16 * HD + THREADS - 1) / THREADS];
#pragma unroll
        for (int i = 0; i < (16 * HD + THREADS - 1) / THREADS; ++i) acc[i] = 0.f;
        for (int s0 = 0; s0 < n_parts; s0 += chunk) {
          const int ns = min(chunk, n_parts - s0);
          // rows of HD floats are 16-byte multiples: copy row by row, 16 bytes a thread
          for (int c = tid; c < ns * n_rep * (HD / 4); c += THREADS) {
            const int part = c / (n_rep * (HD / 4)), rem = c - part * (n_rep * (HD / 4));
            cp_async16(po_s + (size_t)part * n_rep * HD + rem * 4, part_o + ((slot0 + s0 + part) * 16) * HD + rem * 4);
          }
          cp_async_commit();
          if (s0 == 0) {
            // maxima and sums travel while the copies are in flight
            for (int e = tid; e < n_rep * n_parts; e += THREADS) {
              const int row = e / n_parts, sidx = e - row * n_parts;
              const float2 ml = __ldcg((const float2*)(part_ml + ((slot0 + sidx) * 16 + row) * 2));
              wm[row * n_parts + sidx] = ml.x;
              wl[row * n_parts + sidx] = ml.y;
            }
            __syncthreads();                               // wm, wl are written
            for (int row = warp; row < n_rep; row += THREADS / 32) {
              float M = -INFINITY;
              for (int sidx = lane; sidx < n_parts; sidx += 32) M = fmaxf(M, wm[row * n_parts + sidx]);
              M = warp_max(M);
              float Lsum = 0.f;
              for (int sidx = lane; sidx < n_parts; sidx += 32) {
                const float ms = wm[row * n_parts + sidx];
                const float f = (ms == -INFINITY) ? 0.f : ex2_fast(ms - M);
                wm[row * n_parts + sidx] = f;
                Lsum += f * wl[row * n_parts + sidx];
              }
              Lsum = warp_sum(Lsum);
              if (lane == 0) winv[row] = Lsum > 0.f ? 1.f / Lsum : 0.f;
            }
          }
          cp_async_wait<0>();
          __syncthreads();
          int i = 0;
          for (int e = tid; e < n_rep * HD; e += THREADS, ++i) {
            const int row = e / HD;
            float a = acc[i];
            for (int sidx = 0; sidx < ns; ++sidx) a += wm[row * n_parts + s0 + sidx] * po_s[(size_t)sidx * n_rep * HD + e];
            acc[i] = a;
          }
          __syncthreads();                                 // po_s is reused by the next chunk
        }
        int i = 0;
        for (int e = tid; e < n_rep * HD; e += THREADS, ++i) {
          const int row = e / HD, d = e - row * HD;
          out[(size_t)b * out_stride + (size_t)(g * n_rep + row) * HD + d] = __float2bfloat16_rn(acc[i] * winv[row]);
        }
      }
    }
    __syncthreads();                                       // shared memory is reused by the next segment
    u = seg_end;
  }
}

// ---- decode, a cluster to a pair ------------------------------------------------------------------
// When the (sequence, kv head) pairs are few and about equally long, the CTAs of a pair form a
// thread-block cluster of C ranks (up to 16); rank r takes the r-th share of the pages that the pair's
// query sees.  The partial results do not go through global memory: every rank writes its
// unnormalised outputs for the r'-th share of the pair's n_rep * HD output elements straight
// into rank r''s shared memory, and its running maxima and sums into every rank's; one
// cluster barrier makes them visible, and every rank then normalises and writes its share of
// the output, adding the ranks in order.  No scratch, no tickets, no second pass.
// One long sequence alone leaves most SMs without work even with 16 ranks: then G clusters (groups)
// share a pair's pages, every group leaves its unnormalised sums and its maxima in global
// scratch (a few KB), and the cluster of the pair that takes the last ticket adds the G parts in order.
constexpr int CLUSTER_DECODE_MAX_OUT = 1024;      // n_rep * HD that the receive buffer takes
constexpr int CLUSTER_DECODE_MAX_RANKS = 16;      // beyond 8 a cluster needs the kernel's consent (see the launch)
constexpr int CLUSTER_DECODE_MAX_GROUPS = 16;     // clusters that share a pair's pages
constexpr int CLUSTER_SEGMENT_PAGES = 256;        // page numbers of a rank's share kept in shared memory

template <int HD, int DECODE_STAGES, bool GROUPED>
__global__ void __launch_bounds__(THREADS)
decode_cluster_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out, int out_stride,
                      const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                      const int* __restrict__ page_table, int table_width, const int* __restrict__ ctx_lens, int B,
                      int nh, int nkv, float scale_log2, int window, int C, int early_pages, int n_groups,
                      float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters) {
  pdl_trigger();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* ks = (__nv_bfloat16*)smem_raw;                       // [DECODE_STAGES][PAGE][STRIDE]
  __nv_bfloat16* vs = ks + DECODE_STAGES * Cfg<HD>::PAGE_ELEMS;
  __shared__ int s_last;
  __shared__ int s_pages[CLUSTER_SEGMENT_PAGES];                      // page numbers of this rank's share
  __shared__ __align__(16) float s_recv_o[CLUSTER_DECODE_MAX_OUT + 4 * CLUSTER_DECODE_MAX_RANKS];   // [rank][element of this rank's share]
  __shared__ __align__(8) float s_recv_ml[CLUSTER_DECODE_MAX_RANKS * 16 * 2];      // [rank][row][maximum, sum]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rep = nh / nkv;
  const size_t page_elems = (size_t)nkv * PAGE * HD;
  const int rank = (int)cluster_rank();
  // (the variant with one cluster to a pair is compiled on its own: the tail below is code that
  // runs once a launch, and every line that it does not need is a line more to fetch)
  const int G = GROUPED ? n_groups : 1;
  const int cl = blockIdx.x / C, pair = cl / G, grp = cl - pair * G, b = pair / nkv, g = pair - b * nkv;
  cluster_sync_all();                       // every rank runs: its shared memory may be written

  const int L = ctx_lens[b];
  const int pos = L - 1;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int nb = pos >= 0 ? pos / PAGE - lo / PAGE + 1 : 0;           // pages that the query sees
  const int g_base = nb / G, g_extra = nb - g_base * G;               // the first groups take a page more,
  const int g_blk0 = lo / PAGE + grp * g_base + min(grp, g_extra), g_nb = g_base + (grp < g_extra ? 1 : 0);
  const int base = g_nb / C, extra = g_nb - base * C;                 // and so do the first ranks of a group
  const int blk0 = g_blk0 + rank * base + min(rank, extra), blk1 = blk0 + base + (rank < extra ? 1 : 0);
  const int* gtable = page_table + (size_t)b * table_width + blk0;
  const int n_seg = blk1 - blk0;
  for (int i = tid; i < min(n_seg, CLUSTER_SEGMENT_PAGES); i += THREADS) s_pages[i] = gtable[i];
  __syncthreads();                                       // the page numbers are in shared memory for every thread
  auto page_of = [&](int blk) { const int i = blk - blk0; return i < CLUSTER_SEGMENT_PAGES ? s_pages[i] : gtable[i]; };

  // The first pages of the ring are started ahead of the dependency wait, except the sequence's
  // last page, which holds the key and value that the kernel ahead writes (see decode_kernel).
  const int last_blk = pos / PAGE;
  int filled = 0;
#pragma unroll
  for (; early_pages && filled < DECODE_STAGES - 1; ++filled) {
    if (blk0 + filled < blk1) {
      if (blk0 + filled == last_blk) break;
      const size_t src = (size_t)max(page_of(blk0 + filled), 0) * page_elems + (size_t)g * PAGE * HD;
      load_page<HD>(ks + filled * Cfg<HD>::PAGE_ELEMS, k_pages + src, tid);
      load_page<HD>(vs + filled * Cfg<HD>::PAGE_ELEMS, v_pages + src, tid);
    }
    cp_async_commit();
  }
  pdl_wait();
  for (int i = filled; i < DECODE_STAGES - 1; ++i) {
    if (blk0 + i < blk1) {
      const size_t src = (size_t)max(page_of(blk0 + i), 0) * page_elems + (size_t)g * PAGE * HD;
      load_page<HD>(ks + i * Cfg<HD>::PAGE_ELEMS, k_pages + src, tid);
      load_page<HD>(vs + i * Cfg<HD>::PAGE_ELEMS, v_pages + src, tid);
    }
    cp_async_commit();
  }
  const int r_lo = lane >> 2, r_hi = r_lo + 8;                        // rows = heads of the group
  const __nv_bfloat16* qtok = q + (size_t)b * q_stride + (size_t)g * n_rep * HD;
  uint32_t qf[HD / 16][4];
  load_q<HD>(qf, r_lo < n_rep ? qtok + r_lo * HD : nullptr, r_hi < n_rep ? qtok + r_hi * HD : nullptr, lane);
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[d][i] = 0.f;
  for (int blk = blk0; blk < blk1; ++blk) {
    const int buf = (blk - blk0) % DECODE_STAGES;
    if (blk + DECODE_STAGES - 1 < blk1) {
      const int nbuf = (buf + DECODE_STAGES - 1) % DECODE_STAGES;
      const size_t src = (size_t)max(page_of(blk + DECODE_STAGES - 1), 0) * page_elems + (size_t)g * PAGE * HD;
      load_page<HD>(ks + nbuf * Cfg<HD>::PAGE_ELEMS, k_pages + src, tid);
      load_page<HD>(vs + nbuf * Cfg<HD>::PAGE_ELEMS, v_pages + src, tid);
    }
    cp_async_commit();
    cp_async_wait<DECODE_STAGES - 1>();
    __syncthreads();
    const int key0 = warp * 16;                                       // this warp's quarter of the page
    const int abs0 = blk * PAGE + key0;
    if (abs0 <= pos && abs0 + 15 >= lo) {
      float s[2][4];
      scores<HD, 2>(qf, ks + buf * Cfg<HD>::PAGE_ELEMS, key0, s, lane);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int kabs = abs0 + nt * 8 + (lane & 3) * 2 + (i & 1);
          s[nt][i] = (kabs >= lo && kabs <= pos) ? s[nt][i] * scale_log2 : -INFINITY;
        }
      softmax_step<HD, 2>(s, m, l, o);
      uint32_t pf[1][4];
      to_fragments<2>(s, pf);
      weighted_values<HD, 2>(pf, vs + buf * Cfg<HD>::PAGE_ELEMS, key0, o, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the four warps (each saw a quarter of every page) through shared memory ----
  float* so = (float*)smem_raw;                         // [4][16][HD]
  float* sm = so + 4 * 16 * HD;                         // [4][16]
  float* sl = sm + 4 * 16;                              // [4][16]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) {
    const int c = d * 8 + (lane & 3) * 2;
    *(float2*)(so + (warp * 16 + r_lo) * HD + c) = make_float2(o[d][0], o[d][1]);
    *(float2*)(so + (warp * 16 + r_hi) * HD + c) = make_float2(o[d][2], o[d][3]);
  }
  if ((lane & 3) == 0) {
    sm[warp * 16 + r_lo] = m[0];
    sm[warp * 16 + r_hi] = m[1];
    sl[warp * 16 + r_lo] = l[0];
    sl[warp * 16 + r_hi] = l[1];
  }
  __syncthreads();
  // ---- this rank's partial result goes to the ranks that own its elements, 16 bytes a store ----
  // (every store into a peer's shared memory is a packet between two SMs; the shares are
  // multiples of four elements so that no store straddles two owners)
  const int n_out = n_rep * HD, share = ((n_out + C - 1) / C + 3) & ~3;
  const uint32_t recv_o = smem_u32(s_recv_o), recv_ml = smem_u32(s_recv_ml);
  for (int e = tid * 4; e < n_out; e += THREADS * 4) {
    const int row = e / HD, d = e - row * HD;                  // four elements of one row: HD is a multiple of 16
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm[w * 16 + row]);
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, Lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sm[w * 16 + row];
      const float f = (mw == -INFINITY) ? 0.f : ex2_fast(mw - M);
      const float4 ow = *(const float4*)(so + (w * 16 + row) * HD + d);
      acc[0] += f * ow.x; acc[1] += f * ow.y; acc[2] += f * ow.z; acc[3] += f * ow.w;
      Lsum += f * sl[w * 16 + row];
    }
    const int owner = e / share, idx = e - owner * share;
    st_peer_f32x4(peer_smem(recv_o + (uint32_t)(rank * share + idx) * 4, (uint32_t)owner), acc[0], acc[1], acc[2], acc[3]);
    if (d == 0) {
      for (int c = 0; c < C; ++c) {
        st_peer_f32x2(peer_smem(recv_ml + (uint32_t)((rank * 16 + row) * 2) * 4, (uint32_t)c), M, Lsum);
      }
    }
  }
  cluster_arrive();
  cluster_wait();                            // every rank's results for this rank's share have arrived
  float* const group_o = part_o + (size_t)(pair * G + grp) * n_out;
  float* const group_ml = part_ml + (size_t)(pair * G + grp) * 32;
  for (int t = tid; t < share; t += THREADS) {
    const int e = rank * share + t;
    if (e < n_out) {
      const int row = e / HD, d = e - row * HD;
      float M = -INFINITY;
      for (int c = 0; c < C; ++c) M = fmaxf(M, s_recv_ml[(c * 16 + row) * 2]);
      float num = 0.f, den = 0.f;
      for (int c = 0; c < C; ++c) {                        // in rank order
        const float mc = s_recv_ml[(c * 16 + row) * 2];
        const float f = (mc == -INFINITY) ? 0.f : ex2_fast(mc - M);
        num += f * s_recv_o[c * share + t];
        den += f * s_recv_ml[(c * 16 + row) * 2 + 1];
      }
      if (G == 1) {
        out[(size_t)b * out_stride + (size_t)(g * n_rep + row) * HD + d] = __float2bfloat16_rn(den > 0.f ? __fdividef(num, den) : 0.f);
      } else {
        group_o[e] = num;
        if (d == 0) *(float2*)(group_ml + row * 2) = make_float2(M, den);
      }
    }
  }
  if (G == 1) return;
  // ---- several groups to the pair: the cluster that finishes last adds the groups' parts ----
  // Every thread fences its part; after a cluster barrier rank 0 takes the pair's ticket and
  // tells every rank whether this cluster is the last; if so each rank adds, for its share of
  // the elements, the G parts in group order (all loads of a thread in flight at once).
  __threadfence();
  cluster_arrive();
  cluster_wait();
  if (rank == 0 && tid == 0) {
    __threadfence();
    const int ticket = atomicAdd(counters + pair, 1);
    const int last = ticket == G - 1;
    if (last) counters[pair] = 0;            // zero again for the next launch
    __threadfence();
    const uint32_t flag = smem_u32(&s_last);
    for (int c = 0; c < C; ++c) st_peer_b32(peer_smem(flag, (uint32_t)c), (uint32_t)last);
  }
  cluster_arrive();
  cluster_wait();
  if (!s_last) return;
  const float* const pair_o = part_o + (size_t)pair * G * n_out;
  const float* const pair_ml = part_ml + (size_t)pair * G * 32;
  for (int t = tid; t < share; t += THREADS) {
    const int e = rank * share + t;
    if (e < n_out) {
      const int row = e / HD, d = e - row * HD;
      float2 ml[CLUSTER_DECODE_MAX_GROUPS];
      float po[CLUSTER_DECODE_MAX_GROUPS];
#pragma unroll
      for (int c = 0; c < CLUSTER_DECODE_MAX_GROUPS; ++c)
        if (c < G) {
          ml[c] = __ldcg((const float2*)(pair_ml + c * 32 + row * 2));
          po[c] = __ldcg(pair_o + (size_t)c * n_out + e);
        }
      float M = -INFINITY;
#pragma unroll
      for (int c = 0; c < CLUSTER_DECODE_MAX_GROUPS; ++c)
        if (c < G) M = fmaxf(M, ml[c].x);
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int c = 0; c < CLUSTER_DECODE_MAX_GROUPS; ++c)             // in group order
        if (c < G) {
          const float f = (ml[c].x == -INFINITY) ? 0.f : ex2_fast(ml[c].x - M);
          num += f * po[c];
          den += f * ml[c].y;
        }
      out[(size_t)b * out_stride + (size_t)(g * n_rep + row) * HD + d] = __float2bfloat16_rn(den > 0.f ? __fdividef(num, den) : 0.f);
    }
  }
}

// ---- prefill ------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(THREADS)
prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out, int out_stride,
               const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
               const int* __restrict__ page_table, int table_width, const int* __restrict__ cu_seqlens,
               const int* __restrict__ ctx_lens, int nh, int nkv, float scale_log2, int window) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* ks = (__nv_bfloat16*)smem_raw;
  __nv_bfloat16* vs = ks + 2 * Cfg<HD>::PAGE_ELEMS;
  // the last tiles of a sequence see the most keys: they start first
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rep = nh / nkv;
  const int tok0 = cu_seqlens[b];
  const int n_new = cu_seqlens[b + 1] - tok0;
  const int n_rows = n_new * n_rep;
  const int row0 = tile * 64;
  if (row0 >= n_rows) return;                         // whole CTA: no barrier has been used yet
  const int L = ctx_lens[b];
  const int start = L - n_new;                        // position of the sequence's first new token
  const int* table = page_table + (size_t)b * table_width;
  const size_t page_elems = (size_t)nkv * PAGE * HD;

  // rows of this thread: (token, head in group)
  const int r_lo = row0 + warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const bool v_lo = r_lo < n_rows, v_hi = r_hi < n_rows;
  const int t_lo = v_lo ? r_lo / n_rep : 0, t_hi = v_hi ? r_hi / n_rep : 0;
  const int h_lo = g * n_rep + (v_lo ? r_lo % n_rep : 0), h_hi = g * n_rep + (v_hi ? r_hi % n_rep : 0);
  const int p_lo = start + t_lo, p_hi = start + t_hi;                // positions of the two rows
  uint32_t qf[HD / 16][4];
  load_q<HD>(qf, v_lo ? q + (size_t)(tok0 + t_lo) * q_stride + (size_t)h_lo * HD : nullptr,
             v_hi ? q + (size_t)(tok0 + t_hi) * q_stride + (size_t)h_hi * HD : nullptr, lane);

  // key range of the tile: from the first key its first row sees to the position of its last row
  const int last_row = min(row0 + 63, n_rows - 1);
  const int tile_pos_hi = start + last_row / n_rep;
  const int tile_pos_lo = start + row0 / n_rep;
  const int tile_lo = (window > 0 && tile_pos_lo - window + 1 > 0) ? tile_pos_lo - window + 1 : 0;
  const int blk0 = tile_lo / PAGE, blk1 = tile_pos_hi / PAGE + 1;
  const int lo_lo = (window > 0 && p_lo - window + 1 > 0) ? p_lo - window + 1 : 0;
  const int lo_hi = (window > 0 && p_hi - window + 1 > 0) ? p_hi - window + 1 : 0;
  // this warp's rows see keys in [warp_lo, warp_hi]
  const int wr0 = min(row0 + warp * 16, n_rows - 1), wr1 = min(row0 + warp * 16 + 15, n_rows - 1);
  const int warp_hi = start + wr1 / n_rep;
  const int warp_pos0 = start + wr0 / n_rep;
  const int warp_lo = (window > 0 && warp_pos0 - window + 1 > 0) ? warp_pos0 - window + 1 : 0;
  const bool warp_active = row0 + warp * 16 < n_rows;
  const bool warp_full = row0 + warp * 16 + 15 < n_rows;            // all 16 rows exist
  const int warp_lo_last = (window > 0 && warp_hi - window + 1 > 0) ? warp_hi - window + 1 : 0;

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[d][i] = 0.f;

  {
    const size_t src0 = (size_t)max(table[blk0], 0) * page_elems + (size_t)g * PAGE * HD;
    load_page<HD>(ks, k_pages + src0, tid);
    load_page<HD>(vs, v_pages + src0, tid);
  }
  cp_async_commit();
  for (int blk = blk0; blk < blk1; ++blk) {
    const int buf = (blk - blk0) & 1;
    if (blk + 1 < blk1) {
      const size_t src = (size_t)max(table[blk + 1], 0) * page_elems + (size_t)g * PAGE * HD;
      load_page<HD>(ks + (buf ^ 1) * Cfg<HD>::PAGE_ELEMS, k_pages + src, tid);
      load_page<HD>(vs + (buf ^ 1) * Cfg<HD>::PAGE_ELEMS, v_pages + src, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int abs0 = blk * PAGE;
    if (warp_active && abs0 <= warp_hi && abs0 + PAGE - 1 >= warp_lo) {
      float s[8][4];
      scores<HD, 8>(qf, ks + buf * Cfg<HD>::PAGE_ELEMS, 0, s, lane);
      // a page that every row of the warp sees whole needs no mask
      if (warp_full && abs0 + PAGE - 1 <= warp_pos0 && abs0 >= warp_lo_last) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) s[nt][i] *= scale_log2;
      } else {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int kabs = abs0 + nt * 8 + (lane & 3) * 2 + (i & 1);
            const bool vis = (i < 2) ? (v_lo && kabs >= lo_lo && kabs <= p_lo) : (v_hi && kabs >= lo_hi && kabs <= p_hi);
            s[nt][i] = vis ? s[nt][i] * scale_log2 : -INFINITY;
          }
      }
      softmax_step<HD, 8>(s, m, l, o);
      uint32_t pf[4][4];
      to_fragments<8>(s, pf);
      weighted_values<HD, 8>(pf, vs + buf * Cfg<HD>::PAGE_ELEMS, 0, o, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  const float inv_lo = l[0] > 0.f ? 1.f / l[0] : 0.f, inv_hi = l[1] > 0.f ? 1.f / l[1] : 0.f;
  __nv_bfloat16* o_lo = out + (size_t)(tok0 + t_lo) * out_stride + (size_t)h_lo * HD;
  __nv_bfloat16* o_hi = out + (size_t)(tok0 + t_hi) * out_stride + (size_t)h_hi * HD;
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) {
    const int c = d * 8 + (lane & 3) * 2;
    if (v_lo) *(uint32_t*)(o_lo + c) = pack_bf16(o[d][0] * inv_lo, o[d][1] * inv_lo);
    if (v_hi) *(uint32_t*)(o_hi + c) = pack_bf16(o[d][2] * inv_hi, o[d][3] * inv_hi);
  }
}

template <int HD, int STAGES>
static int launch_decode_stages(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                const void* v_pages, const int* page_table, int table_width, const int* ctx_lens, int B,
                                int nh, int nkv, float scale, int window, int n_ctas, float* part_o, float* part_ml,
                                int* counters, cudaStream_t stream) {
  // shared memory: the page buffers, reused for the merge of the warps and for the combine
  const int merge_bytes = (4 * 16 * HD + 2 * 4 * 16) * (int)sizeof(float);
  const int combine_bytes = (2 * 16 * n_ctas + 16 + 16 * HD) * (int)sizeof(float);   // weights and room for one part
  int smem = STAGES * 2 * Cfg<HD>::PAGE_ELEMS * 2;
  if (merge_bytes > smem) smem = merge_bytes;
  if (combine_bytes > smem) smem = combine_bytes;
  static int configured[MAX_DEVICES];
  if (int rc = allow_smem(decode_kernel<HD, STAGES>, smem, configured)) return rc;
  wpc::launch(decode_kernel<HD, STAGES>, dim3(n_ctas), THREADS, smem, stream, 
      (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages,
      (const __nv_bfloat16*)v_pages, page_table, table_width, ctx_lens, B, nh, nkv, scale * LOG2E, window,
      part_o, part_ml, counters, smem, early_pages());
  return launch_status();
}

template <int HD>
static int launch_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                         const void* v_pages, const int* page_table, int table_width, const int* ctx_lens, int B,
                         int nh, int nkv, float scale, int window, int n_ctas, float* part_o, float* part_ml,
                         int* counters, cudaStream_t stream) {
  // with at most a CTA to an SM the ring takes all the shared memory it can use
  if (n_ctas <= sm_count() && DECODE_STAGES_ALONE * 2 * Cfg<HD>::PAGE_ELEMS * 2 <= 220 * 1024)
    return launch_decode_stages<HD, DECODE_STAGES_ALONE>(q, q_stride, out, out_stride, k_pages, v_pages, page_table,
                                                         table_width, ctx_lens, B, nh, nkv, scale, window, n_ctas,
                                                         part_o, part_ml, counters, stream);
  return launch_decode_stages<HD, DECODE_STAGES_SHARED>(q, q_stride, out, out_stride, k_pages, v_pages, page_table,
                                                        table_width, ctx_lens, B, nh, nkv, scale, window, n_ctas,
                                                        part_o, part_ml, counters, stream);
}

template <int HD, int STAGES, bool GROUPED>
static int launch_decode_cluster_stages(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                        const void* v_pages, const int* page_table, int table_width,
                                        const int* ctx_lens, int B, int nh, int nkv, float scale, int window,
                                        int cluster, int groups, float* part_o, float* part_ml, int* counters,
                                        cudaStream_t stream) {
  const int merge_bytes = (4 * 16 * HD + 2 * 4 * 16) * (int)sizeof(float);
  int smem = STAGES * 2 * Cfg<HD>::PAGE_ELEMS * 2;
  if (merge_bytes > smem) smem = merge_bytes;
  static int configured[MAX_DEVICES];
  if (configured[current_device()] < smem) {
    // clusters of more than 8 CTAs need the kernel's consent
    cudaError_t e = cudaFuncSetAttribute(decode_cluster_kernel<HD, STAGES, GROUPED>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
    if (int rc = allow_smem(decode_cluster_kernel<HD, STAGES, GROUPED>, smem, configured)) return rc;
  }
  wpc::launch_clusters(decode_cluster_kernel<HD, STAGES, GROUPED>, dim3((unsigned)(B * nkv * groups * cluster)), THREADS, smem,
                       stream, (unsigned)cluster, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
                       (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, page_table, table_width, ctx_lens,
                       B, nh, nkv, scale * LOG2E, window, cluster, early_pages(), groups, part_o, part_ml, counters);
  return launch_status();
}

template <int HD, bool GROUPED>
static int launch_decode_cluster_grouped(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                         const void* v_pages, const int* page_table, int table_width,
                                         const int* ctx_lens, int B, int nh, int nkv, float scale, int window,
                                         int cluster, int groups, float* part_o, float* part_ml, int* counters,
                                         cudaStream_t stream) {
  if (B * nkv * groups * cluster <= sm_count() && DECODE_STAGES_ALONE * 2 * Cfg<HD>::PAGE_ELEMS * 2 <= 215 * 1024)
    return launch_decode_cluster_stages<HD, DECODE_STAGES_ALONE, GROUPED>(
        q, q_stride, out, out_stride, k_pages, v_pages, page_table, table_width, ctx_lens, B, nh, nkv, scale, window,
        cluster, groups, part_o, part_ml, counters, stream);
  return launch_decode_cluster_stages<HD, DECODE_STAGES_SHARED, GROUPED>(
      q, q_stride, out, out_stride, k_pages, v_pages, page_table, table_width, ctx_lens, B, nh, nkv, scale, window,
      cluster, groups, part_o, part_ml, counters, stream);
}

template <int HD>
static int launch_decode_cluster(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                 const void* v_pages, const int* page_table, int table_width, const int* ctx_lens,
                                 int B, int nh, int nkv, float scale, int window, int cluster, int groups,
                                 float* part_o, float* part_ml, int* counters, cudaStream_t stream) {
  if (groups > 1)
    return launch_decode_cluster_grouped<HD, true>(q, q_stride, out, out_stride, k_pages, v_pages, page_table,
                                                   table_width, ctx_lens, B, nh, nkv, scale, window, cluster, groups,
                                                   part_o, part_ml, counters, stream);
  return launch_decode_cluster_grouped<HD, false>(q, q_stride, out, out_stride, k_pages, v_pages, page_table,
                                                  table_width, ctx_lens, B, nh, nkv, scale, window, cluster, 1,
                                                  part_o, part_ml, counters, stream);
}

// How many clusters of `cluster` CTAs of the cluster decode kernel the device holds at once, by
// the runtime's count for this device's GPCs (a cluster lives inside one GPC, and the number
// of SMs that a GPC has differs from chip to chip); -1 on a CUDA error.
template <int HD, int STAGES>
static int decode_cluster_capacity(int cluster) {
  const int smem = STAGES * 2 * Cfg<HD>::PAGE_ELEMS * 2;
  cudaError_t e = cudaFuncSetAttribute(decode_cluster_kernel<HD, STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(decode_cluster_kernel<HD, STAGES, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e != cudaSuccess) { cudaGetLastError(); return -1; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(cluster * sm_count()));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  e = cudaOccupancyMaxActiveClusters(&n, decode_cluster_kernel<HD, STAGES, false>, &cfg);
  if (e != cudaSuccess) { cudaGetLastError(); return -1; }
  return n;
}

template <int HD>
static int launch_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                          const void* v_pages, const int* page_table, int table_width, const int* cu_seqlens,
                          const int* ctx_lens, int B, int max_new, int nh, int nkv, float scale, int window,
                          cudaStream_t stream) {
  static int configured[MAX_DEVICES];
  if (int rc = allow_smem(prefill_kernel<HD>, Cfg<HD>::SMEM_BYTES, configured)) return rc;
  const int n_rep = nh / nkv;
  dim3 grid((max_new * n_rep + 63) / 64, nkv, B);
  wpc::launch(prefill_kernel<HD>, grid, THREADS, Cfg<HD>::SMEM_BYTES, stream, 
      (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages,
      (const __nv_bfloat16*)v_pages, page_table, table_width, cu_seqlens, ctx_lens, nh, nkv, scale * LOG2E, window);
  return launch_status();
}

}  // namespace fa
}  // namespace wpc

using namespace wpc;

#define WPC_DISPATCH_HD(hd, ...)                              \
  switch (hd) {                                               \
    case 16: { constexpr int HD = 16; return __VA_ARGS__; }   \
    case 32: { constexpr int HD = 32; return __VA_ARGS__; }   \
    case 48: { constexpr int HD = 48; return __VA_ARGS__; }   \
    case 64: { constexpr int HD = 64; return __VA_ARGS__; }   \
    case 80: { constexpr int HD = 80; return __VA_ARGS__; }   \
    case 96: { constexpr int HD = 96; return __VA_ARGS__; }   \
    case 112: { constexpr int HD = 112; return __VA_ARGS__; } \
    case 128: { constexpr int HD = 128; return __VA_ARGS__; } \
    default: return WPC_ERR_UNSUPPORTED;                      \
  }

extern "C" {

// Decode attention copies pages of earlier positions before the kernel ahead has finished
// (1, the default) or starts every copy after it (0); returns the old setting.
int wpc_attention_decode_early_pages(int on) {
  const int was = fa::early_pages();
  fa::early_pages() = on ? 1 : 0;
  return was;
}

// 1 if these sizes can take the tensor-core kernels, else 0 (the plain kernel takes them).
int wpc_attention_mma_supports(int nh, int nkv, int hd) {
  return hd >= 16 && hd <= 128 && hd % 16 == 0 && nkv >= 1 && nh % nkv == 0 && nh / nkv <= 16;
}

// One query token per sequence: q row b belongs to sequence b (at most 1024 sequences).
// n_ctas CTAs share the pages of all sequences evenly (1..1024).  part_o: float32
// [(n_ctas + B * nkv) * 16 * hd], part_ml: float32 [(n_ctas + B * nkv) * 16 * 2], counters:
// B * nkv tickets that are zero between launches.
int wpc_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                         const void* v_pages, const int* page_table, int table_width, const int* ctx_lens, int B,
                         int nh, int nkv, int hd, float scale, int window, int n_ctas, float* part_o,
                         float* part_ml, int* counters, int n_counters, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (!wpc_attention_mma_supports(nh, nkv, hd) || (q_stride % 2) || (out_stride % 2) || B > fa::MAX_DECODE_SEQS)
    return WPC_ERR_UNSUPPORTED;
  if (n_ctas < 1 || n_ctas > 1024 || !part_o || !part_ml || !counters || B * nkv > n_counters)
    return WPC_ERR_BAD_ARGUMENT;
  WPC_DISPATCH_HD(hd, fa::launch_decode<HD>(q, q_stride, out, out_stride, k_pages, v_pages, page_table, table_width,
                                           ctx_lens, B, nh, nkv, scale, window, n_ctas, part_o, part_ml, counters,
                                           stream));
}

// The same with a thread-block cluster of `cluster` CTAs (2..16) to each (sequence, kv head) pair,
// which share the pair's pages and add up through one another's shared memory; for few pairs
// of about equal lengths.  Needs (nh / nkv) * hd <= 1024 and at most 1024 CTAs.  With groups > 1
// that many clusters share a pair's pages through part_o (float32 [B * nkv * groups * (nh / nkv)
// * hd]), part_ml (float32 [B * nkv * groups * 32]) and B * nkv tickets that are zero between
// launches.
int wpc_attention_decode_cluster(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                 const void* v_pages, const int* page_table, int table_width, const int* ctx_lens,
                                 int B, int nh, int nkv, int hd, float scale, int window, int cluster, int groups,
                                 float* part_o, float* part_ml, int* counters, int n_counters,
                                 cudaStream_t stream) {
  if (B <= 0) return 0;
  if (!wpc_attention_mma_supports(nh, nkv, hd) || (q_stride % 2) || (out_stride % 2) ||
      (nh / nkv) * hd > fa::CLUSTER_DECODE_MAX_OUT)
    return WPC_ERR_UNSUPPORTED;
  if (cluster < 2 || cluster > fa::CLUSTER_DECODE_MAX_RANKS || groups < 1 ||
      groups > fa::CLUSTER_DECODE_MAX_GROUPS || (long)B * nkv * cluster * groups > 1024)
    return WPC_ERR_BAD_ARGUMENT;
  if (groups > 1 && (!part_o || !part_ml || !counters || B * nkv > n_counters)) return WPC_ERR_BAD_ARGUMENT;
  WPC_DISPATCH_HD(hd, fa::launch_decode_cluster<HD>(q, q_stride, out, out_stride, k_pages, v_pages, page_table,
                                                   table_width, ctx_lens, B, nh, nkv, scale, window, cluster, groups,
                                                   part_o, part_ml, counters, stream));
}

// Clusters of `cluster` CTAs of the cluster decode kernel that run at once: with the short ring
// (two CTAs to an SM) or, `alone`, with the long one.
int wpc_attention_decode_cluster_capacity(int hd, int cluster, int alone) {
  if (cluster < 2 || cluster > fa::CLUSTER_DECODE_MAX_RANKS) return 0;
  if (alone) { WPC_DISPATCH_HD(hd, fa::decode_cluster_capacity<HD, fa::DECODE_STAGES_ALONE>(cluster)); }
  WPC_DISPATCH_HD(hd, fa::decode_cluster_capacity<HD, fa::DECODE_STAGES_SHARED>(cluster));
}

int wpc_attention_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                          const void* v_pages, const int* page_table, int table_width, const int* cu_seqlens,
                          const int* ctx_lens, int B, int max_new, int nh, int nkv, int hd, float scale, int window,
                          cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (!wpc_attention_mma_supports(nh, nkv, hd) || (q_stride % 2) || (out_stride % 2)) return WPC_ERR_UNSUPPORTED;
  WPC_DISPATCH_HD(hd, fa::launch_prefill<HD>(q, q_stride, out, out_stride, k_pages, v_pages, page_table, table_width,
                                            cu_seqlens, ctx_lens, B, max_new, nh, nkv, scale, window, stream));
}

}  // extern "C"
