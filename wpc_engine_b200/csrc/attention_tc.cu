// Causal grouped-query attention of a prompt over the paged cache on the 5th-generation tensor
// cores (wpc-runtime/src/model.rs:476-510 is the arithmetic).
//
// A CTA takes 128 rows of (token, head-in-group) of one sequence and one KV head and walks the
// pages (64 keys) that its rows see.  Per page:
//
//   S = Q K^T      tcgen05.mma, Q [128, hd] and the K page [64, hd] in shared memory (K-major,
//                  128-byte swizzle), S [128, 64] float32 in tensor memory
//   softmax        thread r owns row r: tcgen05.ld of its 64 scores, scale, mask, running
//                  maximum and sum in float32, P = exp2(S - m) as bfloat16 into shared memory
//   O += P V       tcgen05.mma, P [128, 64] K-major, the V page [64, hd] as it lies in the
//                  cache (hd contiguous: an MN-major B operand), O [128, hd] float32 in tensor
//                  memory
//
// The running maximum that the exponentials use is only raised when the true maximum has
// grown by more than 8 (a factor 256, harmless in float32); then the thread rescales its row
// of O in tensor memory.  There are two score buffers: while the threads do the softmax of
// page j, the tensor pipe computes the scores of page j + 1 and the weighted values of page
// j - 1; two CTAs share an SM on top of that.  Pages are copied with cp.async into swizzled
// shared memory a whole page ahead.  Every wait on an MMA barrier is bounded.  head_dim 64
// or 128; other sizes take the mma.sync kernel.
#include "api.h"
#include "common.cuh"

namespace wpc {
namespace fatc {

constexpr int PAGE = WPC_PAGE;
constexpr int THREADS = 128;
constexpr int ROWS = 128;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}
__device__ __forceinline__ void tmem_alloc(uint32_t* holder, int cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, int cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Descriptor of a swizzled (128-byte rows, 1024-byte groups of 8 rows) operand in shared memory.
// K-major: rows are M or N, the 128 bytes of a row run along K; lbo unused.
// MN-major: rows are K, the 128 bytes of a row run along M or N; lbo = bytes to the next 64
// elements along M or N.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// float32 accumulator, bfloat16 operands, A K-major, M = 128, N = n; B K-major or MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}
// Byte offset of 16-byte chunk c (0..7) of row `row` inside a swizzled [rows, 64] bfloat16 block.
__device__ __forceinline__ uint32_t swz(int row, int c) { return (uint32_t)(row * 128 + ((c ^ (row & 7)) << 4)); }

// 2^x in one instruction (relative error 2^-22, results below the normal range are zero): the
// weights are rounded to bfloat16 right after, and exp2f's handling of subnormal results costs
// three more instructions for each of the 64 scores of a row and page.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD>
struct Cfg {
  static constexpr int NB = HD / 64;                      // 64-wide blocks along head_dim
  static constexpr int Q_BYTES = NB * ROWS * 128;
  static constexpr int PAGE_BYTES = NB * PAGE * 128;      // one K or V page
  static constexpr int P_BYTES = ROWS * 128;
  // 896 bytes of slack bring the 128-byte aligned start to a 1024-byte boundary; two CTAs fit an SM
  static constexpr int SMEM = 896 + Q_BYTES + 4 * PAGE_BYTES + P_BYTES + 64;
  static constexpr int TMEM_COLS = 256;                   // two S buffers of 64, HD for O; a power of two
};

// Copies one page ([64, HD] contiguous) into NB swizzled [64, 64] blocks.
template <int HD>
__device__ __forceinline__ void load_page(uint32_t dst, const __nv_bfloat16* src, int tid) {
  constexpr int CPR = HD / 8;
  for (int c = tid; c < PAGE * CPR; c += THREADS) {
    const int row = c / CPR, col = c - row * CPR;
    cp_async16(dst + (col >> 3) * (PAGE * 128) + swz(row, col & 7), src + row * HD + col * 8);
  }
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
prefill_tc_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out, int out_stride,
                  const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                  const int* __restrict__ page_table, int table_width, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ ctx_lens, int nh, int nkv, float scale_log2, int window,
                  int* __restrict__ status) {
  using C = Cfg<HD>;
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // the last tiles of a sequence see the most keys: they start first
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_rep = nh / nkv;
  const int tok0 = cu_seqlens[b];
  const int n_new = cu_seqlens[b + 1] - tok0;
  const int n_rows = n_new * n_rep;
  const int row0 = tile * ROWS;
  if (row0 >= n_rows) return;                         // whole CTA, before anything is allocated

  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t q_s = smem_u32(base);
  const uint32_t k_s = q_s + C::Q_BYTES;              // two stages
  const uint32_t v_s = k_s + 2 * C::PAGE_BYTES;       // two stages
  uint8_t* p_ptr = base + C::Q_BYTES + 4 * C::PAGE_BYTES;
  const uint32_t p_s = smem_u32(p_ptr);
  uint64_t* bar_s = (uint64_t*)(p_ptr + C::P_BYTES);      // [2]: the scores in buffer b are ready
  uint64_t* bar_o = bar_s + 2;                             // the weighted values of a page are added
  uint32_t* tmem_holder = (uint32_t*)(bar_o + 1);
  int* failed = (int*)(tmem_holder + 1);

  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 1, 1);
    mbar_init(bar_o, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(tmem_holder, C::TMEM_COLS);

  const int L = ctx_lens[b];
  const int start = L - n_new;
  const int* table = page_table + (size_t)b * table_width;
  const size_t page_elems = (size_t)nkv * PAGE * HD;

  // this thread's row
  const int r = row0 + tid;
  const bool valid = r < n_rows;
  const int t_row = valid ? r / n_rep : 0;
  const int h_row = g * n_rep + (valid ? r % n_rep : 0);
  const int p_row = start + t_row;
  const int lo_row = (window > 0 && p_row - window + 1 > 0) ? p_row - window + 1 : 0;

  // Q rows into swizzled shared memory (rows past the end are zero)
  {
    const __nv_bfloat16* src = q + (size_t)(tok0 + t_row) * q_stride + (size_t)h_row * HD;
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) {
      uint4 v = valid ? *(const uint4*)(src + c * 8) : make_uint4(0, 0, 0, 0);
      *(uint4*)(base + (c >> 3) * (ROWS * 128) + swz(tid, c & 7)) = v;
    }
  }

  const int last_row = min(row0 + ROWS - 1, n_rows - 1);
  const int tile_pos_hi = start + last_row / n_rep;
  const int tile_pos_lo = start + row0 / n_rep;
  const int tile_lo = (window > 0 && tile_pos_lo - window + 1 > 0) ? tile_pos_lo - window + 1 : 0;
  const int blk0 = tile_lo / PAGE, blk1 = tile_pos_hi / PAGE + 1;

  // ---- copies ahead: K of pages 0 and 1, V of page 0 (one cp.async group each) ----
  const int n_pg = blk1 - blk0;
  auto page_src = [&](int j) { return (size_t)max(table[blk0 + j], 0) * page_elems + (size_t)g * PAGE * HD; };
  load_page<HD>(k_s, k_pages + page_src(0), tid);
  cp_async_commit();
  load_page<HD>(v_s, v_pages + page_src(0), tid);
  cp_async_commit();
  if (n_pg > 1) load_page<HD>(k_s + C::PAGE_BYTES, k_pages + page_src(1), tid);
  cp_async_commit();

  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base;                 // two score buffers: columns 0..63 and 64..127
  const uint32_t tmem_O = tmem_base + 128;           // columns 128..128+HD-1
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

  constexpr uint32_t idesc_qk = instr_desc(64, false);
  constexpr uint32_t idesc_pv = instr_desc(HD, true);
  float m_used = -INFINITY, l_sum = 0.f;
  bool ok = true;

  // S_j = Q K_j^T into score buffer j & 1 (issued by one thread)
  auto issue_qk = [&](int j) {
    fence_after_sync();
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
      const uint32_t qa = q_s + (kk >> 2) * (ROWS * 128) + (kk & 3) * 32;
      const uint32_t ka = k_s + (j & 1) * C::PAGE_BYTES + (kk >> 2) * (PAGE * 128) + (kk & 3) * 32;
      umma_bf16(tmem_S + (j & 1) * 64, smem_desc(qa, 16), smem_desc(ka, 16), idesc_qk, kk > 0 ? 1u : 0u);
    }
    umma_commit(bar_s + (j & 1));
  };

  // The products of page j + 1 (scores) and of page j - 1 (weighted values) run on the tensor
  // pipe while the threads do the softmax of page j; copies are issued a whole page ahead.
  for (int j = 0; j < n_pg; ++j) {
    // (A) the keys of the next page are in shared memory (only the newest group of copies, the
    // values of this page, may still be on its way); start the scores of the next page
    if (j == 0) cp_async_wait<0>(); else cp_async_wait<1>();
    fence_async_smem();
    fence_before_sync();
    __syncthreads();
    if (tid == 0 && j == 0) issue_qk(0);
    if (tid == 0 && j + 1 < n_pg) issue_qk(j + 1);

    // (B) the scores of this page
    ok = mbar_wait(bar_s + (j & 1), (j >> 1) & 1);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) { atomicExch(failed, 1); break; }
    fence_after_sync();
    if (j + 2 < n_pg) load_page<HD>(k_s + (j & 1) * C::PAGE_BYTES, k_pages + page_src(j + 2), tid);   // K_j has been read
    cp_async_commit();

    // (C) softmax of this thread's row, in registers
    uint32_t su[64];
    tmem_ld32(tmem_S + (j & 1) * 64 + lane_off, su);
    tmem_ld32(tmem_S + (j & 1) * 64 + lane_off + 32, su + 32);
    tmem_ld_wait();
    const int abs0 = (blk0 + j) * PAGE;
    // raw scores; the scale (positive) goes into the exponent's multiply-add.  Only pages that
    // this row does not see whole are masked.
    // four partial maxima (and sums below): a single running value would be a chain of 64
    // dependent instructions
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    if (valid && abs0 + PAGE - 1 <= p_row && abs0 >= lo_row) {
#pragma unroll
      for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(su[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const int kabs = abs0 + i;
        const float sc = (valid && kabs >= lo_row && kabs <= p_row) ? __uint_as_float(su[i]) : -INFINITY;
        su[i] = __float_as_uint(sc);
        mx4[i & 3] = fmaxf(mx4[i & 3], sc);
      }
    }
    float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    mx *= scale_log2;
    // raise the maximum in use only when the true one has outgrown it
    float alpha = 1.f;
    bool rescale = false;
    if (mx > m_used + RESCALE_STEP || (m_used == -INFINITY && mx > -INFINITY)) {
      alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
      rescale = m_used != -INFINITY;
      m_used = mx;
    }
    l_sum *= alpha;
    const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;     // all scores are -inf then: p = 0
    float sum4[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t pw[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float p0 = ex2(fmaf(__uint_as_float(su[2 * i]), scale_log2, neg_m));
      const float p1 = ex2(fmaf(__uint_as_float(su[2 * i + 1]), scale_log2, neg_m));
      sum4[i & 3] += p0 + p1;
      const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
      pw[i] = *(const uint32_t*)&pb;
    }
    const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
    l_sum += sum;

    // (D) the weighted values of the page before must be done before O and P are touched
    if (j > 0) {
      ok = mbar_wait(bar_o, (j - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { atomicExch(failed, 1); break; }
      fence_after_sync();
    }
    if (j + 1 < n_pg) load_page<HD>(v_s + ((j + 1) & 1) * C::PAGE_BYTES, v_pages + page_src(j + 1), tid);   // V_{j-1} has been read
    cp_async_commit();
    if (__any_sync(0xffffffffu, rescale)) {
      // the whole warp takes part (tcgen05.ld/st are warp-wide); rows that keep their maximum use 1
      const float a = rescale ? alpha : 1.f;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t ou[32];
        tmem_ld32(tmem_O + lane_off + c, ou);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) ou[i] = __float_as_uint(__uint_as_float(ou[i]) * a);
        tmem_st32(tmem_O + lane_off + c, ou);
      }
      tmem_st_wait();
    }
#pragma unroll
    for (int c = 0; c < 8; ++c)
      *(uint4*)(p_ptr + swz(tid, c)) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
    cp_async_wait<2>();                 // the values of this page (two groups have been started since)
    fence_before_sync();
    fence_async_smem();
    __syncthreads();

    // (E) O += P V_j
    if (tid == 0) {
      fence_after_sync();
#pragma unroll
      for (int kc = 0; kc < PAGE / 16; ++kc) {
        const uint32_t pa = p_s + kc * 32;
        const uint32_t va = v_s + (j & 1) * C::PAGE_BYTES + kc * 2048;
        umma_bf16(tmem_O, smem_desc(pa, 16), smem_desc(va, PAGE * 128), idesc_pv, (j > 0 || kc > 0) ? 1u : 0u);
      }
      umma_commit(bar_o);
    }
  }
  cp_async_wait<0>();
  if (ok) {
    ok = mbar_wait(bar_o, (n_pg - 1) & 1);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) atomicExch(failed, 1);
    fence_after_sync();
  }

  if (ok) {
    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
    __nv_bfloat16* dst = out + (size_t)(tok0 + t_row) * out_stride + (size_t)h_row * HD;
#pragma unroll
    for (int c = 0; c < HD; c += 32) {
      uint32_t ou[32];
      tmem_ld32(tmem_O + lane_off + c, ou);
      tmem_ld_wait();
      if (valid) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 o;
          __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(ou[j]) * inv, __uint_as_float(ou[j + 1]) * inv);
          __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(ou[j + 2]) * inv, __uint_as_float(ou[j + 3]) * inv);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(ou[j + 4]) * inv, __uint_as_float(ou[j + 5]) * inv);
          __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(ou[j + 6]) * inv, __uint_as_float(ou[j + 7]) * inv);
          o.x = *(uint32_t*)&a0; o.y = *(uint32_t*)&a1; o.z = *(uint32_t*)&a2; o.w = *(uint32_t*)&a3;
          *(uint4*)(dst + c + j) = o;
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (*failed && tid == 0 && status) atomicExch(status, WPC_ERR_DEVICE_WAIT);
  if (warp == 0) {
    fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int HD>
static int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pages, const void* v_pages,
                  const int* page_table, int table_width, const int* cu_seqlens, const int* ctx_lens, int B,
                  int max_new, int nh, int nkv, float scale, int window, int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<HD>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int n_rep = nh / nkv;
  dim3 grid((max_new * n_rep + ROWS - 1) / ROWS, nkv, B);
  wpc::launch(prefill_tc_kernel<HD>, grid, THREADS, Cfg<HD>::SMEM, stream, (const __nv_bfloat16*)q, q_stride,
              (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
              page_table, table_width, cu_seqlens, ctx_lens, nh, nkv, scale * LOG2E, window, status);
  return launch_status();
}

}  // namespace fatc
}  // namespace wpc

extern "C" {

int wpc_attention_prefill_tc_supports(int nh, int nkv, int hd) {
  return (hd == 64 || hd == 128) && nkv >= 1 && nh % nkv == 0 && nh / nkv <= 128;
}

// q rows and out rows must be 16-byte aligned (strides multiples of 8 elements).
int wpc_attention_prefill_tc(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                             const void* v_pages, const int* page_table, int table_width, const int* cu_seqlens,
                             const int* ctx_lens, int B, int max_new, int nh, int nkv, int hd, float scale,
                             int window, int* status, cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (!wpc_attention_prefill_tc_supports(nh, nkv, hd) || (q_stride % 8) || (out_stride % 8) ||
      (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15))
    return WPC_ERR_UNSUPPORTED;
  if (hd == 128)
    return wpc::fatc::launch<128>(q, q_stride, out, out_stride, k_pages, v_pages, page_table, table_width,
                                  cu_seqlens, ctx_lens, B, max_new, nh, nkv, scale, window, status, stream);
  return wpc::fatc::launch<64>(q, q_stride, out, out_stride, k_pages, v_pages, page_table, table_width, cu_seqlens,
                               ctx_lens, B, max_new, nh, nkv, scale, window, status, stream);
}

}  // extern "C"
