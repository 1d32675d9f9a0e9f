// Causal grouped-query attention of a prompt over the paged cache on the 5th-generation tensor
// cores (wpc-runtime/src/model.rs:476-510 is the arithmetic).
//
// A CTA takes 128 rows of (token, head-in-group) of one sequence and one KV head (or two such
// tiles) and walks the pages (64 keys) that its rows see.  Per page:
//
//   S = Q K^T      tcgen05.mma, Q [128, hd] and the K page [64, hd] in shared memory (K-major,
//                  128-byte swizzle), S [128, 64] float32 in tensor memory
//   softmax        thread r owns row r: tcgen05.ld of its 64 scores, scale, mask, running
//                  maximum and sum in float32, P = exp2(S - m) as bfloat16 back into tensor
//                  memory, over the first 32 columns of the scores that it came from
//   O += P V       tcgen05.mma with the A operand P [128, 64] from tensor memory, the V page
//                  [64, hd] as it lies in the cache (hd contiguous: an MN-major B operand),
//                  O [128, hd] float32 in tensor memory
//
// The running maximum that the exponentials use is only raised when the true maximum has
// grown by more than 8 (a factor 256, harmless in float32); then the thread rescales its row
// of O in tensor memory.  Separate warps copy the pages (TMA), issue the MMAs and do the
// softmax; they meet at mbarriers only (see the kernel).  Every wait is bounded.  head_dim 64
// or 128; other sizes take the mma.sync kernel.
#include <cuda.h>

#include "api.h"
#include "common.cuh"
#include "tensor_map.h"

namespace wpc {
namespace fatc {

constexpr int PAGE = WPC_PAGE;
constexpr int THREADS = 128;
constexpr int ROWS = 128;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > limit_ns) return false;
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
// D[tmem] (+)= A[tmem] * B[smem]: A is 128 rows (lanes) of packed bfloat16 pairs, 8 columns for K = 16
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
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
};

// ---- the kernel -------------------------------------------------------------------------------------
// A CTA takes NT row tiles of 128 rows (NT = 2: 256 rows, one CTA to an SM; NT = 1: two CTAs to
// an SM).  Warps 0 .. 4 NT - 1: one thread per row, softmax only.  The next warp (one thread)
// issues every tcgen05.mma, the last warp (one thread) copies the K and V pages with TMA.
// Nothing in the page loop stops the whole CTA: the roles meet at mbarriers only where data
// passes from one to the other.
//
//   q_full                  softmax threads -> MMA    the Q rows are in shared memory
//   k_full[NS], v_full[NS]  TMA -> MMA                a page has landed (transaction bytes)
//   k_empty[NS], v_empty[NS]  MMA (commit) -> TMA     the MMAs that read the page have finished
//   s_full[NT][2]           MMA (commit) -> softmax   a tile's scores of a page are in tensor memory
//   s_empty[NT][2]          softmax -> MMA            they have been read (128 arrivals)
//   p_full[NT]              softmax -> MMA            P is in tensor memory and O is rescaled (128)
//   p_empty[NT]             MMA (commit) -> softmax   P V of the page has finished: P may be
//                                                     overwritten and O touched
// While the threads do the softmax of page j the tensor pipe computes the scores of page j + 1
// (second score buffer) and the weighted values of page j - 1.  With two row tiles every page
// is copied once for 256 rows (the copies from L2 bound the one-tile kernel at long prompts:
// 32 KiB for 4.2 MFLOP), and the MMAs of the two tiles, which do not depend on one another,
// take turns, so that one tile's chain of accumulations does not leave the pipe idle.  Both
// tiles walk the same pages; a page that one of them does not see is masked for it.
template <int HD, int NT>
struct WsCfg {
  using C = Cfg<HD>;
  static constexpr int NS = NT == 2 ? 4 : 2;              // stages of K and of V
  static constexpr int THREADS = 128 * NT + 64;
  static constexpr int TMEM_COLS = NT == 2 ? 512 : 256;   // per tile: two score buffers of 64 and HD for O
  static constexpr int N_BARS = 1 + 4 * NS + 6 * NT;
  // 896 bytes of slack bring the 128-byte aligned start to a 1024-byte boundary; with one tile
  // two CTAs fit an SM (tensor memory allows no third: 2 x 256 columns)
  static constexpr int SMEM = 896 + NT * C::Q_BYTES + 2 * NS * C::PAGE_BYTES + N_BARS * 8 + 8;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

template <int HD, int NT>
__global__ void __launch_bounds__(WsCfg<HD, NT>::THREADS, NT == 2 ? 1 : 2)
prefill_ws_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                  const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out, int out_stride,
                  const int* __restrict__ page_table, int table_width, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ ctx_lens, int nh, int nkv, float scale_log2, int window,
                  int* __restrict__ status, unsigned long long wait_ns, int starve, int n_sm, int late_trigger) {
  using C = Cfg<HD>;
  using W = WsCfg<HD, NT>;
  constexpr int NS = W::NS;
  constexpr int TROWS = NT * ROWS;
  if (!late_trigger) pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // The last tiles of a sequence see the most keys: they start first, and for all KV heads
  // before any lighter tile (the KV head is the fastest grid index), so that no heavy tile is
  // left for the end.  An SM takes new CTAs of this kernel in turn: while the older of its two
  // CTAs runs, the place of the younger one, once it has ended, stays empty (seen in a trace of
  // start and end times; without tcgen05.relinquish_alloc_permit an SM even runs one CTA at a
  // time).  So the two CTAs that an SM gets at the start should be equally heavy: the device
  // hands the first n_sm CTAs of a grid to one SM each and the next n_sm to the same SMs in
  // the same order, and position p of the grid takes rank 2 p, or 2 (p - n_sm) + 1, of the
  // pieces in descending order (one sequence only; 53.7 -> 47.3 us at 2,048 tokens of the 7B shape).
  int rank = (int)(blockIdx.y * gridDim.x + blockIdx.x);
  if (gridDim.z == 1) {
    const int n = (int)(gridDim.x * gridDim.y), two = n - n_sm < n_sm ? n - n_sm : n_sm;   // SMs that get two at the start
    if (two > 0) {
      if (rank < n_sm) rank = rank < two ? 2 * rank : rank + two;
      else if (rank < 2 * n_sm) rank = 2 * (rank - n_sm) + 1;
    }
  }
  const int tile = (int)gridDim.y - 1 - rank / (int)gridDim.x, g = rank % (int)gridDim.x, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rep = nh / nkv;
  const int tok0 = cu_seqlens[b];
  const int n_new = cu_seqlens[b + 1] - tok0;
  const int n_rows = n_new * n_rep;
  const int row0 = tile * TROWS;
  if (row0 >= n_rows) return;                         // whole CTA, before anything is allocated

  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t q_s = smem_u32(base);                                 // [NT] tiles of Q
  const uint32_t k_s = q_s + NT * C::Q_BYTES;                          // [NS] pages
  const uint32_t v_s = k_s + NS * C::PAGE_BYTES;                       // [NS] pages
  uint64_t* bars = (uint64_t*)(base + NT * C::Q_BYTES + 2 * NS * C::PAGE_BYTES);
  uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = k_full + NS, *v_full = k_empty + NS, *v_empty = v_full + NS,
           *s_full = v_empty + NS /* [NT][2] */, *s_empty = s_full + 2 * NT, *p_full = s_empty + 2 * NT,
           *p_empty = p_full + NT;
  uint32_t* tmem_holder = (uint32_t*)(p_empty + NT);
  int* failed = (int*)(tmem_holder + 1);
  constexpr int MMA_WARP = 4 * NT, COPY_WARP = 4 * NT + 1;

  if (tid == 0) {
    mbar_init(q_full, 128 * NT);
    for (int i = 0; i < NS; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
    }
    for (int i = 0; i < 2 * NT; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(s_empty + i, 128);
    }
    for (int i = 0; i < NT; ++i) {
      mbar_init(p_full + i, 128);
      mbar_init(p_empty + i, 1);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_holder, W::TMEM_COLS);

  const int L = ctx_lens[b];
  const int start = L - n_new;
  const int* table = page_table + (size_t)b * table_width;
  // pages that any row of the CTA sees: from the window start of its first row to the position of its last
  const int last_row = min(row0 + TROWS - 1, n_rows - 1);
  const int tile_pos_hi = start + last_row / n_rep;
  const int tile_pos_lo = start + row0 / n_rep;
  const int tile_lo = (window > 0 && tile_pos_lo - window + 1 > 0) ? tile_pos_lo - window + 1 : 0;
  const int blk0 = tile_lo / PAGE, blk1 = tile_pos_hi / PAGE + 1;
  const int n_pg = blk1 - blk0;

  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  // tile t: scores in columns t * 128 .. + 127 (two buffers of 64), O in columns NT * 128 + t * HD ..
  auto tmem_S = [&](int t, int bb) { return tmem_base + t * 128 + bb * 64; };
  auto tmem_O = [&](int t) { return tmem_base + NT * 128 + t * HD; };

  if (warp == COPY_WARP) {
    // ---- copies (none with `starve`, the tests' way to make the waits below run out) ----
    if (lane == 0 && !starve) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      int page_next = max(table[blk0], 0);
      for (int j = 0; j < n_pg; ++j) {
        const int st = j % NS, n = j / NS;
        const int row = (page_next * nkv + g) * PAGE;
        if (j + 1 < n_pg) page_next = max(table[blk0 + j + 1], 0);
        if (!mbar_wait(k_empty + st, (n & 1) ^ 1, wait_ns)) { atomicExch(failed, 1); break; }
        mbar_expect_tx(k_full + st, C::PAGE_BYTES);
#pragma unroll
        for (int hb = 0; hb < C::NB; ++hb)
          tma_load_2d(k_s + st * C::PAGE_BYTES + hb * (PAGE * 128), &map_k, hb * 64, row, k_full + st);
        if (!mbar_wait(v_empty + st, (n & 1) ^ 1, wait_ns)) { atomicExch(failed, 1); break; }
        mbar_expect_tx(v_full + st, C::PAGE_BYTES);
#pragma unroll
        for (int hb = 0; hb < C::NB; ++hb)
          tma_load_2d(v_s + st * C::PAGE_BYTES + hb * (PAGE * 128), &map_v, hb * 64, row, v_full + st);
      }
    }
    // a long prompt's kernel lets the kernel after it go only now, when this CTA's copies are all
    // on their way (its CTAs would otherwise sit on SMs that this kernel still needs)
    if (late_trigger) pdl_trigger();
  } else if (warp == MMA_WARP) {
    // ---- MMA issue ----
    if (lane == 0) {
      constexpr uint32_t idesc_qk = instr_desc(64, false);
      constexpr uint32_t idesc_pv = instr_desc(HD, true);
      // the scores of page j for all tiles, the tiles taking turns
      auto issue_qk = [&](int j) {
        fence_after_sync();
        const uint32_t kb = k_s + (j % NS) * C::PAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t ka = kb + (kk >> 2) * (PAGE * 128) + (kk & 3) * 32;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint32_t qa = q_s + t * C::Q_BYTES + (kk >> 2) * (ROWS * 128) + (kk & 3) * 32;
            umma_bf16(tmem_S(t, j & 1), smem_desc(qa, 16), smem_desc(ka, 16), idesc_qk, kk > 0 ? 1u : 0u);
          }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) umma_commit(s_full + t * 2 + (j & 1));
        umma_commit(k_empty + j % NS);
      };
      bool ok = mbar_wait(q_full, 0, wait_ns) && mbar_wait(k_full, 0, wait_ns);
      if (ok) issue_qk(0);
      for (int j = 0; ok && j < n_pg; ++j) {
        if (j + 1 < n_pg) {
          const int j1 = j + 1;
          ok = mbar_wait(k_full + j1 % NS, (j1 / NS) & 1, wait_ns);
#pragma unroll
          for (int t = 0; t < NT; ++t) ok = ok && mbar_wait(s_empty + t * 2 + (j1 & 1), ((j1 >> 1) & 1) ^ 1, wait_ns);
          if (!ok) break;
          issue_qk(j1);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) ok = ok && mbar_wait(p_full + t, j & 1, wait_ns);
        ok = ok && mbar_wait(v_full + j % NS, (j / NS) & 1, wait_ns);
        if (!ok) break;
        fence_after_sync();
        const uint32_t vb = v_s + (j % NS) * C::PAGE_BYTES;
#pragma unroll
        for (int kc = 0; kc < PAGE / 16; ++kc) {
#pragma unroll
          for (int t = 0; t < NT; ++t)
            umma_bf16_ts(tmem_O(t), tmem_S(t, j & 1) + kc * 8, smem_desc(vb + kc * 2048, PAGE * 128),
                      idesc_pv, (j > 0 || kc > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) umma_commit(p_empty + t);
        umma_commit(v_empty + j % NS);
      }
      if (!ok) atomicExch(failed, 1);
    }
  } else {
    // ---- softmax: thread (t, rt) owns row row0 + t * 128 + rt of tile t ----
    const int t = warp >> 2, rt = tid & 127;
    const int r = row0 + t * ROWS + rt;
    const bool valid = r < n_rows;
    const int t_row = valid ? r / n_rep : 0;
    const int h_row = g * n_rep + (valid ? r % n_rep : 0);
    const int p_row = start + t_row;
    const int lo_row = (window > 0 && p_row - window + 1 > 0) ? p_row - window + 1 : 0;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    {
      const __nv_bfloat16* src = q + (size_t)(tok0 + t_row) * q_stride + (size_t)h_row * HD;
      uint8_t* my_q = base + t * C::Q_BYTES;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        uint4 v = valid ? *(const uint4*)(src + c * 8) : make_uint4(0, 0, 0, 0);
        *(uint4*)(my_q + (c >> 3) * (ROWS * 128) + swz(rt, c & 7)) = v;
      }
      fence_async_smem();
      mbar_arrive(q_full);
    }
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_pg; ++j) {
      const int bb = j & 1;
      ok = mbar_wait(s_full + t * 2 + bb, (j >> 1) & 1, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      fence_after_sync();
      uint32_t su[64];
      tmem_ld32(tmem_S(t, bb) + lane_off, su);
      tmem_ld32(tmem_S(t, bb) + lane_off + 32, su + 32);
      tmem_ld_wait();
      fence_before_sync();
      mbar_arrive(s_empty + t * 2 + bb);                   // the score buffer may be overwritten
      const int abs0 = (blk0 + j) * PAGE;
      // four partial maxima (and sums below): a single running value would be a chain of 64
      // dependent instructions.  Only pages that this row does not see whole are masked.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (valid && abs0 + PAGE - 1 <= p_row && abs0 >= lo_row) {
#pragma unroll
        for (int i = 0; i < 64; i += 8) {                  // (pairs of values to a maximum: one three-input instruction)
          mx4[0] = fmaxf(fmaxf(mx4[0], __uint_as_float(su[i])), __uint_as_float(su[i + 1]));
          mx4[1] = fmaxf(fmaxf(mx4[1], __uint_as_float(su[i + 2])), __uint_as_float(su[i + 3]));
          mx4[2] = fmaxf(fmaxf(mx4[2], __uint_as_float(su[i + 4])), __uint_as_float(su[i + 5]));
          mx4[3] = fmaxf(fmaxf(mx4[3], __uint_as_float(su[i + 6])), __uint_as_float(su[i + 7]));
        }
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
      // (two values to an instruction where there is one: fma.f32x2, add.f32x2)
      const float2 scale2 = make_float2(scale_log2, scale_log2), neg_m2 = make_float2(neg_m, neg_m);
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t pw[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(su[2 * i]), __uint_as_float(su[2 * i + 1])), scale2, neg_m2);
        const float2 pr = make_float2(ex2(x.x), ex2(x.y));
        sum2[i & 1] = __fadd2_rn(sum2[i & 1], pr);
        const __nv_bfloat162 pb = __floats2bfloat162_rn(pr.x, pr.y);
        pw[i] = *(const uint32_t*)&pb;
      }
      l_sum += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
      // the weighted values of the page before must be done before O and P are touched
      if (j > 0) {
        ok = mbar_wait(p_empty + t, (j - 1) & 1, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        fence_after_sync();
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // the whole warp takes part (tcgen05.ld/st are warp-wide); rows that keep their maximum use 1
        const float a = rescale ? alpha : 1.f;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t ou[32];
          tmem_ld32(tmem_O(t) + lane_off + c, ou);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ou[i] = __float_as_uint(__uint_as_float(ou[i]) * a);
          tmem_st32(tmem_O(t) + lane_off + c, ou);
        }
        tmem_st_wait();
      }
      // P goes back into tensor memory, over the first 32 columns of the scores that it came
      // from (two bfloat16 a column): P V takes its A operand from there.  The MMAs that wrote
      // those columns and the one that read the weights of two pages ago are done (the scores'
      // barrier came after them); the scores of the page after next, which will overwrite them,
      // are issued after this page's P V and run after it.
      tmem_st32(tmem_S(t, bb) + lane_off, pw);
      tmem_st_wait();
      fence_before_sync();
      mbar_arrive(p_full + t);
    }
    if (ok) {
      ok = mbar_wait(p_empty + t, (n_pg - 1) & 1, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      fence_after_sync();
    }
    if (!ok) atomicExch(failed, 1);
    if (ok) {
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* dst = out + (size_t)(tok0 + t_row) * out_stride + (size_t)h_row * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t ou[32];
        tmem_ld32(tmem_O(t) + lane_off + c, ou);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int jj = 0; jj < 32; jj += 8) {
            uint4 o;
            __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(ou[jj]) * inv, __uint_as_float(ou[jj + 1]) * inv);
            __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(ou[jj + 2]) * inv, __uint_as_float(ou[jj + 3]) * inv);
            __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(ou[jj + 4]) * inv, __uint_as_float(ou[jj + 5]) * inv);
            __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(ou[jj + 6]) * inv, __uint_as_float(ou[jj + 7]) * inv);
            o.x = *(uint32_t*)&a0; o.y = *(uint32_t*)&a1; o.z = *(uint32_t*)&a2; o.w = *(uint32_t*)&a3;
            *(uint4*)(dst + c + jj) = o;
          }
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (*failed) {
    // a wait ran out: give copies in flight time to land before shared memory goes away
    if (tid == 0 && status) atomicExch(status, WPC_ERR_DEVICE_WAIT);
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == MMA_WARP) {
    fence_after_sync();
    tmem_dealloc(tmem_base, W::TMEM_COLS);
  }
}

template <int HD, int NT>
static int launch_ws(const void* q, int q_stride, void* out, int out_stride, const void* k_pages, const void* v_pages,
                     int n_pages, const int* page_table, int table_width, const int* cu_seqlens, const int* ctx_lens,
                     int B, int max_new, int nh, int nkv, float scale, int window, int* status, cudaStream_t stream) {
  using W = WsCfg<HD, NT>;
  static int configured[MAX_DEVICES];
  if (int rc = allow_smem(prefill_ws_kernel<HD, NT>, W::SMEM, configured)) return rc;
  // the cache as a matrix [n_pages * nkv * PAGE, HD]: a page of one KV head is 64 of its rows
  const long rows = (long)n_pages * nkv * PAGE;
  if (rows > 0x7fffffffL) return WPC_ERR_TOO_LARGE;
  CUtensorMap mk, mv;
  int rc = tc::tensor_map(k_pages, (int)rows, HD, HD, PAGE, &mk);
  if (rc) return rc;
  rc = tc::tensor_map(v_pages, (int)rows, HD, HD, PAGE, &mv);
  if (rc) return rc;
  const int n_rep = nh / nkv;
  dim3 grid(nkv, (max_new * n_rep + NT * ROWS - 1) / (NT * ROWS), B);
  wpc::launch(prefill_ws_kernel<HD, NT>, grid, W::THREADS, W::SMEM, stream, mk, mv, (const __nv_bfloat16*)q, q_stride,
              (__nv_bfloat16*)out, out_stride, page_table, table_width, cu_seqlens, ctx_lens, nh, nkv, scale * LOG2E,
              window, status, wait_policy().limit_ns, wait_policy().starve, NT == 1 ? sm_count() : 1 << 30,
              max_new >= 1024 ? 1 : 0);
  return launch_status();
}

}  // namespace fatc
}  // namespace wpc

extern "C" {

int wpc_attention_prefill_tc_supports(int nh, int nkv, int hd) {
  return (hd == 64 || hd == 128) && nkv >= 1 && nh % nkv == 0 && nh / nkv <= 128;
}

// tiles: 1 or 2 row tiles of 128 rows to a CTA (1: two CTAs to an SM, the faster one: 54 against
// 60 us at 2,048 tokens of the 7B shape, 480 against 659 us at 8,192).  n_pages: pages of the cache.
// q rows and out rows must be 16-byte aligned (strides multiples of 8 elements).
int wpc_attention_prefill_tc(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                             const void* v_pages, const int* page_table, int table_width, const int* cu_seqlens,
                             const int* ctx_lens, int B, int max_new, int nh, int nkv, int hd, float scale,
                             int window, int* status, int n_pages, int tiles, cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (!wpc_attention_prefill_tc_supports(nh, nkv, hd) || (q_stride % 8) || (out_stride % 8) ||
      (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15))
    return WPC_ERR_UNSUPPORTED;
  if (tiles == 1 || tiles == 2) {
    // one or two row tiles to a CTA
#define WPC_WS(HD_, NT_)                                                                                          \
  return wpc::fatc::launch_ws<HD_, NT_>(q, q_stride, out, out_stride, k_pages, v_pages, n_pages, page_table,      \
                                        table_width, cu_seqlens, ctx_lens, B, max_new, nh, nkv, scale, window,     \
                                        status, stream)
    if (hd == 128 && tiles == 2) WPC_WS(128, 2);
    if (hd == 128) WPC_WS(128, 1);
    if (tiles == 2) WPC_WS(64, 2);
    WPC_WS(64, 1);
#undef WPC_WS
  }
  return WPC_ERR_BAD_ARGUMENT;
}

}  // extern "C"
