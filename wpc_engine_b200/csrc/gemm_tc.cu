// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//
//     D[M, N] = A[M, K] . B[N, K]^T        (both operands row-major with K contiguous)
//
// Two kernels.  gemm_tc_kernel: one CTA computes one 128 x BN tile of D (optionally only a slice
// of K: split-K); it serves few tokens (swapped arrangement) and the sizes that the second
// does not take.  gemm_pair_kernel (further down): two CTAs of a cluster compute one 256 x 256
// tile with tcgen05.mma.cta_group::2; it serves many tokens.  In gemm_tc_kernel operand
// tiles of 64 K-elements (one 128-byte swizzle row) travel from global to shared memory by TMA
// through a ring of stages; a single thread issues tcgen05.mma into a float32 accumulator in
// tensor memory; four warps read the accumulator back with tcgen05.ld and write the result.
//
//   warp 0      producer: arms a stage's "full" barrier and starts the two TMA loads
//   warp 1      allocates tensor memory, issues the MMAs, frees tensor memory at the end
//   warps 2..5  epilogue: TMEM -> registers -> (+bias, +residual, type) -> global
//
// Two output arrangements:
//   normal   A = activations [tokens, K], B = weights [features, K]; out[token, feature]
//   swapped  A = weights [features, K], B = activations [tokens <= 128, K]; the tile is
//            D^T and the epilogue writes out[token, feature].  This keeps the 128-row MMA
//            full when there are only a few tokens (decode), so the weights stream once at
//            full width.
// Split K, three ways.  (1) Swapped arrangement, the usual one for few tokens: the CTAs of a
// tile form a thread-block cluster (2..8); every rank writes its partial sums of a token row
// into the shared memory of the rank that owns the row (distributed shared memory), and after
// one cluster barrier each rank adds up its rows in rank order and writes them.  No scratch, no
// atomics, the same bits every run.  The ring is kept so short that two CTAs fit on an SM.  (2) With
// tickets: every CTA of a tile writes its partial sums to scratch memory and takes a ticket;
// the CTA that draws the last ticket adds them in slice order and runs the epilogue.  Nobody
// waits for anybody.  (3) When the product is added to a float32 output anyway, the slices
// may add their shares with red.global.add (split products of the normal arrangement; in the
// swapped one the caller chooses it for few tokens and a short K, see ops.py).
// Every wait on an mbarrier is bounded: when it runs out the kernel records
// WPC_ERR_DEVICE_WAIT in `status`, lets its copies land, frees its tensor memory and returns.
// The cluster barriers are hardware barriers that every thread of every CTA reaches on every
// path (each role arrives when its loop ends, however it ended), so a CTA that gave up still
// arrives.
//
// The math is the reference's y = W x + b (wpc-runtime/src/weights.rs:59-78) in bfloat16
// inputs with float32 accumulation.
#include <cuda.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "api.h"
#include "common.cuh"
#include "tensor_map.h"

namespace wpc {
namespace tc {

constexpr int BM = 128;            // rows of A per tile = MMA M
constexpr int BK = 64;             // K elements per stage: 128 bytes of bfloat16, one swizzle row
constexpr int UMMA_K = 16;         // K of one tcgen05.mma for 16-bit inputs
constexpr int THREADS = 192;

struct Params {
  int M, N, K;                 // rows of A, rows of B, shared dimension
  int k_blocks;                // ceil(K / BK)
  int splits;                  // CTAs along K per tile
  const float* bias;           // [features] or null
  void* out;
  int ldc;                     // row stride of out, in elements
  int out_bf16;                // 1: bfloat16, 0: float32
  int accumulate;              // 1: out (float32) += result
  int gated;                   // 0, or the activation (WPC_ACT_*): features come as [64 gate | 64 up] blocks;
                               //    out = act(gate) * up, bfloat16
  float* scratch;              // split-K partial sums: [tile][split][BN][BM] float32
  int* counters;               // one ticket counter per tile, zero between launches
  int* status;                 // device error word (may be null)
  int stages;                  // depth of the operand ring (2..MAX_STAGES)
  int pair_n;                  // gemm_pair_kernel: columns of a pair's tile (128..256 in steps of 16)
  // Cluster variant only (rope_hd != 0): the rows of the output are [q heads | k heads | v heads]
  // of an attention layer.  The tail rotates q and k (pairs (i, i + hd/2), the first rope_R of
  // them, wpc-runtime/src/rope.rs:24-40), writes q to `out` and the rotated k and the v of every
  // token into the cache page of its position (wpc-runtime/src/model.rs:464-475); the k and v
  // columns of `out` are not written.
  int rope_nh, rope_nkv, rope_hd, rope_R;
  const float* rope_cos;       // [tokens, rope_R]
  const float* rope_sin;
  __nv_bfloat16* k_pages;      // [n_pages, nkv, PAGE, hd]
  __nv_bfloat16* v_pages;
  const int* page_table;       // [sequences, table_width]
  int table_width;
  const int* seq_of_token;
  const int* positions;
  int n_pages;
  unsigned long long wait_ns;  // how long a wait on an mbarrier may last (wpc::wait_policy)
  int starve;                  // test switch: the producer starts no copies, so that the waits run out
  int prefetch_weights;        // 1: the weight operand (A when swapped, else B) is never written while the
                               //    model runs, so its first stages may be fetched before the kernel
                               //    ahead in the stream has finished
  int late_trigger;            // 1: the kernel after this one is let go only when this CTA's copies are all on their way
                               //    (pair kernel), not at the start
};

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Bounded wait: false if the barrier did not flip within limit_ns.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > limit_ns) return false;
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
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
// The barrier gets one arrival when all MMAs issued so far by this thread have finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 lanes x 32 columns of 32 bits: thread i of the warp gets lane (base lane + i), columns c..c+31.
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled in
// 1024-byte groups of 8 rows (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): start address,
// 1024 bytes from one group of 8 rows to the next, descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // bits 0..13: start address / 16
  d |= (uint64_t)1 << 16;                            // bits 16..29: leading byte offset / 16 (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                  // bits 32..45: stride byte offset / 16
  d |= (uint64_t)1 << 46;                            // bits 46..47: version 1 (sm_100)
  d |= (uint64_t)2 << 61;                            // bits 61..63: SWIZZLE_128B
  return d;
}
// Instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}


// Shared memory: 1 KiB of barriers and flags, then (1 KiB aligned) the ring of operand stages.
// The number of stages is chosen at launch: a CTA that is alone on its SM takes as many as fit,
// so that enough bytes are in flight to cover the memory latency; two co-resident CTAs share.
constexpr int MAX_STAGES = 12;
constexpr int SMEM_LIMIT = 227 * 1024;
template <int BN, int MT = 1>
struct Smem {
  static constexpr int A_BYTES = MT * BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int HEAD_BYTES = 1024;
  static constexpr int TMEM_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;   // a power of two
  static constexpr int total(int stages) { return HEAD_BYTES + 1024 /* alignment slack */ + stages * STAGE_BYTES; }
  static constexpr int max_stages(int ctas_per_sm, int extra_bytes = 0) {
    int s = (SMEM_LIMIT / ctas_per_sm - HEAD_BYTES - 1024 - 1024 /* per-CTA reserve */ - extra_bytes) / STAGE_BYTES;
    return s > MAX_STAGES ? MAX_STAGES : (s < 2 ? 2 : s);
  }
  // Cluster variant: behind the ring, the partial sums that the ranks of the cluster send to this
  // CTA, [rank][feature][row of this CTA] floats, and the [8][128] floats through which the two
  // halves of a head (or the gate and the up rows of a feature) exchange their values.  Token rows belong to the ranks in groups of four
  // (see the kernel), so a CTA has room for 4 * ceil(ceil(BN / 4) / ranks) rows from each rank.
  __host__ __device__ static constexpr int recv_rows(int ranks) { return 4 * (((BN + 3) / 4 + ranks - 1) / ranks); }
  __host__ __device__ static constexpr int recv_bytes(int ranks) { return (ranks * recv_rows(ranks) + 8) * BM * 4; }
};

__device__ __forceinline__ void store_row32(const Params& p, int row, int col0, int n_cols, const float (&v)[32]) {
  // out[row, col0 .. col0 + n_cols) from v (normal arrangement: this thread owns a row)
  if (p.accumulate) {
    float* dst = (float*)p.out + (size_t)row * p.ldc + col0;
    // all loads first, then all stores: a store between two loads would serialise them
    if (n_cols == 32 && (((uintptr_t)dst) & 15) == 0) {
      float4 o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __ldcg((const float4*)(dst + 4 * j));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j].x += v[4 * j]; o[j].y += v[4 * j + 1]; o[j].z += v[4 * j + 2]; o[j].w += v[4 * j + 3];
        *(float4*)(dst + 4 * j) = o[j];
      }
    } else {
      float o[32];
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < n_cols) o[j] = __ldcg(dst + j);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < n_cols) dst[j] = o[j] + v[j];
    }
  } else if (p.out_bf16) {
    __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)row * p.ldc + col0;
    if (n_cols == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[j], v[j + 1]), b = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 c = __floats2bfloat162_rn(v[j + 4], v[j + 5]), d = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        uint4 o;
        o.x = *(uint32_t*)&a; o.y = *(uint32_t*)&b; o.z = *(uint32_t*)&c; o.w = *(uint32_t*)&d;
        *(uint4*)(dst + j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < n_cols) dst[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float* dst = (float*)p.out + (size_t)row * p.ldc + col0;
    if (n_cols == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *(float4*)(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < n_cols) dst[j] = v[j];
    }
  }
}

// One piece of work of a CTA: a tile and a range of its k-blocks.
struct Work {
  int tile_id, split, m0, n0, kb0, n_kb;
  bool partial;                // the range does not cover the tile's whole K
};
// The pieces of one CTA, in order: (tile, K slice) units blockIdx.x, + gridDim.x, ... with the
// M tile fastest, so that CTAs running side by side share weight tiles.
template <int BN, int MT = 1>
struct WorkIter {
  int n_tiles, tiles_m, k_blocks, splits, kb_per;
  int u, n_units, stride;
  bool split_fastest;          // units count (tile, split) with the split fastest: the CTAs of a cluster share a tile
  __device__ WorkIter(const Params& p, bool split_fastest_ = false) {
    split_fastest = split_fastest_;
    tiles_m = (p.M + MT * BM - 1) / (MT * BM);
    n_tiles = tiles_m * ((p.N + BN - 1) / BN);
    k_blocks = p.k_blocks;
    splits = p.splits;
    kb_per = (k_blocks + splits - 1) / splits;
    u = blockIdx.x;
    n_units = n_tiles * splits;
    stride = gridDim.x;
  }
  __device__ bool next(Work& w) {
    if (u >= n_units) return false;
    if (split_fastest) {
      w.tile_id = u / splits;
      w.split = u - w.tile_id * splits;
    } else {
      w.split = u / n_tiles;
      w.tile_id = u - w.split * n_tiles;
    }
    w.kb0 = w.split * kb_per;
    w.n_kb = max(min(k_blocks, w.kb0 + kb_per) - w.kb0, 0);
    w.partial = splits > 1;
    u += stride;
    const int tile_n = w.tile_id / tiles_m, tile_m = w.tile_id - tile_n * tiles_m;
    w.m0 = tile_m * MT * BM;
    w.n0 = tile_n * BN;
    return true;
  }
};

// MT = 2: the tile is 256 rows of A by BN; the two 128-row halves are two MMAs that share the B
// tile in shared memory (a third less operand traffic per flop) and fill both accumulators, so
// the epilogue does not overlap the next tile.
// CL (swapped arrangement, split K): the CTAs that share a tile form a thread-block cluster.  The
// token rows of the tile belong to the ranks in groups of four (group i to rank i % S): every
// rank writes its partial sums of a group straight into the owner's shared memory, 16 bytes a
// thread (writes to a peer need no answer, but each is a packet between two SMs: one float at a
// time, 64 tokens took 7 to 17 us), one cluster barrier makes them visible, and the owner adds
// them up in rank order and writes the rows.  No scratch, no tickets, no atomics.  The epilogue warps run this whole path once before the dependency
// wait, with every store switched off: a kernel runs each of its instructions once, so on the
// first pass every line of code comes from L2 or beyond, and a dry pass while the warps
// have nothing to do takes those misses off the critical path.
template <int BN, bool SWAP, int MT, bool CL>
__global__ void __launch_bounds__(THREADS, (BN <= 64 ? 2 : 1))     // narrow tiles run two CTAs to an SM
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  using S = Smem<BN, MT>;
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  uint64_t* full = (uint64_t*)smem_raw;
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* accum_full = empty + MAX_STAGES;      // [2]: the MMAs of a unit have finished
  uint64_t* accum_empty = accum_full + 2;         // [2]: the epilogue has read the accumulator
  uint32_t* tmem_holder = (uint32_t*)(accum_empty + 2);
  int* flags = (int*)(tmem_holder + 1);          // [0]: a wait ran out, [1]: this CTA drew the last ticket
  long long* s_rowbase = (long long*)(smem_raw + 512);   // [64] cache places of this CTA's token rows (rope_hd)
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + S::HEAD_BYTES + 1023) & ~(uintptr_t)1023);
  const int STAGES = p.stages;
  float* red_stage = (float*)(tiles + STAGES * S::STAGE_BYTES);    // [4][32][33], present where cut tiles add (see launch)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A CTA walks its pieces of work (see WorkIter) and keeps two accumulators in tensor memory,
  // so that the epilogue of one piece runs while the MMAs of the next fill the other.
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accum_full + b, 1);
      mbar_init(accum_empty + b, 128);
    }
    flags[0] = 0;
    flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_holder, 2 * S::TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  // Cluster variant: a rank may write into a peer's shared memory only once every CTA of the
  // cluster runs.  This comes before the dependency wait, while the kernel before still runs.
  if (CL && p.splits > 1) cluster_sync_all();

  if (warp == 0) {
    if (lane == 0 && !p.starve) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");     // the descriptors themselves
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      int it = 0;                                   // k-blocks loaded so far: position in the ring
      bool ok = true;
      WorkIter<BN, MT> work(p, CL);
      Work w;
      bool first = true;
      while (ok && work.next(w)) {
        const int m0 = w.m0, n0 = w.n0, kb0 = w.kb0, n_kb = w.n_kb;
        int i = 0;
        if (first) {
          first = false;
          // the first ring of stages: the weight operand may start before the dependency wait
          const int pre = p.prefetch_weights ? min(n_kb, STAGES) : 0;
          for (i = 0; i < pre; ++i) {
            mbar_expect_tx(full + i, S::STAGE_BYTES);
            uint8_t* a_dst = tiles + i * S::STAGE_BYTES;
            if (SWAP) tma_load_2d(a_dst, &map_a, (kb0 + i) * BK, m0, full + i);
            else tma_load_2d(a_dst + S::A_BYTES, &map_b, (kb0 + i) * BK, n0, full + i);
          }
          pdl_wait();
          for (i = 0; i < pre; ++i) {
            uint8_t* a_dst = tiles + i * S::STAGE_BYTES;
            if (SWAP) tma_load_2d(a_dst + S::A_BYTES, &map_b, (kb0 + i) * BK, n0, full + i);
            else tma_load_2d(a_dst, &map_a, (kb0 + i) * BK, m0, full + i);
          }
          it = pre;
        }
        for (; i < n_kb; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty + s, ph ^ 1, p.wait_ns)) { atomicExch(flags, 1); ok = false; break; }
          mbar_expect_tx(full + s, S::STAGE_BYTES);
          uint8_t* a_dst = tiles + s * S::STAGE_BYTES;
          tma_load_2d(a_dst, &map_a, (kb0 + i) * BK, m0, full + s);
          tma_load_2d(a_dst + S::A_BYTES, &map_b, (kb0 + i) * BK, n0, full + s);
        }
      }
    }
    __syncwarp();
    if (CL && p.splits > 1) { cluster_arrive(); cluster_wait(); }    // see the epilogue warps
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN);
      bool ok = true;
      int it = 0, j = 0;
      WorkIter<BN, MT> work(p, CL);
      Work w;
      for (; ok && work.next(w); ++j) {
        const int n_kb = w.n_kb;
        const int b = MT == 1 ? (j & 1) : 0;           // two accumulators take turns, or both serve one tile
        const int use = MT == 1 ? (j >> 1) : j;        // how often this accumulator has been used before
        if (!mbar_wait(accum_empty + b, (use & 1) ^ 1, p.wait_ns)) { atomicExch(flags, 1); break; }
        fence_after_sync();
        const uint32_t tmem_d = tmem_base + b * S::TMEM_COLS;
        for (int i = 0; i < n_kb; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(full + s, ph, p.wait_ns)) { atomicExch(flags, 1); ok = false; break; }
          fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + s * S::STAGE_BYTES);
          const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // 32 bytes further along K inside the swizzled row: + 2 in the (address / 16) field
            umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            if (MT == 2)      // rows 128..255 of the A tile lie 16 KiB further; second accumulator
              umma_bf16(tmem_d + S::TMEM_COLS, da + 2 * k + ((BM * BK * 2) >> 4), db + 2 * k, idesc,
                        (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty + s);       // the stage is free again once these MMAs have read it
        }
        if (ok) umma_commit(accum_full + b);    // arrives when everything issued above has finished
      }
    }
    __syncwarp();
    if (CL && p.splits > 1) { cluster_arrive(); cluster_wait(); }
  } else {
    // ---- epilogue: warps 2..5 read lanes 32*(warp % 4) .. +31 of the accumulator ----
    const int q = warp & 3;
    const int r = q * 32 + lane;                        // row of the tile = TMEM lane
    const int et = threadIdx.x - 64;                    // 0..127 among the epilogue threads
    if (CL && p.rope_hd && p.splits > 1) {
      // where in the cache the token rows that this CTA will write go:
      // three dependent loads a row, done here so that they are over when the tail needs them.
      // Positions and page numbers are the step's inputs, written by the host before its first
      // kernel started: they may be read ahead of the dependency wait.
      const int S = p.splits, my = (int)cluster_rank();
      const int tiles_m = (p.M + BM - 1) / BM;
      const int n0 = (blockIdx.x / S / tiles_m) * BN;
      const int n_valid = min(BN, p.N - n0);
      for (int k = et; k < S::recv_rows(S); k += 128) {       // row k of this CTA: group k / 4 of its groups
        const int j = ((k >> 2) * S + my) * 4 + (k & 3);
        if (j >= n_valid) continue;
        const int tok = n0 + j;
        const int pos = p.positions[tok], block = pos / WPC_PAGE;
        const int page = block < p.table_width ? p.page_table[(size_t)p.seq_of_token[tok] * p.table_width + block] : -1;
        s_rowbase[k] = (page >= 0 && page < p.n_pages) ? ((long long)page * p.rope_nkv * WPC_PAGE + pos % WPC_PAGE) : -1;
      }
    }
    if (CL && p.splits > 1) {
      // ---- cluster variant: one unit of work; see the comment above the kernel ----
      asm volatile("bar.sync 1, 128;" ::: "memory");     // s_rowbase is complete
      const int S = p.splits, my = (int)cluster_rank(), kmax = S::recv_rows(S);
      WorkIter<BN, MT> work(p, true);
      Work w;
      work.next(w);
      const int m0 = w.m0, n0 = w.n0;
      const int n_valid = min(BN, p.N - n0);
      const int feat = m0 + r;                           // this thread's feature: row of the tile = TMEM lane
      const bool in_range = feat < p.M;
      // With rope_hd: what this feature is (q, k or v; which head; which element)
      const int hd = p.rope_hd, half = hd >> 1;
      const int nq = p.rope_nh * hd, nk = p.rope_nkv * hd;
      const int kind = !hd ? 0 : (feat < nq ? 0 : (feat < nq + nk ? 1 : 2));       // q, k, v
      const int d = hd ? feat % hd : 0;
      const int kvh = hd ? (kind == 1 ? (feat - nq) / hd : (kind == 2 ? (feat - nq - nk) / hd : 0)) : 0;
      const int pr = hd ? d % half : 0;                   // index of the pair within the head
      const bool rotated = hd && kind < 2 && pr < p.rope_R;
      const float* recv = red_stage + r * kmax;           // [rank][feature][row of this CTA] received sums
      float* xbuf = red_stage + S * kmax * BM;            // [8][128]
      const uint32_t mine = smem_u32(red_stage) + (uint32_t)((my * BM + r) * kmax) * 4;
      // This CTA's groups of four token rows are my, my + S, ...; a round takes ROWS rows: a group
      // where q and k are rotated, two otherwise (64 tokens on 8 ranks are then one round; a round
      // more costs about 2 us, most of it the trip to L2 for what it adds to).  What a round needs from
      // global memory is fetched a round ahead: for the first round, before the MMAs end.
      float bias = 0.f, cs[4], sn[4], old[8];
      __nv_bfloat16* dst[4];
      auto fetch = [&](auto rows_c, int k0) {
        constexpr int ROWS = decltype(rows_c)::value;
#pragma unroll
        for (int u = 0; u < ROWS; ++u) {
          const int k = k0 + u, j = ((k >> 2) * S + my) * 4 + (k & 3);      // row k of this CTA is token j of the tile
          old[u] = 0.f;
          if (ROWS == 4) { cs[u & 3] = 1.f; sn[u & 3] = 0.f; dst[u & 3] = nullptr; }
          if (in_range && j < n_valid) {
            const int tok = n0 + j;
            if (ROWS == 4 && rotated) {
              // past L1: the dry pass may have read these before the kernel that writes them ended
              cs[u & 3] = __ldcg(p.rope_cos + (size_t)tok * p.rope_R + pr);
              sn[u & 3] = __ldcg(p.rope_sin + (size_t)tok * p.rope_R + pr);
            }
            if (ROWS == 4 && hd && kind > 0) {
              const long long base = s_rowbase[k];                 // page * nkv * PAGE + place in the page
              if (base >= 0)
                dst[u & 3] = (kind == 1 ? p.k_pages : p.v_pages) + ((size_t)base + (size_t)kvh * WPC_PAGE) * hd + d;
              else if (p.status) atomicExch(p.status, WPC_ERR_BAD_ARGUMENT);
            } else if (!hd && p.accumulate) {
              old[u] = __ldcg((const float*)p.out + (size_t)tok * p.ldc + feat);   // only this thread writes it
            }
          }
        }
      };
      // the rounds of the tail: sums of the received slices in rank order, rotation, store
      auto rounds = [&](auto rows_c, bool dry) {
        constexpr int ROWS = decltype(rows_c)::value;
        for (int k0 = 0; ((k0 >> 2) * S + my) * 4 < n_valid; k0 += ROWS) {
          float val[ROWS];
#pragma unroll
          for (int g4 = 0; g4 < ROWS; g4 += 4) {
            float4 sum = *(const float4*)(recv + k0 + g4);
            for (int s2 = 1; s2 < S; ++s2) {                                   // in rank order
              const float4 t = *(const float4*)(recv + s2 * kmax * BM + k0 + g4);
              sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
            }
            val[g4] = sum.x + bias; val[g4 + 1] = sum.y + bias; val[g4 + 2] = sum.z + bias; val[g4 + 3] = sum.w + bias;
          }
          if (ROWS == 8 && p.gated) {
            // rows 64..127 of the tile are the up rows of the features in rows 0..63: the upper
            // half hands its sums over, the lower half writes silu(gate) * up (model.rs:527-531)
#pragma unroll
            for (int u = 0; u < ROWS; ++u) xbuf[u * BM + r] = val[u];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (r < 64) {
              WPC_WITH_ACT(p.gated, ACT, {
#pragma unroll
                for (int u = 0; u < ROWS; ++u) val[u] = xbuf[u * BM + r + 64] * gate_act<true, ACT>(val[u]);
              });
#pragma unroll
              for (int u = 0; u < ROWS; ++u) {
                const int k = k0 + u, j = ((k >> 2) * S + my) * 4 + (k & 3);
                if (j < n_valid && !dry)
                  ((__nv_bfloat16*)p.out)[(size_t)(n0 + j) * p.ldc + (m0 >> 1) + r] = __float2bfloat16_rn(val[u]);
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");     // the buffer is written again in the next round
            continue;
          }
          if (ROWS == 4 && hd) {
            // x'_i = x_i c - x_{i+half} s;  x'_{i+half} = x_{i+half} c + x_i s  (rope.rs:36-39)
#pragma unroll
            for (int u = 0; u < ROWS; ++u) xbuf[(u & 3) * BM + r] = val[u];
            asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
            for (int u = 0; u < ROWS; ++u) {
              const float other = xbuf[(u & 3) * BM + (r ^ half)];
              if (rotated) val[u] = d < half ? val[u] * cs[u & 3] - other * sn[u & 3] : val[u] * cs[u & 3] + other * sn[u & 3];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");     // the buffer is written again in the next round
          }
#pragma unroll
          for (int u = 0; u < ROWS; ++u) {
            const int k = k0 + u, j = ((k >> 2) * S + my) * 4 + (k & 3);
            if (j < n_valid && in_range && !dry) {
              const size_t o = (size_t)(n0 + j) * p.ldc + feat;
              if (ROWS == 4 && hd && kind > 0) { if (dst[u & 3]) *dst[u & 3] = __float2bfloat16_rn(val[u]); }
              else if (p.accumulate) ((float*)p.out)[o] = old[u] + val[u];
              else if (p.out_bf16) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(val[u]);
              else ((float*)p.out)[o] = val[u];
            }
          }
          if ((((k0 + ROWS) >> 2) * S + my) * 4 < n_valid) fetch(rows_c, k0 + ROWS);
        }
      };
      const std::integral_constant<int, 4> four;
      const std::integral_constant<int, 8> eight;
      const int passes = p.k_blocks > 0 ? 2 : 1;          // always 2; the compiler must keep one copy of the body
#pragma unroll 1
      for (int pass = 0; pass < passes; ++pass) {
        const bool dry = pass + 1 < passes;               // the pass that only brings the code in
        if (!dry) pdl_wait();                             // the output and the inputs of fetch() are shared
        if (in_range && p.bias) bias = p.bias[feat];
        if (hd) fetch(four, 0); else fetch(eight, 0);
        bool ok = true;
        if (!dry) {
          ok = mbar_wait(accum_full, 0, p.wait_ns);
          ok = __all_sync(0xffffffffu, ok);               // tcgen05.ld needs the whole warp on one path
          if (!ok) atomicExch(flags, 1);
          fence_after_sync();
        }
        const bool have_acc = w.n_kb > 0 && ok;
        // the dry pass reads the accumulator that this variant never fills
        const uint32_t lane_addr = tmem_base + (dry ? S::TMEM_COLS : 0) + ((uint32_t)(q * 32) << 16);
        for (int c = 0; c < n_valid; c += 32) {
          uint32_t v[32];
          if (BN >= 32) tmem_ld32(lane_addr + c, v); else tmem_ld16(lane_addr + c, v);
          tmem_ld_wait();
          int owner = (c >> 2) % S, lg = (c >> 2) / S;        // the group of columns c .. c + 3: whose, and which of theirs
#pragma unroll
          for (int j = 0; j < (BN >= 32 ? 32 : 16); j += 4) {
            if (c + j < n_valid && !dry) {
              const uint32_t at = peer_smem(mine + (uint32_t)lg * 16, (uint32_t)owner);
              if (have_acc)
                st_peer_f32x4(at, __uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
              else
                st_peer_f32x4(at, 0.f, 0.f, 0.f, 0.f);
            }
            if (++owner == S) { owner = 0; ++lg; }
          }
        }
        if (!dry) {
          fence_before_sync();
          mbar_arrive(accum_empty);
          cluster_arrive();                               // this rank's sums are on their way
          cluster_wait();                                 // every rank's sums for this CTA's rows have arrived
        }
        if (hd) rounds(four, dry); else rounds(eight, dry);
      }
      // Nothing reads a peer's shared memory: the CTA may leave when its own rows are written.
    } else {
    pdl_wait();                                         // the output, the scratch and the tickets are shared
    int j = 0;
    WorkIter<BN, MT> work(p, CL);
    Work w;
    for (; work.next(w); ++j) {
      const int n0 = w.n0, n_kb = w.n_kb, split = w.split, tile_id = w.tile_id;
      const int b = MT == 1 ? (j & 1) : 0;
      const int use = MT == 1 ? (j >> 1) : j;
      bool ok = mbar_wait(accum_full + b, use & 1, p.wait_ns);
      ok = __all_sync(0xffffffffu, ok);              // tcgen05.ld needs the whole warp on one path
      if (!ok) atomicExch(flags, 1);
      fence_after_sync();
      const int n_valid = min(BN, p.N - n0);              // columns of the tile that exist
      const bool have_acc = n_kb > 0 && ok;
      for (int half = 0; half < MT; ++half) {             // the 128-row halves of a 256-row tile
      const int m0 = w.m0 + half * BM;
      const uint32_t lane_addr = tmem_base + (MT == 1 ? b : half) * S::TMEM_COLS + ((uint32_t)(q * 32) << 16);

      bool run_epilogue = ok;
      if (w.partial && p.accumulate) {
        // Every slice adds its share straight into the float32 output with red.global.add: no
        // scratch, no tickets, no fences.  The order in which the slices arrive is not fixed,
        // so the sum may differ in its last bits from run to run.
        run_epilogue = false;
        for (int c = 0; c < n_valid && have_acc; c += 32) {
          uint32_t v[32];
          if (BN >= 32) tmem_ld32(lane_addr + c, v); else tmem_ld16(lane_addr + c, v);
          tmem_ld_wait();
          const int nc = min(32, n_valid - c);
          if (!SWAP) {
            // this thread holds 32 columns of one row; through shared memory the warp turns its
            // 32 x 32 block around, so that one red.add instruction covers 32 columns of a row
            float* st = red_stage + q * (32 * 33);
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              st[lane * 33 + j] = __uint_as_float(v[j]) + ((p.bias && split == 0 && j < nc) ? p.bias[n0 + c + j] : 0.f);
            __syncwarp();
            if (lane < nc) {
              for (int rr = 0; rr < 32; ++rr) {
                const int row = m0 + q * 32 + rr;
                if (row < p.M) atomicAdd((float*)p.out + (size_t)row * p.ldc + n0 + c + lane, st[rr * 33 + lane]);
              }
            }
          } else {
            const int feat = m0 + r;
            if (feat < p.M) {
              const float bsum = (p.bias && split == 0) ? p.bias[feat] : 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < nc) atomicAdd((float*)p.out + (size_t)(n0 + c + j) * p.ldc + feat, __uint_as_float(v[j]) + bsum);
            }
          }
        }
      } else if (p.splits > 1) {
        // partial sums to scratch: [tile][split][column][row], rows contiguous
        float* part = p.scratch + ((size_t)tile_id * p.splits + split) * (size_t)(BN * BM);
        for (int c = 0; c < n_valid; c += 32) {
          uint32_t v[32];
          if (have_acc) {
            if (BN >= 32) tmem_ld32(lane_addr + c, v); else tmem_ld16(lane_addr + c, v);
            tmem_ld_wait();
          }
          const int nc = min(32, n_valid - c);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < nc) part[(size_t)(c + j) * BM + r] = have_acc ? __uint_as_float(v[j]) : 0.f;
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          const int ticket = atomicAdd(p.counters + tile_id, 1);
          flags[1] = (ticket == p.splits - 1);
          if (ticket == p.splits - 1) p.counters[tile_id] = 0;      // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        run_epilogue = ok && flags[1];
        if (run_epilogue) __threadfence();
      }

      if (run_epilogue && p.gated) {
        // gate and up rows are interleaved in blocks of 64 features (wpc-runtime/src/model.rs:527-531)
        if (!SWAP) {
          // columns of the tile: [64 gate | 64 up] repeated; this thread owns token row m0 + r
          const int row = m0 + r;
          for (int c = 0; c < (BN >= 128 ? BN : 0); c += 128) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              uint32_t ug[32], uu[32];
              float v[32];
              if (have_acc) {
                tmem_ld32(lane_addr + c + 32 * k, ug);
                tmem_ld32(lane_addr + c + 64 + 32 * k, uu);
                tmem_ld_wait();
              }
              WPC_WITH_ACT(p.gated, ACT, {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float g = have_acc ? __uint_as_float(ug[j]) : 0.f, u = have_acc ? __uint_as_float(uu[j]) : 0.f;
                  v[j] = gate_act<true, ACT>(g) * u;
                }
              });
              if (row < p.M) store_row32(p, row, (n0 + c) / 2 + 32 * k, 32, v);
            }
          }
        } else {
          // rows of the tile: 64 gate features, then the 64 up rows of the same features; the
          // upper half hands its values to the lower half through shared memory (the operand
          // stages are free: every MMA has finished).  The lower half works on all columns of a
          // chunk at once, whether they hold tokens or not: a test per column would turn the
          // chains of exp and division into branches that run one after the other (stamps of
          // clock64 gave 85 ns a token, 2.6 us for 32 tokens).  The results of a chunk then pass
          // through shared memory once more, so that a thread stores 16 bytes of a token's row
          // (a store of one bfloat16 per thread and token took 50 ns each, 1.7 us for 32 tokens).
          float* xch = (float*)tiles;                                          // [BN][64]
          __nv_bfloat16* xo = (__nv_bfloat16*)(tiles + BN * 64 * 4);           // [32][64] a chunk's results
          const bool wide = (p.ldc & 7) == 0 && (((uintptr_t)p.out) & 15) == 0;
          constexpr int W = BN >= 32 ? 32 : 16;
          for (int c = 0; c < n_valid; c += 32) {
            uint32_t u32[32];
            if (have_acc) {
              if (BN >= 32) tmem_ld32(lane_addr + c, u32); else tmem_ld16(lane_addr + c, u32);
              tmem_ld_wait();
            }
            const int nc = min(32, n_valid - c);
            if (r >= 64) {
#pragma unroll
              for (int j = 0; j < W; ++j)
                if (j < nc) xch[(c + j) * 64 + (r - 64)] = have_acc ? __uint_as_float(u32[j]) : 0.f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (r < 64) {
              const int feat = (m0 >> 1) + r;
              float res[W];
#pragma unroll
              for (int j = 0; j < W; ++j) res[j] = xch[(c + j) * 64 + r];
              // (SiLU's quotient to 2 units in the last place of float32, far inside the bfloat16
              // that it becomes: the exact division has a slow path, a branch again)
              WPC_WITH_ACT(p.gated, ACT, {
#pragma unroll
                for (int j = 0; j < W; ++j) {
                  const float g = have_acc ? __uint_as_float(u32[j]) : 0.f;
                  res[j] *= gate_act<true, ACT>(g);
                }
              });
              if (wide) {
#pragma unroll
                for (int j = 0; j < W; ++j) xo[j * 64 + r] = __float2bfloat16_rn(res[j]);
                asm volatile("bar.sync 2, 64;" ::: "memory");                 // the two warps of the lower half
                for (int piece = r; piece < nc * 8; piece += 64) {
                  const int token = piece >> 3, part = piece & 7;
                  *(uint4*)((__nv_bfloat16*)p.out + (size_t)(n0 + c + token) * p.ldc + (m0 >> 1) + part * 8) =
                      *(const uint4*)(xo + token * 64 + part * 8);
                }
              } else if (feat < (p.M >> 1)) {
#pragma unroll
                for (int j = 0; j < W; ++j)
                  if (j < nc)
                    ((__nv_bfloat16*)p.out)[(size_t)(n0 + c + j) * p.ldc + feat] = __float2bfloat16_rn(res[j]);
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
        }
      } else if (run_epilogue) {
        const float* part0 = p.scratch ? p.scratch + (size_t)tile_id * p.splits * (size_t)(BN * BM) : nullptr;
        for (int c = 0; c < n_valid; c += 32) {
          const int nc = min(32, n_valid - c);
          float v[32];
          if (p.splits > 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
            for (int z = 0; z < p.splits; ++z) {
              const float* pz = part0 + (size_t)z * (BN * BM);
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < nc) v[j] += __ldcg(pz + (size_t)(c + j) * BM + r);
            }
          } else {
            uint32_t u[32];
            if (have_acc) {
              if (BN >= 32) tmem_ld32(lane_addr + c, u); else tmem_ld16(lane_addr + c, u);
              tmem_ld_wait();
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = have_acc ? __uint_as_float(u[j]) : 0.f;
          }
          if (!SWAP) {
            // this thread owns token row m0 + r and features n0 + c ..
            const int row = m0 + r;
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < nc) v[j] += __ldg(p.bias + n0 + c + j);
            }
            if (row < p.M) store_row32(p, row, n0 + c, nc, v);
          } else {
            // this thread owns feature m0 + r, the columns are tokens n0 + c ..
            const int feat = m0 + r;
            if (feat < p.M) {
              const float b = p.bias ? p.bias[feat] : 0.f;
              if (p.accumulate) {
                // all loads first, then all stores: a store between two loads would serialise them
                float old[32];
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j < nc) old[j] = __ldcg((const float*)p.out + (size_t)(n0 + c + j) * p.ldc + feat);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j < nc) ((float*)p.out)[(size_t)(n0 + c + j) * p.ldc + feat] = old[j] + v[j] + b;
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (j < nc) {
                    const size_t o = (size_t)(n0 + c + j) * p.ldc + feat;
                    const float val = v[j] + b;
                    if (p.out_bf16) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(val);
                    else ((float*)p.out)[o] = val;
                  }
                }
              }
            }
          }
        }
      }

      }                                                   // halves
      // the accumulator may be overwritten now
      fence_before_sync();
      mbar_arrive(accum_empty + b);
      if (!ok) break;
    }
    }
  }

  fence_before_sync();
  __syncthreads();
  if (flags[0]) {
    // a wait ran out: give copies in flight time to land before shared memory goes away
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, WPC_ERR_DEVICE_WAIT);
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, 2 * S::TMEM_COLS);
  }
}

// ---- the product on pairs of SMs (tcgen05 cta_group::2) -----------------------------------------
// Normal arrangement, many tokens.  Two CTAs of a cluster compute one 256 x 256 tile of D: CTA
// `rank` holds rows m0 + 128*rank .. +127 of A and rows n0 + 128*rank .. +127 of B in its shared
// memory; one thread of the leader (rank 0) issues tcgen05.mma.cta_group::2 with M = 256, which
// reads A from each CTA's own memory and B from both, and leaves each CTA's 128 rows of D in its
// own tensor memory.  Against 128 x 256 tiles on single SMs every SM fetches a third less per
// flop.  Protocol (as in CUTLASS's sm100 2-SM kernels):
//   * both producers copy with cta_group::2 TMA loads that signal the LEADER's "full" barrier;
//     the leader's producer arms it with the bytes of both CTAs;
//   * the leader's MMA thread commits to the "empty" barrier of both CTAs (multicast commit),
//     and to the "accumulator full" barrier of both;
//   * the epilogue warps of both CTAs arrive on the leader's "accumulator empty" barrier;
//   * tensor memory is allocated and freed by one warp of each CTA with cta_group::2.
// Cluster barriers (hardware, reached by every thread on every path) stand after the set-up
// and before the exit; every mbarrier wait is bounded as in the kernel above.
// With few tiles and a float32 output that is added to (p.splits > 1), a pair's unit of work is a
// slice of a tile's K; every slice adds its share with red.global.add.v4 (the last bits of the sum
// then depend on the order of arrival).
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = 2 * BM * BK * 2;       // this CTA's halves of A and B: 16 KiB each
constexpr int PAIR_SMEM = 1024 + 1024 + PAIR_STAGES * PAIR_STAGE_BYTES + 1024;     // + a tile's bias
constexpr int PAIR_N = 256;

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival at `bar` of both CTAs of the pair when all MMAs issued so far have finished.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void red_add_f32x4(float* dst, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* holder, int cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, int cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

template <bool ROPE>      // ROPE: the epilogue of the q/k/v projection (rotation and cache write), see there
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  if (!p.late_trigger) pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  uint64_t* full = (uint64_t*)smem_raw;                  // [PAIR_STAGES], used in the leader
  uint64_t* empty = full + PAIR_STAGES;                   // [PAIR_STAGES], in each CTA
  uint64_t* accum_full = empty + PAIR_STAGES;             // [2], in each CTA
  uint64_t* accum_empty = accum_full + 2;                 // [2], used in the leader: 256 arrivals
  uint32_t* tmem_holder = (uint32_t*)(accum_empty + 2);
  int* flags = (int*)(tmem_holder + 1);
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1024 + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                   // 0: leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int PN = p.pair_n;                                // columns of the tile; each CTA holds PN / 2 rows of B
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int n_tiles = tiles_m * ((p.N + PN - 1) / PN);
  // units of work: (tile, slice of K), the slices of a tile side by side
  const int S = p.splits, kb_per = (p.k_blocks + S - 1) / S;
  const int n_units = n_tiles * S;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accum_full + b, 1);
      mbar_init(accum_empty + b, 256);
    }
    flags[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(tmem_holder, 512);
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                                     // both CTAs' barriers exist before anything signals them
  fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0 && !p.starve) {
      pdl_wait();
      int it = 0;
      bool ok = true;
      for (int u = pair; ok && u < n_units; u += n_pairs) {
        const int t = u / S, slice = u - t * S;
        const int tile_n = t / tiles_m, tile_m = t - tile_n * tiles_m;
        const int m0 = tile_m * 2 * BM + (int)rank * BM, n0 = tile_n * PN + (int)rank * (PN >> 1);
        const int kb0 = slice * kb_per, n_kb = max(min(p.k_blocks, kb0 + kb_per) - kb0, 0);
        for (int i = 0; i < n_kb; ++i, ++it) {
          const int s = it % PAIR_STAGES;
          const uint32_t ph = (it / PAIR_STAGES) & 1;
          if (!mbar_wait(empty + s, ph ^ 1, p.wait_ns)) { atomicExch(flags, 1); ok = false; break; }
          if (rank == 0) mbar_expect_tx(full + s, 2 * (BM * BK * 2 + (PN >> 1) * BK * 2));
          const uint32_t leader_bar = peer_smem(smem_u32(full + s), 0);
          uint8_t* dst = tiles + s * PAIR_STAGE_BYTES;
          tma_load_2d_pair(dst, &map_a, (kb0 + i) * BK, m0, leader_bar);
          tma_load_2d_pair(dst + BM * BK * 2, &map_b, (kb0 + i) * BK, n0, leader_bar);
        }
      }
      if (p.late_trigger) pdl_trigger();
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // M = 256 over the pair, N = 256, bfloat16 inputs, float32 accumulator, both operands K-major
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PN >> 3) << 17) |
                             ((uint32_t)((2 * BM) >> 4) << 24);
      int it = 0, j = 0;
      bool ok = true;
      for (int u = pair; ok && u < n_units; u += n_pairs, ++j) {
        const int slice = u % S;
        const int kb0 = slice * kb_per, n_kb = max(min(p.k_blocks, kb0 + kb_per) - kb0, 0);
        const int b = j & 1, use = j >> 1;
        if (!mbar_wait(accum_empty + b, (use & 1) ^ 1, p.wait_ns)) { atomicExch(flags, 1); break; }
        fence_after_sync();
        const uint32_t tmem_d = tmem_base + b * PAIR_N;
        for (int i = 0; i < n_kb; ++i, ++it) {
          const int s = it % PAIR_STAGES;
          const uint32_t ph = (it / PAIR_STAGES) & 1;
          if (!mbar_wait(full + s, ph, p.wait_ns)) { atomicExch(flags, 1); ok = false; break; }
          fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + s * PAIR_STAGE_BYTES);
          const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + BM * BK * 2);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(empty + s);
        }
        if (ok) umma_commit_pair(accum_full + b);
      }
    }
  } else {
    pdl_wait();
    const int q = warp & 3;
    const int r = q * 32 + lane;
    // The bias of a tile's columns comes into shared memory while the tile's MMAs run: read from
    // global memory chunk by chunk in the epilogue, each chunk's line was a trip to L2 or beyond
    // between two stores (8 us a tile, measured with one tile to a pair).
    float* s_bias = (float*)(tiles + PAIR_STAGES * PAIR_STAGE_BYTES);      // [256]
    int j = 0;
    for (int u = pair; u < n_units; u += n_pairs, ++j) {
      const int t = u / S, slice = u - t * S;
      const int tile_n = t / tiles_m, tile_m = t - tile_n * tiles_m;
      const int m0 = tile_m * 2 * BM + (int)rank * BM, n0 = tile_n * PN;
      const int n_kb = max(min(p.k_blocks, (slice + 1) * kb_per) - slice * kb_per, 0);
      const int b = j & 1, use = j >> 1;
      if (p.bias) {
        asm volatile("bar.sync 1, 128;" ::: "memory");     // the epilogue of the tile before has read its bias
        s_bias[r] = n0 + r < p.N ? __ldg(p.bias + n0 + r) : 0.f;
        s_bias[r + 128] = n0 + r + 128 < p.N ? __ldg(p.bias + n0 + r + 128) : 0.f;
      }
      // (the place of this thread's token in the cache: three loads that hang on one another,
      // looked up while the tile's MMAs run)
      long long rope_base = -1;
      if (ROPE && m0 + r < p.M) {
        const int pos = p.positions[m0 + r], block = pos / WPC_PAGE;
        const int page = block < p.table_width ? p.page_table[(size_t)p.seq_of_token[m0 + r] * p.table_width + block] : -1;
        if (page >= 0 && page < p.n_pages) rope_base = (long long)page * p.rope_nkv * WPC_PAGE + pos % WPC_PAGE;
      }
      bool ok = mbar_wait(accum_full + b, use & 1, p.wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (p.bias) {
        // the bias is written; and the four warps agree on whether the wait ran out, so that
        // none of them meets the barrier above alone
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 q, %1, 0;\n\t"
            "bar.red.and.pred p, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
        ok = all_ok != 0;
      }
      if (!ok) atomicExch(flags, 1);
      fence_after_sync();
      const int n_valid = min(PN, p.N - n0);
      const bool have_acc = n_kb > 0 && ok;
      const uint32_t lane_addr = tmem_base + b * PAIR_N + ((uint32_t)(q * 32) << 16);
      const int row = m0 + r;
      if (ok && p.gated) {
        // columns: [64 gate | 64 up] repeated (wpc-runtime/src/model.rs:527-531)
        for (int c = 0; c < PN; c += 128) {
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            uint32_t ug[32], uu[32];
            float v[32];
            if (have_acc) {
              tmem_ld32(lane_addr + c + 32 * k, ug);
              tmem_ld32(lane_addr + c + 64 + 32 * k, uu);
              tmem_ld_wait();
            }
            // (SiLU's quotient by __fdividef, as in the epilogues for few tokens: the result
            // becomes bfloat16 at once, and the exact division has a slow path, a branch an element)
            WPC_WITH_ACT(p.gated, ACT, {
#pragma unroll
              for (int jj = 0; jj < 32; ++jj) {
                const float g = have_acc ? __uint_as_float(ug[jj]) : 0.f, u = have_acc ? __uint_as_float(uu[jj]) : 0.f;
                v[jj] = gate_act<true, ACT>(g) * u;
              }
            });
            if (row < p.M && c < n_valid) store_row32(p, row, (n0 + c) / 2 + 32 * k, 32, v);
          }
        }
      } else if (ROPE && ok) {
        // The q/k/v projection: the columns are [q heads | k heads | v heads] of width hd (64 or
        // 128, so that a head lies inside the tile).  This thread's token row: q and k are rotated
        // (pairs (i, i + hd/2), the first rope_R of them, rope.rs:24-40); q goes to `out`, the
        // rotated k and v into the page of the token's position (model.rs:464-475).
        const int hd = p.rope_hd, half = hd >> 1;
        const int nq = p.rope_nh * hd, nk = p.rope_nkv * hd;
        const long long base = rope_base;                  // page * nkv * PAGE + place in the page
        const bool in_m = row < p.M;
        if (in_m && base < 0 && n0 + PN > nq && p.status) atomicExch(p.status, WPC_ERR_BAD_ARGUMENT);
        // a block of 32 pairs at a time: its cosines and sines serve every head of the tile
        // (each thread reads its own row of the tables: 16 bytes a load where the rows allow it; a
        // load of 4 bytes a lane from 32 different lines costs the load unit as much)
        const bool vec = (p.rope_R & 3) == 0 && ((((uintptr_t)p.rope_cos) | ((uintptr_t)p.rope_sin)) & 15) == 0;
        for (int pb = 0; pb < half; pb += 32) {
          float cs[32], sn[32];
          if (vec) {
#pragma unroll
            for (int jj = 0; jj < 32; jj += 4) {
              const bool rot = in_m && pb + jj < p.rope_R;
              const float4 c4 = rot ? __ldg((const float4*)(p.rope_cos + (size_t)row * p.rope_R + pb + jj)) : make_float4(1.f, 1.f, 1.f, 1.f);
              const float4 s4 = rot ? __ldg((const float4*)(p.rope_sin + (size_t)row * p.rope_R + pb + jj)) : make_float4(0.f, 0.f, 0.f, 0.f);
              cs[jj] = c4.x; cs[jj + 1] = c4.y; cs[jj + 2] = c4.z; cs[jj + 3] = c4.w;
              sn[jj] = s4.x; sn[jj + 1] = s4.y; sn[jj + 2] = s4.z; sn[jj + 3] = s4.w;
            }
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const bool rot = in_m && pb + jj < p.rope_R;
              cs[jj] = rot ? __ldg(p.rope_cos + (size_t)row * p.rope_R + pb + jj) : 1.f;
              sn[jj] = rot ? __ldg(p.rope_sin + (size_t)row * p.rope_R + pb + jj) : 0.f;
            }
          }
          for (int h0 = 0; h0 < n_valid; h0 += hd) {       // heads of the tile
            const int feat0 = n0 + h0;                     // first feature of the head
            const int kind = feat0 < nq ? 0 : (feat0 < nq + nk ? 1 : 2);
            uint32_t ua[32], ub[32];
            if (have_acc) {
              tmem_ld32(lane_addr + h0 + pb, ua);
              tmem_ld32(lane_addr + h0 + half + pb, ub);
              tmem_ld_wait();
            }
            float va[32], vb[32];
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const float a = (have_acc ? __uint_as_float(ua[jj]) : 0.f) + (p.bias ? s_bias[h0 + pb + jj] : 0.f);
              const float bq = (have_acc ? __uint_as_float(ub[jj]) : 0.f) + (p.bias ? s_bias[h0 + half + pb + jj] : 0.f);
              if (kind < 2) {
                va[jj] = a * cs[jj] - bq * sn[jj];
                vb[jj] = bq * cs[jj] + a * sn[jj];
              } else {
                va[jj] = a;
                vb[jj] = bq;
              }
            }
            if (!in_m) continue;
            if (kind == 0) {
              store_row32(p, row, feat0 + pb, 32, va);
              store_row32(p, row, feat0 + half + pb, 32, vb);
            } else if (base >= 0) {
              const int kvh = (kind == 1 ? feat0 - nq : feat0 - nq - nk) / hd;
              __nv_bfloat16* dst = (kind == 1 ? p.k_pages : p.v_pages) + ((size_t)base + (size_t)kvh * WPC_PAGE) * hd;
#pragma unroll
              for (int jj = 0; jj < 32; jj += 8) {
                uint4 oa, ob;
                __nv_bfloat162 t0 = __floats2bfloat162_rn(va[jj], va[jj + 1]), t1 = __floats2bfloat162_rn(va[jj + 2], va[jj + 3]);
                __nv_bfloat162 t2 = __floats2bfloat162_rn(va[jj + 4], va[jj + 5]), t3 = __floats2bfloat162_rn(va[jj + 6], va[jj + 7]);
                oa.x = *(uint32_t*)&t0; oa.y = *(uint32_t*)&t1; oa.z = *(uint32_t*)&t2; oa.w = *(uint32_t*)&t3;
                t0 = __floats2bfloat162_rn(vb[jj], vb[jj + 1]); t1 = __floats2bfloat162_rn(vb[jj + 2], vb[jj + 3]);
                t2 = __floats2bfloat162_rn(vb[jj + 4], vb[jj + 5]); t3 = __floats2bfloat162_rn(vb[jj + 6], vb[jj + 7]);
                ob.x = *(uint32_t*)&t0; ob.y = *(uint32_t*)&t1; ob.z = *(uint32_t*)&t2; ob.w = *(uint32_t*)&t3;
                *(uint4*)(dst + pb + jj) = oa;
                *(uint4*)(dst + half + pb + jj) = ob;
              }
            }
          }
        }
      } else if (ok && (S > 1 || p.accumulate)) {
        // Added to the float32 output, 16 bytes a reduction (the bias comes with the first slice
        // of K).  Also when K is whole: a reduction needs no answer, where loading the old
        // values, adding and storing is a round trip to L2 for each of the eight chunks of a row
        // (about 19 us for a tile's epilogue, measured; each element still gets exactly one
        // addition, so the result is the same bits every run).
        for (int c = 0; c < n_valid && have_acc; c += 32) {
          const int nc = min(32, n_valid - c);
          uint32_t uu[32];
          tmem_ld32(lane_addr + c, uu);
          tmem_ld_wait();
          if (row >= p.M) continue;
          float* dst = (float*)p.out + (size_t)row * p.ldc + n0 + c;
          const bool with_bias = p.bias && slice == 0;
          if (nc == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
            for (int jj = 0; jj < 32; jj += 4) {
              float a4[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) a4[e] = __uint_as_float(uu[jj + e]) + (with_bias ? s_bias[c + jj + e] : 0.f);
              red_add_f32x4(dst + jj, a4[0], a4[1], a4[2], a4[3]);
            }
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              if (jj < nc) atomicAdd(dst + jj, __uint_as_float(uu[jj]) + (with_bias ? s_bias[c + jj] : 0.f));
          }
        }
      } else if (ok) {
        for (int c = 0; c < n_valid; c += 32) {
          const int nc = min(32, n_valid - c);
          uint32_t u[32];
          float v[32];
          if (have_acc) {
            tmem_ld32(lane_addr + c, u);
            tmem_ld_wait();
          }
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) v[jj] = have_acc ? __uint_as_float(u[jj]) : 0.f;
          if (p.bias) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              if (jj < nc) v[jj] += s_bias[c + jj];
          }
          if (row < p.M) store_row32(p, row, n0 + c, nc, v);
        }
      }
      fence_before_sync();
      mbar_arrive_cluster(peer_smem(smem_u32(accum_empty + b), 0));   // the leader's barrier, from both CTAs
      if (!ok) break;
    }
  }

  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                                     // the peer is done with this CTA's memory and barriers
  if (flags[0]) {
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, WPC_ERR_DEVICE_WAIT);
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  int rows, cols, ld, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.ld;
    h = h * 1000003u ^ (size_t)k.box_rows;
    return h;
  }
};

// A tensor map for a row-major bfloat16 matrix [rows, cols] with row stride ld elements,
// copied in boxes of box_rows x 64 with the 128-byte swizzle.  Encoded maps are kept: the
// same weights are multiplied step after step.
int tensor_map(const void* ptr, int rows, int cols, int ld, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  const MapKey key{ptr, rows, cols, ld, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return WPC_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return WPC_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache[key] = *out;
  return 0;
}

// Upper limit of the ring depth (a tuning knob; MAX_STAGES by default).
static int g_stage_limit = MAX_STAGES;

template <int BN, bool SWAP, int MT = 1, bool CL = false>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, Params& p, cudaStream_t stream) {
  using S = Smem<BN, MT>;
  static int configured[MAX_DEVICES];
  if (int rc = allow_smem(gemm_tc_kernel<BN, SWAP, MT, CL>, S::total(S::max_stages(1)), configured)) return rc;
  p.wait_ns = wait_policy().limit_ns;
  p.starve = wait_policy().starve;
  const int sms = sm_count();
  const long units = (long)((p.M + MT * BM - 1) / (MT * BM)) * ((p.N + BN - 1) / BN) * p.splits;
  if (units > 0x7fffffffL) return WPC_ERR_TOO_LARGE;
  if (CL) {
    // one CTA per (tile, K slice), the slices of a tile side by side in one cluster
    if (p.splits < 2 || p.splits > 8) return WPC_ERR_UNSUPPORTED;
    // a ring so short that two CTAs fit on an SM: more clusters then run side by side (the
    // clusters of a GPC's SMs leave fewer SMs idle), and all of them must stream at once
    const int recv_bytes = S::recv_bytes(p.splits);
    int stages = S::max_stages(BN <= 64 ? 2 : 1, recv_bytes);
    const int kb_per = (p.k_blocks + p.splits - 1) / p.splits;
    if (stages > kb_per) stages = kb_per < 2 ? 2 : kb_per;
    if (stages > g_stage_limit) stages = g_stage_limit < 2 ? 2 : g_stage_limit;
    p.stages = stages;
    // behind the ring: the sums that the other ranks send (see Smem::recv_bytes)
    wpc::launch_clusters(gemm_tc_kernel<BN, SWAP, MT, CL>, dim3((unsigned)units), THREADS, S::total(stages) + recv_bytes,
                         stream, (unsigned)p.splits, ma, mb, p);
    return launch_status();
  }
  // Many tiles in the normal arrangement: one persistent CTA per SM walks the tiles, its
  // epilogue overlapping the next tile's MMAs.  Otherwise one CTA per unit; if those are few,
  // each is alone on its SM and takes a deep ring, if many, two share an SM.
  const bool persistent = !SWAP && p.splits == 1 && units > sms;
  const int per_sm = persistent ? 1 : ((units > sms && S::max_stages(2) >= 4) ? 2 : 1);
  int stages = S::max_stages(per_sm);
  const int kb_per = (p.k_blocks + p.splits - 1) / p.splits;
  if (!persistent && stages > kb_per) stages = kb_per < 2 ? 2 : kb_per;
  if (stages > g_stage_limit) stages = g_stage_limit < 2 ? 2 : g_stage_limit;
  p.stages = stages;
  dim3 grid(persistent ? (unsigned)sms : (unsigned)units);
  // cut tiles of the normal arrangement that add into the output turn their blocks around in
  // shared memory first (see the epilogue): room for [4][32][33] floats behind the ring
  constexpr int RED_STAGE_BYTES = 4 * 32 * 33 * 4;
  const bool red_stage = !SWAP && p.accumulate && p.splits > 1;
  if (red_stage && S::total(stages) + RED_STAGE_BYTES > S::total(S::max_stages(1))) p.stages = --stages;
  // A product over many tokens does not start ahead of the kernel before it: measured on B200,
  // CTAs of these long kernels that become resident early (as SMs happen to fall free) run the
  // whole product slower (o_proj 97 against 75 us, down 268 against 236 us at 2,048 tokens of
  // the 7B shape), far more than the two microseconds of launch latency that the overlap saves.
  // With 512 tokens the kernels are short and the overlap still wins (10.5 against 10.7 ms).
  if (!SWAP && p.M >= 1024) wpc::pdl_skip_next() = 1;
  wpc::launch(gemm_tc_kernel<BN, SWAP, MT, CL>, grid, THREADS, S::total(stages) + (red_stage ? RED_STAGE_BYTES : 0), stream,
              ma, mb, p);
  return launch_status();
}

template <bool ROPE>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, Params& p, cudaStream_t stream) {
  static int configured[MAX_DEVICES];
  if (int rc = allow_smem(gemm_pair_kernel<ROPE>, PAIR_SMEM, configured)) return rc;
  p.wait_ns = wait_policy().limit_ns;
  p.starve = wait_policy().starve;
  const long max_pairs = sm_count() / 2;
  if (p.splits < 1) p.splits = 1;
  const long n_tiles = (long)((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + p.pair_n - 1) / p.pair_n) * p.splits;
  if (n_tiles > 0x3fffffffL) return WPC_ERR_TOO_LARGE;
  const unsigned pairs = (unsigned)(n_tiles < max_pairs ? n_tiles : max_pairs);
  p.stages = PAIR_STAGES;
  // Long kernels neither start early nor let the kernel after them start early (see launch()):
  // early CTAs of either would hold SMs that the running kernel still needs.  They signal their
  // dependents only when a CTA's last copies are on their way, which hides the launch of the
  // next kernel behind the last tiles (a 2,048-token prefill of the 7B shape 25.1 to 24.8 ms).
  p.late_trigger = p.M >= 1024 ? 1 : 0;
  wpc::launch_clusters(gemm_pair_kernel<ROPE>, dim3(2 * pairs), THREADS, PAIR_SMEM, stream, 2u, ma, mb, p);
  return launch_status();
}

}  // namespace tc
}  // namespace wpc

using namespace wpc;
using namespace wpc::tc;

extern "C" {

// Limits the depth of the operand ring (2..12); returns the old limit.
int wpc_gemm_tc_set_stage_limit(int limit) {
  const int was = g_stage_limit;
  g_stage_limit = limit < 2 ? 2 : (limit > MAX_STAGES ? MAX_STAGES : limit);
  return was;
}

// How many float32 of scratch and how many counters a call with these sizes needs.
int wpc_gemm_tc_workspace(int rows_a, int rows_b, int bn, int splits, size_t* scratch_floats, int* n_counters) {
  const int tiles = ((rows_a + BM - 1) / BM) * ((rows_b + bn - 1) / bn);
  *scratch_floats = splits > 1 ? (size_t)tiles * splits * bn * BM : 0;
  *n_counters = splits > 1 ? tiles : 0;
  return 0;
}

// a: [rows_a, K] bfloat16, row stride lda; b: [rows_b, K] bfloat16, row stride ldb.
// swap = 0: out[rows_a, rows_b] (bias over rows_b);  swap = 1: out[rows_b, rows_a] (bias over
// rows_a).  bn: the tile's extent along rows_b (16, 32, 64, 128; 256 without swap).
// gated = WPC_ACT_SILU (1) or WPC_ACT_GELU_TANH (2): the weights hold gate and up rows interleaved
// in blocks of 64 features (64 gate rows, then the 64 up rows of the same features); out is
// [tokens, features / 2] bfloat16 = act(gate) * up.  Needs no bias, no split except in clusters, and bn >= 128 in the normal arrangement.
// tall = 1 (no split; normal arrangement with bn 256, or swapped with bn 128): tiles of 256 rows
// of a on one SM, see the kernel;
// tall = 2: 256 x bn tiles on pairs of SMs (gemm_pair_kernel), bn 128..256 in steps of 16; with
// accumulate (and no gate) splits > 1 cuts K into that many slices, which add with red.add.
// prefetch_weights = 1 promises that the weights are not written by earlier work still in
// flight on the stream (model parameters): their first tiles are then fetched before the
// preceding kernel has finished.
int wpc_gemm_tc(const void* a, int lda, int rows_a, const void* b, int ldb, int rows_b, int K, const float* bias,
                void* out, int out_dtype, int ldc, int accumulate, int gated, int swap, int bn, int splits,
                float* scratch, size_t scratch_floats, int* counters, int n_counters, int* status,
                int prefetch_weights, int tall, int cluster, cudaStream_t stream) {
  if (rows_a <= 0 || rows_b <= 0) return 0;
  if (cluster && (!swap || splits < 2 || splits > 8)) return WPC_ERR_UNSUPPORTED;
  if (tall && swap && (tall != 1 || splits > 1 || cluster || bn != 128)) return WPC_ERR_UNSUPPORTED;
  // (pair tiles may split K when the result is added to a float32 output and nothing else is done to it)
  if (tall && !swap && (tall > 2 || (tall == 1 && (bn != 256 || splits > 1)) ||
                        (tall == 2 && splits > 1 && (!accumulate || gated))))
    return WPC_ERR_UNSUPPORTED;
  if (tall == 2 && (bn < 128 || bn > 256 || bn % 16 || (gated && bn % 128))) return WPC_ERR_UNSUPPORTED;
  if (K <= 0 || (lda % 8) || (ldb % 8) || (((uintptr_t)a) & 15) || (((uintptr_t)b) & 15)) return WPC_ERR_UNSUPPORTED;
  if (accumulate && out_dtype != WPC_DTYPE_F32) return WPC_ERR_BAD_ARGUMENT;
  if (gated != 0 && gated != WPC_ACT_SILU && gated != WPC_ACT_GELU_TANH) return WPC_ERR_BAD_ARGUMENT;
  Params p = {};
  p.stages = 2;
  p.M = rows_a; p.N = rows_b; p.K = K;
  p.k_blocks = (K + BK - 1) / BK;
  p.splits = splits < 1 ? 1 : (splits > p.k_blocks ? p.k_blocks : splits);
  p.bias = bias; p.out = out; p.ldc = ldc;
  p.out_bf16 = out_dtype == WPC_DTYPE_BF16; p.accumulate = accumulate;
  p.gated = gated;
  p.scratch = scratch; p.counters = counters; p.status = status;
  p.prefetch_weights = prefetch_weights;
  if (gated && (bn < (swap ? 16 : 128) || (p.splits != 1 && !cluster) || accumulate || !p.out_bf16 || bias ||
                (swap ? rows_a % BM : rows_b % 128)))
    return WPC_ERR_UNSUPPORTED;
  if (cluster && p.splits < 2) cluster = 0;
  if (p.splits > 1 && !accumulate && !cluster) {
    size_t need_f; int need_c;
    wpc_gemm_tc_workspace(rows_a, rows_b, bn, p.splits, &need_f, &need_c);
    if (!scratch || !counters || need_f > scratch_floats || need_c > n_counters) return WPC_ERR_TOO_LARGE;
  }
  CUtensorMap ma, mb;
  int rc = tensor_map(a, rows_a, K, lda, tall == 1 ? 2 * BM : BM, &ma);
  if (rc) return rc;
  rc = tensor_map(b, rows_b, K, ldb, tall == 2 ? bn / 2 : bn, &mb);
  if (rc) return rc;
  if (!swap && tall == 2) {
    p.pair_n = bn;
    return launch_pair<false>(ma, mb, p, stream);
  }
  if (!swap && tall) {
    if (bn == 256) return launch<256, false, 2>(ma, mb, p, stream);
  } else if (!swap) {
    switch (bn) {
      case 64: return launch<64, false>(ma, mb, p, stream);
      case 128: return launch<128, false>(ma, mb, p, stream);
      case 256: return launch<256, false>(ma, mb, p, stream);
    }
  } else if (tall) {
    if (bn == 128) return launch<128, true, 2>(ma, mb, p, stream);
  } else if (cluster) {
    switch (bn) {
      case 16: return launch<16, true, 1, true>(ma, mb, p, stream);
      case 32: return launch<32, true, 1, true>(ma, mb, p, stream);
      case 64: return launch<64, true, 1, true>(ma, mb, p, stream);
      case 128: return launch<128, true, 1, true>(ma, mb, p, stream);
    }
  } else {
    switch (bn) {
      case 16: return launch<16, true>(ma, mb, p, stream);
      case 32: return launch<32, true>(ma, mb, p, stream);
      case 64: return launch<64, true>(ma, mb, p, stream);
      case 128: return launch<128, true>(ma, mb, p, stream);
    }
  }
  return WPC_ERR_UNSUPPORTED;
}

// The q/k/v projection of an attention layer with the rotation and the cache write in the
// product's epilogue.  Few tokens (bn 16..128): the cluster variant, 2 <= splits <= 8, tokens
// <= 128.  Many tokens (bn = 256): the pair kernel, hd 64 or 128.
//   x [tokens, K] bfloat16, w [(nh + 2 nkv) * hd, K] bfloat16 (rows: q heads, k heads, v
//   heads), bias float32 or null, out [tokens, (nh + 2 nkv) * hd] bfloat16 (row stride ldc).
// q is rotated and written to its columns of out; k is rotated and, like v, written into the
// page of its token's position; the k and v columns of out are left alone.  hd must be 16, 32,
// 64 or 128, so that both halves of a head lie in one 128-feature tile.  cos, sin: float32
// [tokens, R] (R <= hd / 2 pairs are rotated), or R = 0.
int wpc_gemm_tc_rope_store(const void* w, int ldw, const void* x, int ldx, int tokens, int K, const float* bias, void* out,
                           int ldc, int bn, int splits, int prefetch_weights, int nh, int nkv, int hd, int R,
                           const float* cosv, const float* sinv, void* k_pages, void* v_pages, const int* page_table,
                           int table_width, const int* seq_of_token, const int* positions, int n_pages, int* status,
                           cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int features = (nh + 2 * nkv) * hd;
  const bool many = bn == 256;                       // many tokens: the pair kernel (splits is ignored)
  if ((hd != 16 && hd != 32 && hd != 64 && hd != 128) || nh < 1 || nkv < 1 || R < 0 || R > hd / 2 ||
      (R > 0 && (!cosv || !sinv)))
    return WPC_ERR_UNSUPPORTED;
  if (many ? (hd < 64) : (tokens > 128 || splits < 2 || splits > 8)) return WPC_ERR_UNSUPPORTED;
  if (K <= 0 || (ldw % 8) || (ldx % 8) || (((uintptr_t)w) & 15) || (((uintptr_t)x) & 15)) return WPC_ERR_UNSUPPORTED;
  Params p = {};
  p.k_blocks = (K + BK - 1) / BK;
  p.K = K;
  p.bias = bias; p.out = out; p.ldc = ldc; p.out_bf16 = 1;
  p.status = status;
  p.prefetch_weights = prefetch_weights;
  p.rope_nh = nh; p.rope_nkv = nkv; p.rope_hd = hd; p.rope_R = R;
  p.rope_cos = cosv; p.rope_sin = sinv;
  p.k_pages = (__nv_bfloat16*)k_pages; p.v_pages = (__nv_bfloat16*)v_pages;
  p.page_table = page_table; p.table_width = table_width;
  p.seq_of_token = seq_of_token; p.positions = positions; p.n_pages = n_pages;
  if (many) {
    // normal arrangement: A = tokens, B = weights, 256 x 256 tiles on pairs of SMs
    p.M = tokens; p.N = features; p.splits = 1; p.pair_n = 256;
    CUtensorMap ma, mb;
    int rc = tensor_map(x, tokens, K, ldx, BM, &ma);
    if (rc) return rc;
    rc = tensor_map(w, features, K, ldw, BM, &mb);
    if (rc) return rc;
    return launch_pair<true>(ma, mb, p, stream);
  }
  p.M = features; p.N = tokens;
  p.splits = splits > p.k_blocks ? p.k_blocks : splits;
  if (p.splits < 2) return WPC_ERR_UNSUPPORTED;
  CUtensorMap ma, mb;
  int rc = tensor_map(w, features, K, ldw, BM, &ma);
  if (rc) return rc;
  rc = tensor_map(x, tokens, K, ldx, bn, &mb);
  if (rc) return rc;
  switch (bn) {
    case 16: return launch<16, true, 1, true>(ma, mb, p, stream);
    case 32: return launch<32, true, 1, true>(ma, mb, p, stream);
    case 64: return launch<64, true, 1, true>(ma, mb, p, stream);
    case 128: return launch<128, true, 1, true>(ma, mb, p, stream);
  }
  return WPC_ERR_UNSUPPORTED;
}

// How many clusters of `splits` CTAs of the swapped kernel with tile width bn the device can
// hold at once (0 if the sizes are not supported); -1 on a CUDA error.  The runtime's answer is
// for one CTA to an SM; up to a tile width of 64 the kernel keeps its ring so short that two fit
// (see launch), and measured on B200 twice as many clusters then run side by side, so the answer
// is doubled there.
int wpc_gemm_tc_cluster_capacity(int bn, int splits) {
  if (splits < 2 || splits > 8) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(splits * sm_count()));
  cfg.blockDim = dim3(THREADS);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e = cudaErrorInvalidValue;
#define WPC_CAP(BN_)                                                                                              \
  {                                                                                                               \
    using S = Smem<BN_, 1>;                                                                                       \
    cfg.dynamicSmemBytes = S::total(S::max_stages(BN_ <= 64 ? 2 : 1, S::recv_bytes(splits))) + S::recv_bytes(splits); \
    e = cudaFuncSetAttribute(gemm_tc_kernel<BN_, true, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                             S::total(S::max_stages(1)));                                                         \
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<BN_, true, 1, true>, &cfg);       \
  }
  switch (bn) {
    case 16: WPC_CAP(16) break;
    case 32: WPC_CAP(32) break;
    case 64: WPC_CAP(64) break;
    case 128: WPC_CAP(128) break;
    default: return 0;
  }
#undef WPC_CAP
  if (e != cudaSuccess) { cudaGetLastError(); return -1; }
  return bn <= 64 ? 2 * n : n;
}

}  // extern "C"

// ---- the variant that allocates nothing (see no_alloc.h) ------------------------------------------
#include "no_alloc.h"

// Scratch of the static variant: partial sums, then the tickets, then a status word.  In host
// code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char wpc_static_scratch[WPC_STATIC_SCRATCH_BYTES];

namespace wpc {
namespace tc {

// The device address of the scratch array on the current device, looked up once per device.
static int static_scratch_address(unsigned char** out) {
  static unsigned char* addr[MAX_DEVICES] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return WPC_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> g(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, wpc_static_scratch);
    if (e != cudaSuccess) return (int)e;
    addr[dev] = (unsigned char*)p;
  }
  *out = addr[dev];
  return 0;
}

// A tensor map built on the caller's stack: the static variant keeps no cache, so that it
// touches no heap either.
static int tensor_map_uncached(const void* ptr, int rows, int cols, int ld, int box_rows, CUtensorMap* out) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return WPC_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : WPC_ERR_UNSUPPORTED;
}

}  // namespace tc
}  // namespace wpc

extern "C" int wpc_linear_few_tokens_static(const void* x, int ldx, int tokens, const void* w, int ldw, int features,
                                            int K, const float* bias, void* out, int out_dtype, int ldc, int splits,
                                            cudaStream_t stream) {
  if (tokens < 1 || tokens > 128 || features < 1 || K < 1 || splits < 0) return WPC_ERR_BAD_ARGUMENT;
  if ((ldx % 8) || (ldw % 8) || (((uintptr_t)x) & 15) || (((uintptr_t)w) & 15)) return WPC_ERR_UNSUPPORTED;
  if (out_dtype != WPC_DTYPE_BF16 && out_dtype != WPC_DTYPE_F32) return WPC_ERR_BAD_ARGUMENT;
  const int bn = tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : 128;
  const int tiles = (features + BM - 1) / BM;
  const int k_blocks = (K + BK - 1) / BK;
  if (tiles > WPC_STATIC_MAX_TILES) return WPC_ERR_TOO_LARGE;
  const size_t per_split = (size_t)tiles * bn * BM;
  if (splits == 0) {
    splits = sm_count() / tiles;
    if (splits > k_blocks / 4) splits = k_blocks / 4;
    if (splits > 16) splits = 16;
    while (splits > 1 && per_split * splits > WPC_STATIC_SCRATCH_FLOATS) --splits;
    if (splits < 1) splits = 1;
  }
  if (splits > k_blocks) splits = k_blocks;
  if (splits > 1 && per_split * splits > WPC_STATIC_SCRATCH_FLOATS) return WPC_ERR_TOO_LARGE;

  unsigned char* base = nullptr;
  int rc = static_scratch_address(&base);
  if (rc) return rc;
  float* scratch = (float*)base;
  int* counters = (int*)(base + (size_t)WPC_STATIC_SCRATCH_FLOATS * 4);
  int* status = counters + WPC_STATIC_MAX_TILES;
  // the tickets must start at zero whatever an earlier call left behind; the status word behind
  // them is left alone, so that wpc_linear_few_tokens_static_status sees what any call recorded
  cudaError_t e = cudaMemsetAsync(counters, 0, WPC_STATIC_MAX_TILES * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;

  Params p = {};
  p.stages = 2;
  p.M = features; p.N = tokens; p.K = K;
  p.k_blocks = k_blocks;
  p.splits = splits;
  p.bias = bias; p.out = out; p.ldc = ldc;
  p.out_bf16 = out_dtype == WPC_DTYPE_BF16; p.accumulate = 0;
  p.gated = 0;
  p.scratch = scratch; p.counters = counters; p.status = status;
  p.prefetch_weights = 0;
  CUtensorMap ma, mb;
  rc = tensor_map_uncached(w, features, K, ldw, BM, &ma);
  if (rc) return rc;
  rc = tensor_map_uncached(x, tokens, K, ldx, bn, &mb);
  if (rc) return rc;
  switch (bn) {
    case 16: return launch<16, true>(ma, mb, p, stream);
    case 32: return launch<32, true>(ma, mb, p, stream);
    case 64: return launch<64, true>(ma, mb, p, stream);
    default: return launch<128, true>(ma, mb, p, stream);
  }
}

extern "C" int wpc_linear_few_tokens_static_status(int* status_out, cudaStream_t stream) {
  if (!status_out) return WPC_ERR_BAD_ARGUMENT;
  unsigned char* base = nullptr;
  int rc = static_scratch_address(&base);
  if (rc) return rc;
  int* status = (int*)(base + (size_t)WPC_STATIC_SCRATCH_FLOATS * 4) + WPC_STATIC_MAX_TILES;
  cudaError_t e = cudaMemcpyAsync(status_out, status, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e == cudaSuccess && *status_out != 0) e = cudaMemsetAsync(status, 0, sizeof(int), stream);
  return (int)e;
}
