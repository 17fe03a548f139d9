// Prefill attention on tcgen05: S = Q.K^T and O += P.V as UMMA instructions with the
// accumulators in tensor memory, operands brought by TMA.
//
// A block takes 256 query tokens of one head of one sequence as two tiles of 128
// rows, A and B.  Warp 0 is the TMA producer, warps 1 and 10 issue the products of tile
// A and of tile B, warps 2-5 are the softmax group of tile A and warps 6-9 that of tile
// B: one query row per thread.  Keys and values come in blocks of 64 through rings of
// three stages each and serve both tiles.  Per block of keys and per tile: the tile's
// issuer puts S = Q.K^T into one of the tile's two buffers of 64 columns of TMEM (two
// blocks ahead of the softmax); each softmax thread reads its row of S (tcgen05.ld),
// applies scale and mask, keeps a reference maximum and the sum in 32-bit, and writes
// exp2(s - reference) in the 16-bit type back over the first 32 columns of that S buffer
// (tcgen05.st, two keys per column); the issuer then puts O += P.V (P as the A operand
// from tensor memory, V as the MN-major B operand exactly as TMA lays its rows down)
// into the tile's O columns.  Nothing of P touches shared memory: at 128 bytes a clock
// shared memory is what bounds these products (Q and K for S alone are 6 KB per 32
// clocks of arithmetic), and P there cost a fifth of the kernel's time.
//
// Each issuer is a whole warp that runs the (uniform) loop, with lane 0 issuing under a
// predicate: the descriptors then stay in uniform registers.  One issuer for both tiles,
// and in a branch that a single lane takes, was what bounded the kernel (about 80 clocks
// per instruction, 23 % tensor pipe); a stage of K or V is free once both have committed it.
//
// O stays in TMEM for the whole row of blocks.  Its reference maximum is raised
// only when a block's maximum exceeds it by more than 8 (in log2 units, so
// probabilities stay below 256): then the warp waits for the previous block's product,
// reads its O rows, scales them and writes them back (tcgen05.st) before the next
// product is issued.  The final division by the sum uses the same reference, so the
// result is the plain softmax.
//
// Same mathematics as the reference's attn_dot / attn_softmax / att_mix
// (infer.cu:339-523) and as attention.cu.  Keys and values are this step's own rows
// (prompts from their first token) or, for prompts that go on from earlier steps and do
// not wrap around their ring in this step, the cache's rows, this step's included (a block
// of 64 keys is then one page, or 64 rows of the sequence's block); head sizes 64 and 128.
// Every wait on a barrier is bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <type_traits>

#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int TA_BM = 128;     // query rows per tile; a block takes two tiles
constexpr int TA_BN = 64;      // keys per iteration
constexpr int TA_THREADS = 352;
constexpr int TA_MMA_B = 10;   // the warp that issues tile B's products (warp 1: tile A's)
constexpr int TA_KSTAGES = 3;
constexpr int TA_VSTAGES = 3;
constexpr float TA_RAISE = 8.f;   // a block's maximum may exceed the reference by this much (log2)

__device__ __forceinline__ void ta_tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                               uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// K-major operand tile: rows of 128 bytes (64 bf16), 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t ta_desc_k(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand (V as TMA stores it: one row per key, 64 head elements = 128 bytes per
// row, the next 64 head elements `lbo` bytes further): 8-key groups 1024 B apart
__device__ __forceinline__ uint64_t ta_desc_mn(uint32_t addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// A product issued from a whole warp: every lane runs the (uniform) descriptor arithmetic, so
// it can stay in uniform registers, and the instruction itself is issued by the lane whose
// `leader` is set.  (Inside a branch that one lane takes, every operand goes from a vector
// register to a uniform one, one transfer after the other: about 80 clocks per instruction.)
__device__ __forceinline__ void ta_umma_by(uint32_t leader, uint32_t tmem_d, uint64_t adesc,
                                           uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
// ... with the A operand in tensor memory (row m in lane m, two 16-bit elements per column)
__device__ __forceinline__ void ta_umma_tmem_a_by(uint32_t leader, uint32_t tmem_d, uint32_t tmem_a,
                                                  uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
__device__ __forceinline__ void ta_commit_by(uint32_t leader, uint32_t bar) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %1, 0;\n"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}"
      ::"r"(bar), "r"(leader) : "memory");
}
__device__ __forceinline__ void ta_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The same load without the wait: several can be in flight; ta_ld_wait32 then makes
// the registers of one of them (and, by the instruction's meaning, of all earlier
// ones) valid, and ta_ld_after32 ties the registers of another to that point.
__device__ __forceinline__ void ta_ld32_issue(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
#define YALM_R32(r)                                                                              \
  "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), \
  "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),       \
  "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),     \
  "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),     \
  "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
__device__ __forceinline__ void ta_ld_wait32(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : YALM_R32(r) : : "memory");
}
__device__ __forceinline__ void ta_ld_after32(uint32_t* r) {
  asm volatile("" : YALM_R32(r) : : "memory");
}
#undef YALM_R32
__device__ __forceinline__ void ta_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])),
        "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
        "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ta_ex2(float x) {            // 2^x; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Where the keys and values come from.  `on` = 0: this step's own rows (every sequence starts
// at its first token; map_k and map_v are one map over [tokens, 2 * G * HD]).  `on` = 1: the
// cache, which already holds this step's rows as well (sequences that go on from `slot_pos`;
// none of them wraps around its ring in this step): map_k and map_v cover the layer's K and V
// as rows of HD elements, one block per sequence ((slot * G + g) * capacity + position) or,
// with a page table, pages of 64 positions ((g * n_pages + page) * 64 + position % 64).
struct ta_cache_args {
  const int* seq_slot;
  const int* slot_pos;
  const int* page_table;
  int pages_per_slot, n_pages, capacity, on;
};

template <int HD, typename T16>
__global__ void __launch_bounds__(TA_THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const ta_cache_args ca,
                       const int* __restrict__ q_start, T16* __restrict__ out, int H, int G,
                       int window, float scale_log2, int* __restrict__ status) {
  constexpr uint32_t FMT = std::is_same<T16, __nv_bfloat16>::value ? 1u : 0u;   // operand format
  constexpr int SUB = HD / 64;                     // 64-column sub-tiles of a head
  constexpr int Q_BYTES = TA_BM * HD * 2;          // one query tile
  constexpr int KV_BYTES = TA_BN * HD * 2;         // one block of K or of V
  constexpr int TMEM_COLS = 512;                   // S: 2 tiles x 2 buffers x 64; O: 2 tiles x HD
  extern __shared__ uint8_t ta_smem[];
  __shared__ __align__(8) uint64_t q_full, s_full[2][2], p_ready[2][2], pv_done[2][2];
  __shared__ __align__(8) uint64_t k_full[TA_KSTAGES], k_empty[TA_KSTAGES];
  __shared__ __align__(8) uint64_t v_full[TA_VSTAGES], v_empty[TA_VSTAGES];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  // heads run fastest in the grid, then sequences, and a sequence's blocks come from its
  // end: the long blocks of every head and sequence start before any short one
  const int b = blockIdx.y, h = blockIdx.x;
  const int g = h / (H / G);
  // (broadcast from lane 0: the same value in every lane, and known to be)
  const int qs = __shfl_sync(0xffffffffu, q_start[b], 0);      // written by a host copy: safe early
  const int q_len = __shfl_sync(0xffffffffu, q_start[b + 1], 0) - qs;
  // Positions are written by the advance kernel alone, which lets nothing start before it
  // has ended: they too may be read while the previous kernel still runs.
  const int slot = ca.on ? __shfl_sync(0xffffffffu, ca.seq_slot[b], 0) : 0;
  const int past = ca.on ? __shfl_sync(0xffffffffu, ca.slot_pos[slot], 0) : 0;
  const int n_blocks = (q_len + 2 * TA_BM - 1) / (2 * TA_BM);
  if ((int)blockIdx.z >= n_blocks) return;
  const int m0 = (n_blocks - 1 - (int)blockIdx.z) * 2 * TA_BM;
  // per tile: first row, rows, and the blocks of keys [kb0, kb1) its rows can see
  int t_m0[2], t_rows[2], t_kb0[2], t_kb1[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    t_m0[x] = m0 + x * TA_BM;
    t_rows[x] = max(0, min(TA_BM, q_len - t_m0[x]));
    const int k_end = past + t_m0[x] + t_rows[x];
    const int k_begin = window > 0 ? max(0, past + t_m0[x] - window + 1) : 0;
    t_kb0[x] = k_begin / TA_BN;
    t_kb1[x] = t_rows[x] > 0 ? (k_end + TA_BN - 1) / TA_BN : t_kb0[x];
  }
  const int kb_lo = t_kb0[0];
  const int kb_hi = t_rows[1] > 0 ? t_kb1[1] : t_kb1[0];
  const int n_it = kb_hi - kb_lo;
  auto active = [&](int x, int kb) { return kb >= t_kb0[x] && kb < t_kb1[x]; };

  const uint32_t base = (smem_u32(ta_smem) + 1023u) & ~1023u;
  const uint32_t q_s = base;                                    // tiles A and B
  const uint32_t k_s = q_s + 2 * Q_BYTES;
  const uint32_t v_s = k_s + TA_KSTAGES * KV_BYTES;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), 1);
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&s_full[x][0]), 1);
      mbar_init(smem_u32(&s_full[x][1]), 1);
      for (int buf = 0; buf < 2; ++buf) {
        mbar_init(smem_u32(&p_ready[x][buf]), TA_BM);
        mbar_init(smem_u32(&pv_done[x][buf]), 1);
      }
    }
    for (int s = 0; s < TA_KSTAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), 2);
    }
    for (int s = 0; s < TA_VSTAGES; ++s) {
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 2);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_slot, 0);
  // columns: two S buffers of tile A, two of tile B, O of tile A, O of tile B
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 2 * TA_BN};
  const uint32_t tmem_o[2] = {tmem_base + 4 * TA_BN, tmem_base + 4 * TA_BN + HD};
  volatile int* abort_p = &abort_flag;
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
      pdl_wait();
      const int n_tiles = t_rows[1] > 0 ? 2 : 1;
      mbar_expect_tx(smem_u32(&q_full), n_tiles * Q_BYTES);
      for (int x = 0; x < n_tiles; ++x)
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub)
          ta_tma_load_2d(q_s + x * Q_BYTES + sub * (TA_BM * 128), &map_q, h * HD + sub * 64,
                         qs + t_m0[x], smem_u32(&q_full));
      for (int it = 0; it < n_it; ++it) {
        // the block's first row in the maps, and the columns of K and of V
        const int kb = kb_lo + it;
        int row = qs + kb * TA_BN, col_k = g * HD, col_v = (G + g) * HD;
        if (ca.on) {
          col_k = col_v = 0;
          if (ca.page_table != nullptr)
            row = (g * ca.n_pages + ca.page_table[(size_t)slot * ca.pages_per_slot + kb]) * KV_PAGE;
          else
            row = (slot * G + g) * ca.capacity + kb * TA_BN;
        }
        {
          const int s = it % TA_KSTAGES;
          if (!mbar_wait(smem_u32(&k_empty[s]), ((it / TA_KSTAGES) & 1) ^ 1u, abort_p)) break;
          const uint32_t bar = smem_u32(&k_full[s]);
          mbar_expect_tx(bar, KV_BYTES);
#pragma unroll
          for (int sub = 0; sub < SUB; ++sub)
            ta_tma_load_2d(k_s + s * KV_BYTES + sub * (TA_BN * 128), &map_k, col_k + sub * 64,
                           row, bar);
        }
        {
          const int s = it % TA_VSTAGES;
          if (!mbar_wait(smem_u32(&v_empty[s]), ((it / TA_VSTAGES) & 1) ^ 1u, abort_p)) break;
          const uint32_t bar = smem_u32(&v_full[s]);
          mbar_expect_tx(bar, KV_BYTES);
#pragma unroll
          for (int sub = 0; sub < SUB; ++sub)
            ta_tma_load_2d(v_s + s * KV_BYTES + sub * (TA_BN * 128), &map_v, col_v + sub * 64,
                           row, bar);
        }
      }
    }
  } else if (warp == 1 || warp == TA_MMA_B) {
    // ---------------- MMA issuers, one per tile: the whole warp runs the loop, lane 0 issues
    {
      const int x = warp == 1 ? 0 : 1;
      const uint32_t leader = lane == 0 ? 1u : 0u;
      // S: M = 128 queries, N = 64 keys, both operands K-major
      const uint32_t idesc_s = (1u << 4) | (FMT << 7) | (FMT << 10) | ((uint32_t)(TA_BN >> 3) << 17) |
                               ((uint32_t)(TA_BM >> 4) << 24);
      // O += P.V: M = 128 queries, N = HD, A (P) K-major, B (V) MN-major
      const uint32_t idesc_pv = (1u << 4) | (FMT << 7) | (FMT << 10) | (1u << 16) |
                                ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TA_BM >> 4) << 24);
      // descriptors: one per operand tile, advanced by constants inside the loops
      // this issuer's tile: its queries, its columns of tensor memory, its barriers
      const uint64_t q_desc = ta_desc_k(q_s + x * Q_BYTES);
      const uint32_t my_s = x ? tmem_s[1] : tmem_s[0], my_o = x ? tmem_o[1] : tmem_o[0];
      const int my_kb0 = x ? t_kb0[1] : t_kb0[0], my_kb1 = x ? t_kb1[1] : t_kb1[0];
      const uint32_t bar_s = smem_u32(x ? &s_full[1][0] : &s_full[0][0]);   // [1] is 8 bytes on
      const uint32_t bar_p = smem_u32(x ? &p_ready[1][0] : &p_ready[0][0]);
      const uint32_t bar_pv = smem_u32(x ? &pv_done[1][0] : &pv_done[0][0]);
      auto mine = [&](int kb) { return kb >= my_kb0 && kb < my_kb1; };
      auto issue_s = [&](int stage, int buf) {                // buf: the block's parity for this tile
        const uint64_t k_desc = ta_desc_k(k_s + stage * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          ta_umma_by(leader, my_s + buf * TA_BN,
                     q_desc + (uint64_t)(((ks / 4) * (TA_BM * 128) + (ks % 4) * 32) >> 4),
                     k_desc + (uint64_t)(((ks / 4) * (TA_BN * 128) + (ks % 4) * 32) >> 4), idesc_s,
                     ks > 0 ? 1u : 0u);
        ta_commit_by(leader, bar_s + 8 * buf);
      };
      auto issue_pv = [&](int stage, int blk) {               // blk: the tile's own count of blocks
        const uint64_t v_desc = ta_desc_mn(v_s + stage * KV_BYTES, TA_BN * 128);
#pragma unroll
        for (int kk = 0; kk < TA_BN / 16; ++kk)
          ta_umma_tmem_a_by(leader, my_o, my_s + (blk & 1) * TA_BN + kk * 8,
                            v_desc + (uint64_t)((kk * 16 * 128) >> 4), idesc_pv,
                            (blk == 0 && kk == 0) ? 0u : 1u);
        ta_commit_by(leader, bar_pv + 8 * (blk & 1));
      };
      // S runs two blocks of keys ahead of the softmax: each tile has two S buffers, and
      // a buffer is free again once the row threads have signalled the block that used it.
      // A stage of K or V is free once both issuers have committed it (also the one whose
      // tile does not see that block: its commit has nothing to wait for).
      bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&q_full), 0, abort_p));
      for (int pre = 0; pre < 2 && pre < n_it && ok; ++pre) {
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&k_full[pre]), 0, abort_p));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (mine(kb_lo + pre)) issue_s(pre, (kb_lo + pre - my_kb0) & 1);
        ta_commit_by(leader, smem_u32(&k_empty[pre]));
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int kb = kb_lo + it;
        const int sv = it % TA_VSTAGES, sk = (it + 2) % TA_KSTAGES;
        const bool more = it + 2 < n_it;
        // (an issuer whose tile does not see a block still waits for the block's stage before
        // it commits it: one arrival per issuer and filling, or the producer would run ahead)
        const bool pv = mine(kb);
        if (pv) {
          // P of this block is in tensor memory, S has been read, O is rescaled
          const int blk = kb - my_kb0;
          ok = __all_sync(0xffffffffu, mbar_wait(bar_p + 8 * (blk & 1), (uint32_t)(blk >> 1) & 1u, abort_p));
          if (!ok) break;
        }
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&v_full[sv]), (it / TA_VSTAGES) & 1, abort_p));
        if (!ok) break;
        if (pv) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_pv(sv, kb - my_kb0);
        }
        if (more) {
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&k_full[sk]), ((it + 2) / TA_KSTAGES) & 1, abort_p));
          if (!ok) break;
          if (mine(kb + 2)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_s(sk, (kb + 2 - my_kb0) & 1);
          }
        }
        ta_commit_by(leader, smem_u32(&v_empty[sv]));         // V of this block is consumed
        if (more) ta_commit_by(leader, smem_u32(&k_empty[sk]));   // and K of the block after next
      }
    }
  } else {
    // ---------------- softmax: one query row per thread; warps 2-5 tile A, 6-9 tile B
    const int x = warp >= 6 ? 1 : 0;
    const int quarter = warp & 3;                             // the TMEM lanes this warp may touch
    const int row = quarter * 32 + lane;
    const int my_m0 = x ? t_m0[1] : t_m0[0], my_rows = x ? t_rows[1] : t_rows[0];
    const int my_kb0 = x ? t_kb0[1] : t_kb0[0], my_kb1 = x ? t_kb1[1] : t_kb1[0];
    const int p = past + my_m0 + row;                         // this row's position
    const int p_hi = past + my_m0 + TA_BM - 1;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t my_s = (x ? tmem_s[1] : tmem_s[0]) + lane_addr;
    const uint32_t my_o = (x ? tmem_o[1] : tmem_o[0]) + lane_addr;
    const uint32_t bar_s = smem_u32(x ? &s_full[1][0] : &s_full[0][0]);   // [1] is 8 bytes on
    const uint32_t bar_p = smem_u32(x ? &p_ready[1][0] : &p_ready[0][0]);   // likewise
    const uint32_t bar_pv = smem_u32(x ? &pv_done[1][0] : &pv_done[0][0]);
    float m_ref = -INFINITY, l_run = 0.f;
    pdl_wait();
    bool ok = true;
    const int n_x = my_kb1 - my_kb0;
    for (int it = 0; it < n_x; ++it) {
      const int j0 = (my_kb0 + it) * TA_BN;
      // every wait is decided per warp (the loads from tensor memory below are warp-wide)
      ok = __all_sync(0xffffffffu, mbar_wait(bar_s + 8 * (it & 1), (it >> 1) & 1, abort_p));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float s[TA_BN];
      {
        uint32_t raw[TA_BN];
        const uint32_t s_addr = my_s + (it & 1) * TA_BN;
        ta_ld32_issue(s_addr, raw);                           // both halves in flight, one wait
        ta_ld32_issue(s_addr + 32, raw + 32);
        ta_ld_wait32(raw);
        ta_ld_after32(raw + 32);
#pragma unroll
        for (int i = 0; i < TA_BN; ++i) s[i] = __uint_as_float(raw[i]);
      }
      // every row of the tile sees every key of the block?
      const bool inside = j0 + TA_BN - 1 <= past + my_m0 && (window <= 0 || j0 > p_hi - window);
      if (!inside) {
#pragma unroll
        for (int i = 0; i < TA_BN; ++i) {
          const int key = j0 + i;
          const bool vis = key <= p && (window <= 0 || key > p - window);
          s[i] = vis ? s[i] : -INFINITY;
        }
      }
      float mx[4] = {s[0], s[1], s[2], s[3]};                 // four chains instead of one
#pragma unroll
      for (int i = 4; i < TA_BN; ++i) mx[i & 3] = fmaxf(mx[i & 3], s[i]);
      const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
      const bool raise = m_blk > m_ref + TA_RAISE;            // always true for the first live block
      const float m_new = raise ? m_blk : m_ref;
      const float corr = raise ? ta_ex2(m_ref - m_new) : 1.f;
      const bool any_raise = __any_sync(0xffffffffu, raise);
      if (it > 0 && any_raise) {                              // uniform over the warp; rare
        // O is rescaled once the previous block's product has been added to it
        ok = __all_sync(0xffffffffu, mbar_wait(bar_pv + 8 * ((it - 1) & 1), ((it - 1) >> 1) & 1, abort_p));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          float v[32];
          ta_ld32(my_o + c, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= corr;
          ta_st32(my_o + c, v);
        }
      }
      m_ref = m_new;
      const float neg = m_ref > -INFINITY ? -m_ref : 0.f;
      float2 ls[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 scale2 = make_float2(scale_log2, scale_log2), neg2 = make_float2(neg, neg);
      float pk[TA_BN / 2];                                    // P, two keys per 32-bit column
#pragma unroll
      for (int j = 0; j < TA_BN / 2; ++j) {                   // pairs of keys, in packed arithmetic
        const float2 x = __ffma2_rn(make_float2(s[2 * j], s[2 * j + 1]), scale2, neg2);
        const float2 e = make_float2(ta_ex2(x.x), ta_ex2(x.y));
        ls[j & 1] = __fadd2_rn(ls[j & 1], e);
        pk[j] = __uint_as_float(pack2<T16>(e.x, e.y));
      }
      // P takes the place of the first half of the S columns it came from: the product
      // reads it from tensor memory, and S of the block after next overwrites it only
      // after that product (the tensor core runs its instructions in order)
      ta_st32(my_s + (it & 1) * TA_BN, pk);
      l_run = l_run * corr + ((ls[0].x + ls[0].y) + (ls[1].x + ls[1].y));
      // P is complete for this row, S has been read, O is rescaled: the MMA thread may go on
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(bar_p + 8 * (it & 1));
    }
    if (ok && n_x > 0)
      ok = __all_sync(0xffffffffu, mbar_wait(bar_pv + 8 * ((n_x - 1) & 1), ((n_x - 1) >> 1) & 1, abort_p));
    if (ok && n_x > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = 1.0f / l_run;
      T16* op = out + ((size_t)(qs + my_m0 + row) * H + h) * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        float v[32];
        ta_ld32(my_o + c, v);                // by the whole warp
        if (row < my_rows) {
#pragma unroll
          for (int c8 = 0; c8 < 32; c8 += 8) {
            uint4 u;
            u.x = pack2<T16>(v[c8 + 0] * inv, v[c8 + 1] * inv);
            u.y = pack2<T16>(v[c8 + 2] * inv, v[c8 + 3] * inv);
            u.z = pack2<T16>(v[c8 + 4] * inv, v[c8 + 5] * inv);
            u.w = pack2<T16>(v[c8 + 6] * inv, v[c8 + 7] * inv);
            *reinterpret_cast<uint4*>(op + c + c8) = u;
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) atomicOr(status, ERR_WAIT_TIMEOUT);
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

typedef CUresult (*TaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                               const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TaEncodeFn ta_encode_fn() {
  static TaEncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TaEncodeFn>(p);
  }
  return fn;
}
// rows x cols of a 16-bit type, row-major; box = box_rows rows x 64 columns, 128-byte swizzle
static int ta_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols,
                       int box_rows, bool half) {
  TaEncodeFn fn = ta_encode_fn();
  if (!fn) return -10;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

template <int HD, typename T16>
static int launch_prefill_tc(const void* q, const void* k_rows, const void* v_rows, long long kv_n_rows,
                             long long kv_cols, const ta_cache_args& ca, const int* q_start, void* out,
                             int n_tokens, int n_seqs, int max_q_len, int H, int G, int window,
                             int* status, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  constexpr bool half = std::is_same<T16, __half>::value;
  int rc = ta_make_map(&mq, q, n_tokens, (long long)H * HD, TA_BM, half);
  if (rc) return rc;
  rc = ta_make_map(&mk, k_rows, kv_n_rows, kv_cols, TA_BN, half);
  if (rc) return rc;
  rc = ta_make_map(&mv, v_rows, kv_n_rows, kv_cols, TA_BN, half);
  if (rc) return rc;
  // two query tiles, the K and V rings, slack to align to 1024
  const size_t smem = (size_t)2 * TA_BM * HD * 2 + (size_t)(TA_KSTAGES + TA_VSTAGES) * TA_BN * HD * 2 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, T16>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const dim3 grid(H, n_seqs, (max_q_len + 2 * TA_BM - 1) / (2 * TA_BM));
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
  launch_pdl(attn_prefill_tc_kernel<HD, T16>, grid, dim3(TA_THREADS), smem, stream, mq, mk, mv, ca, q_start,
             (T16*)out, H, G, window, scale_log2, status);
  YALM_LAUNCH_CHECK();
  return 0;
}

static int ta_dispatch(const void* q, const void* k_rows, const void* v_rows, long long kv_n_rows,
                       long long kv_cols, const ta_cache_args& ca, const int* q_start, void* out, int dtype,
                       int n_tokens, int n_seqs, int max_q_len, int H, int G, int hd, int window,
                       int* status, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0 || n_tokens <= 0) return 0;
  if (dtype != DT_BF16 && dtype != DT_F16) return -3;
  if (hd != 64 && hd != 128) return -2;
  if (G <= 0 || H % G != 0) return -3;
  if (n_seqs > 65535 || (max_q_len + 2 * TA_BM - 1) / (2 * TA_BM) > 65535) return -4;
  if (((uintptr_t)q | (uintptr_t)k_rows | (uintptr_t)v_rows | (uintptr_t)out) & 15) return -6;
#define YALM_TA(HD, T) \
  return launch_prefill_tc<HD, T>(q, k_rows, v_rows, kv_n_rows, kv_cols, ca, q_start, out, n_tokens, \
                                  n_seqs, max_q_len, H, G, window, status, stream)
  if (dtype == DT_F16) {
    if (hd == 64) YALM_TA(64, __half);
    YALM_TA(128, __half);
  }
  if (hd == 64) YALM_TA(64, __nv_bfloat16);
  YALM_TA(128, __nv_bfloat16);
#undef YALM_TA
}

}  // namespace yalm

using namespace yalm;

// Prefill attention on tcgen05 for sequences that start at their first token (every
// key is in kv_step).  q [n_tokens, H*hd], kv_step [n_tokens, 2, G, hd], out like q;
// bfloat16 or float16 (dtype code); hd 64 or 128.  q_start [n_seqs + 1] must be in place
// before the launch (it is read before the wait on the previous kernel).
extern "C" int yalm_attention_prefill_tc(const void* q, const void* kv_step, const int* q_start,
                                         void* out, int dtype, int n_tokens, int n_seqs,
                                         int max_q_len, int H, int G, int hd, int window,
                                         int* status, cudaStream_t stream) {
  const ta_cache_args ca = {nullptr, nullptr, nullptr, 0, 0, 0, 0};
  return ta_dispatch(q, kv_step, kv_step, n_tokens, (long long)2 * G * hd, ca, q_start, out, dtype, n_tokens,
                     n_seqs, max_q_len, H, G, hd, window, status, stream);
}

// The same for sequences that go on from the positions in slot_pos (prompts cut into steps):
// every key, this step's included, is read from the cache, which the step has written
// before this launch.  k_cache / v_cache: the layer's [slots, G, capacity, hd], or with a
// page table [G, n_pages, 64, hd] and page_table [slots, pages_per_slot].  No sequence may
// wrap around its ring in this step (slot_pos + its tokens <= capacity): the caller checks.
// seq_slot, slot_pos and the page table are read before the wait on the previous kernel.
extern "C" int yalm_attention_prefill_tc_cache(const void* q, const void* k_cache, const void* v_cache,
                                               const int* q_start, const int* seq_slot,
                                               const int* slot_pos, void* out, int dtype, int n_tokens,
                                               int n_seqs, int max_q_len, int n_slots, int H, int G,
                                               int hd, int capacity, int window, const int* page_table,
                                               int pages_per_slot, int n_pages, int* status,
                                               cudaStream_t stream) {
  if (capacity <= 0 || n_slots <= 0 || (page_table != nullptr && (pages_per_slot <= 0 || n_pages <= 0)))
    return -4;
  const ta_cache_args ca = {seq_slot, slot_pos, page_table, pages_per_slot, n_pages, capacity, 1};
  const long long rows = page_table != nullptr ? (long long)G * n_pages * KV_PAGE
                                               : (long long)n_slots * G * capacity;
  if (rows > 0x7fffffffLL) return -4;
  return ta_dispatch(q, k_cache, v_cache, rows, hd, ca, q_start, out, dtype, n_tokens, n_seqs, max_q_len,
                     H, G, hd, window, status, stream);
}
