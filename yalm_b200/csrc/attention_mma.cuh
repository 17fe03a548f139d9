// Tensor-core attention for bfloat16 and float16: prefill (many query tokens per
// sequence) and decode (one query token per sequence).
//
// Same mathematics as attention.cu (and as the reference's attn_dot /
// attn_softmax / att_mix, infer.cu:339-523): scores (q.k)/sqrt(hd) over the
// visible keys, max-subtracted softmax in 32-bit, weighted sum of values.  Here
// Q.K^T and P.V run as m16n8k16 16-bit tiles with 32-bit accumulators
// (mma.sync); keys and values are brought into shared memory with cp.async in a
// 16-byte-chunk XOR swizzle so that ldmatrix is free of bank conflicts; the
// softmax is the online form (running max and sum per row), so no score matrix
// ever leaves registers.
//
// Where a key lives: position j of a sequence is in this step's own buffer
// (kv_step [N, 2, G, hd]) when j >= past, else in the cache ring at row
// j % capacity -- the same rule as attention.cu.
#pragma once
#include <cuda_bf16.h>

#include <type_traits>

#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int FA_WARPS = 4;
constexpr int FA_THREADS = FA_WARPS * 32;        // decode blocks and the tile loaders' default
constexpr int FP_WARPS = 8;
constexpr int FP_THREADS = FP_WARPS * 32;        // prefill blocks
constexpr int FA_BM = FP_WARPS * 16;             // query rows per prefill block (16 per warp)
constexpr int FA_BN = 64;                        // keys per block iteration

template <typename T16>
__device__ __forceinline__ void mma_16(float* c, const uint32_t* a, const uint32_t* b) {
  if constexpr (std::is_same<T16, __half>::value) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
}
__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// 16-byte asynchronous copy; with pred false the destination is zero-filled
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n)
               : "memory");
}
// The same under a predicate of the instruction itself (never a branch around it): `live`
// false zero-fills, `issue` false leaves the 16 bytes alone.
__device__ __forceinline__ void cp_async16_if(uint32_t dst, const void* src, bool live, bool issue) {
  const int n = live ? 16 : 0;
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %3, 0;\n\t"
               "@p cp.async.cg.shared.global [%0], [%1], 16, %2;\n\t}" ::"r"(dst), "l"(src), "r"(n),
               "r"((int)issue)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A tile of rows x HDP 16-bit elements in shared memory; HDP is a multiple of 64, so a
// row is a multiple of 128 bytes and the 16-byte chunk index can be XORed with
// (row & 7) without leaving the row.
template <int HDP>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
  return base + (uint32_t)(row * (HDP * 2) + ((chunk ^ (row & 7)) << 4));
}

// Loads `rows` rows of hd elements each into a swizzled tile.  row_ptr(r) gives the
// global address of row r, or nullptr for a row that is to be zero.
template <int HDP, int NT = FA_THREADS, typename T16, typename RowPtr>
__device__ __forceinline__ void load_tile(uint32_t base, int rows, int hd,
                                          const T16* valid_ptr, RowPtr row_ptr) {
  const int cpr = hd >> 3;                                    // 16-byte chunks per row
  for (int idx = threadIdx.x; idx < rows * cpr; idx += NT) {
    const int r = idx / cpr, ch = idx - r * cpr;
    const T16* p = row_ptr(r);
    // a zero-filled chunk still names an address: give it one that exists
    cp_async16(tile_addr<HDP>(base, r, ch), p ? p + ch * 8 : valid_ptr, p != nullptr);
  }
}

// Loads `n` rows that lie `stride` elements apart in global memory (rows of this
// step's own buffers) and zero-fills rows n..rows-1; one 16-byte column per thread.
template <int HDP, int NT, typename T16>
__device__ __forceinline__ void load_strided_tile(uint32_t base, int rows, int n, int hd,
                                                  const T16* first, size_t stride) {
  const int cpr = hd >> 3;
  const int rstep = NT / cpr;
  if ((int)threadIdx.x >= rstep * cpr) return;
  const int ch = threadIdx.x % cpr;
  for (int r = threadIdx.x / cpr; r < rows; r += rstep)
    cp_async16(tile_addr<HDP>(base, r, ch), r < n ? first + (size_t)r * stride + ch * 8 : first,
               r < n);
}

// ----------------------------------------------------------------- prefill
// grid (query tiles of a sequence, heads, sequences); a block takes 64 query
// tokens of one head.  scale_log2 = log2(e) / sqrt(hd).
template <int HDP, typename T16>
__global__ void __launch_bounds__(FP_THREADS, 2)
attn_prefill_mma_kernel(const T16* __restrict__ q, const T16* __restrict__ kv_step,
                        const T16* __restrict__ k_cache,
                        const T16* __restrict__ v_cache, const int* __restrict__ q_start,
                        const int* __restrict__ seq_slot, const int* __restrict__ slot_pos,
                        T16* __restrict__ out, int H, int G, int hd, int capacity,
                        int window, float scale_log2, const int* __restrict__ page_table,
                        int pps, int n_pages) {
  constexpr int NKS = HDP / 16, NOT = HDP / 8;
  extern __shared__ __align__(128) uint8_t fa_smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.z, h = blockIdx.y;
  const int g = h / (H / G);
  const int qs = q_start[b], q_len = q_start[b + 1] - qs;
  // the tiles with the most keys (the last tokens) are scheduled first
  const int m0 = (gridDim.x - 1 - blockIdx.x) * FA_BM;
  if (m0 >= q_len) return;
  const int slot = seq_slot[b];
  const int past = slot_pos[slot];
  const int rows = min(FA_BM, q_len - m0);
  const int nks = hd >> 4, n_ot = hd >> 3;

  const uint32_t q_s = smem_u32(fa_smem);
  const uint32_t k_s0 = q_s + FA_BM * HDP * 2;
  const uint32_t v_s0 = k_s0 + 2 * FA_BN * HDP * 2;           // two K stages, then two V stages
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;

  // the visible key range of the whole tile: [k_begin, k_end)
  const int p_first = past + m0, p_last = past + m0 + rows - 1;
  const int k_end = p_last + 1;
  const int k_begin = window > 0 ? max(0, p_first - window + 1) : 0;
  const int kb0 = k_begin / FA_BN, kb1 = (k_end + FA_BN - 1) / FA_BN;

  const size_t step_row = (size_t)2 * G * hd;
  auto load_kv = [&](int kb, int stage) {
    const int j0 = kb * FA_BN;
    const uint32_t kd = k_s0 + stage * FA_BN * HDP * 2, vd = v_s0 + stage * FA_BN * HDP * 2;
    if (j0 >= past) {
      // the whole block comes from this step's keys and values: rows a fixed stride apart
      const int n = min(FA_BN, k_end - j0);
      const T16* k0 = kv_step + (size_t)(qs + j0 - past) * step_row + (size_t)g * hd;
      load_strided_tile<HDP, FP_THREADS>(kd, FA_BN, n, hd, k0, step_row);
      load_strided_tile<HDP, FP_THREADS>(vd, FA_BN, n, hd, k0 + (size_t)G * hd, step_row);
      return;
    }
    load_tile<HDP, FP_THREADS>(kd, FA_BN, hd, q, [&](int r) -> const T16* {
      const int j = j0 + r;
      if (j >= k_end) return nullptr;
      return j >= past ? kv_step + (size_t)(qs + j - past) * step_row + (size_t)g * hd
                       : k_cache + kv_row_offset(page_table, pps, n_pages, slot, g, G, capacity, j % capacity, hd);
    });
    load_tile<HDP, FP_THREADS>(vd, FA_BN, hd, q, [&](int r) -> const T16* {
      const int j = j0 + r;
      if (j >= k_end) return nullptr;
      return j >= past ? kv_step + (size_t)(qs + j - past) * step_row + (size_t)(G + g) * hd
                       : v_cache + kv_row_offset(page_table, pps, n_pages, slot, g, G, capacity, j % capacity, hd);
    });
  };

  load_strided_tile<HDP, FP_THREADS>(q_s, FA_BM, rows, hd, q + ((size_t)(qs + m0) * H + h) * hd,
                                     (size_t)H * hd);
  load_kv(kb0, 0);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  float o[NOT][4];
#pragma unroll
  for (int i = 0; i < NOT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int p_row[2] = {past + m0 + warp * 16 + gid, past + m0 + warp * 16 + gid + 8};
  const int w_first = past + m0 + warp * 16, w_last = w_first + 15;
  const int q_row = warp * 16 + (lane & 15);

  for (int kb = kb0; kb < kb1; ++kb) {
    const int stage = (kb - kb0) & 1;
    if (kb + 1 < kb1) load_kv(kb + 1, stage ^ 1);             // prefetch the next block
    cp_async_commit();
    const uint32_t k_s = k_s0 + stage * FA_BN * HDP * 2, v_s = v_s0 + stage * FA_BN * HDP * 2;

    // the block's 64 keys in two halves of 32: scores, softmax and P.V per half keep
    // the register count low enough for two blocks per SM
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int j_base = kb * FA_BN + half * 32;
      if (j_base > w_last) break;                             // wholly in this warp's future
      float s[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
      for (int ks = 0; ks < NKS; ++ks) {
        if (ks < nks) {
          uint32_t qf[4];
          ldsm_x4(qf, tile_addr<HDP>(q_s, q_row, ks * 2 + (lane >> 4)));
#pragma unroll
          for (int np = 0; np < 2; ++np) {                    // two n-tiles per ldmatrix.x4
            uint32_t kf[4];
            const int row = half * 32 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
            ldsm_x4(kf, tile_addr<HDP>(k_s, row, ks * 2 + ((lane >> 3) & 1)));
            mma_16<T16>(s[2 * np], qf, kf);
            mma_16<T16>(s[2 * np + 1], qf, kf + 2);
          }
        }
      }
      // mask and online softmax (rows gid and gid + 8 of this warp)
      float m_new[2] = {m_run[0], m_run[1]};
      const bool inside = j_base + 31 <= w_first && (window <= 0 || j_base > w_last - window);
      if (inside) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            s[i][j] *= scale_log2;
            m_new[j >> 1] = fmaxf(m_new[j >> 1], s[i][j]);
          }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int key = j_base + i * 8 + tig * 2 + (j & 1);
            const int pr = p_row[j >> 1];
            const bool vis = key <= pr && (window <= 0 || key > pr - window);
            s[i][j] = vis ? s[i][j] * scale_log2 : -INFINITY;
            m_new[j >> 1] = fmaxf(m_new[j >> 1], s[i][j]);
          }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
        m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
      }
      float corr[2], l_add[2] = {0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 2; ++r)
        corr[r] = m_new[r] > -INFINITY ? exp2f(m_run[r] - m_new[r]) : 1.f;
      uint32_t pf[2][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float mr = m_new[j >> 1];
          p[j] = mr > -INFINITY ? exp2f(s[i][j] - mr) : 0.f;
          l_add[j >> 1] += p[j];
        }
        pf[i >> 1][(i & 1) * 2 + 0] = pack2<T16>(p[0], p[1]);
        pf[i >> 1][(i & 1) * 2 + 1] = pack2<T16>(p[2], p[3]);
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l_run[r] = l_run[r] * corr[r] + l_add[r];
        m_run[r] = m_new[r];
      }
#pragma unroll
      for (int i = 0; i < NOT; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
      // O += P V: k-steps of 16 keys, n-tiles of 8 head elements (two per ldmatrix.x4.trans)
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
        for (int np = 0; np < NOT / 2; ++np) {
          if (np * 2 < n_ot) {
            uint32_t vf[4];
            const int row = half * 32 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            ldsm_x4_t(vf, tile_addr<HDP>(v_s, row, np * 2 + (lane >> 4)));
            mma_16<T16>(o[2 * np], pf[kk], vf);
            mma_16<T16>(o[2 * np + 1], pf[kk], vf + 2);
          }
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();
  }

  // rows' sums live spread over the four lanes of a quad
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + gid + r * 8;
    if (row < rows) {
      const float inv = 1.0f / l_run[r];
      T16* op = out + ((size_t)(qs + m0 + row) * H + h) * hd;
#pragma unroll
      for (int i = 0; i < NOT; ++i) {
        if (i < n_ot) {
          *reinterpret_cast<uint32_t*>(op + i * 8 + tig * 2) =
              pack2<T16>(o[i][r * 2] * inv, o[i][r * 2 + 1] * inv);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ decode
// One query token per sequence; every key in the cache.  The product is taken
// transposed: S^T = K.Q^T and O^T = V^T.P^T, so the 16 rows of an MMA tile are keys
// (or features of the head) and the 8 columns are the query heads that share the kv
// head -- with grouped queries nothing of a tile is padding, and the running
// output is 32 registers instead of 64.  A block takes a run of `cpc` consecutive
// chunks of 64 positions of one (sequence, kv head, group of up to 16 heads).
// Inside the block each warp walks through its own units of 32 keys (unit u of the
// run goes to warp u % 4) with a ring of cp.async stages of its own: no barrier
// of the block inside the loop.  The warps' partial results are merged through
// shared memory at the end; with few sequences cpc is small, many blocks work on
// one sequence and the block that finishes last merges their parts (as in
// attn_decode_kernel); with many sequences a block takes a whole sequence.
// Maxima are kept in the log2 domain (scores times log2(e)/sqrt(hd)).
constexpr int FD_CHUNK = 64;       // the unit of the host's plan
#ifndef YALM_FD_UNIT
#define YALM_FD_UNIT 32
#endif
constexpr int FD_UNIT = YALM_FD_UNIT;   // keys a warp takes at a time (16 or 32)
constexpr int FD_MT = FD_UNIT / 16;
constexpr int FD_ROWS = 16;        // query heads per block
constexpr int FD_STAGES = 3;       // units in flight or in use per warp
constexpr int FD_OPAD = 20;        // row length of the merge buffer [warp][feature][head]
constexpr int FD_WARPS_MAX = 4;    // warps of a block (4, or 2 with two blocks to an SM): each has a ring of its own

__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

__device__ __forceinline__ float ex2_approx(float x) {       // 2^x; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One warp loads the first `n` of FD_UNIT positions into a swizzled tile of FD_UNIT rows and
// zero-fills rows n and up.  Lane l takes rows (l & 7) + 8 rb and the 16-byte columns
// (l >> 3) + 4 j: its row's swizzle is then one constant, and a copy needs an add and an
// exclusive-or.  (A warp is alone on its scheduler here, so every instruction of the address
// arithmetic is paid in full.)
//
// warp_load_run: the unit's rows follow one another in memory from `first` on.
template <int HDP, typename T16>
__device__ __forceinline__ void warp_load_run(uint32_t base, int n, int hd, const T16* first,
                                              int lane) {
  const int r7 = lane & 7, cg = lane >> 3;
  const int cpr = hd >> 3;
  const uint32_t s_lane = base + r7 * (HDP * 2) + ((cg ^ (r7 & 3)) << 4);
  const uint32_t x_lane = (uint32_t)(r7 >> 2) << 6;
  const T16* g = first + (size_t)r7 * hd + cg * 8;
#pragma unroll
  for (int rb = 0; rb < FD_UNIT / 8; ++rb) {
    const bool live = rb * 8 + r7 < n;
#pragma unroll
    for (int j = 0; j < HDP / 32; ++j)
      cp_async16_if(s_lane + rb * 8 * HDP * 2 + ((uint32_t)(j << 6) ^ x_lane), g + j * 32, live,
                    cg + 4 * j < cpr);
    g += (size_t)8 * hd;
  }
}

// warp_load_rows: a unit that wraps around the ring's end or crosses a page; every row is
// looked up (rows first_row, first_row + 1, ... modulo capacity of the kv head's rows at
// `head`; through the sequence's row of the page table if there is one).  Rare, and kept
// out of line so that it does not shape the code around the common path.
template <int HDP, typename T16>
__device__ __noinline__ void warp_load_rows(uint32_t base, int n, int hd, const T16* head,
                                            const int* __restrict__ pages, int first_row,
                                            int capacity, int lane) {
  const int r7 = lane & 7, cg = lane >> 3;
  const int cpr = hd >> 3;
  const uint32_t s_lane = base + r7 * (HDP * 2) + ((cg ^ (r7 & 3)) << 4);
  const uint32_t x_lane = (uint32_t)(r7 >> 2) << 6;
#pragma unroll 1
  for (int rb = 0; rb < FD_UNIT / 8; ++rb) {
    const int r = rb * 8 + r7;
    int row = (first_row + r) % capacity;
    if (pages != nullptr) row = pages[row / KV_PAGE] * KV_PAGE + (row % KV_PAGE);
    const T16* g = head + (size_t)row * hd + cg * 8;
#pragma unroll
    for (int j = 0; j < HDP / 32; ++j)
      if (cg + 4 * j < cpr)
        cp_async16(s_lane + rb * 8 * HDP * 2 + ((uint32_t)(j << 6) ^ x_lane), g + j * 32, r < n);
  }
}

// The fused form's inputs: the q/k/v product of this step as n_partials 32-bit slices
// [slice][token][(H + 2 G) hd] (partial_stride elements apart) and the step's cosines and
// sines [token][hd / 2].  The kernel then does what rope_store_kernel would have done for its
// own heads: it sums the slices (in the same order), rotates q and the new k, rounds to the
// 16-bit type, keeps q in its shared-memory tile and writes the new k and v into the cache row
// (and into the staged unit, where that is already on the chip).  One kernel and one
// hand-over less per layer; bit for bit the two-kernel result.
struct fd_fused_args {
  const float* qkv;
  const float2* cos_sin;
  long long partial_stride;
  int n_partials;
};

template <int HDP, int NT, typename T16, bool PAGED, bool FUSED, int NW>
__global__ void __launch_bounds__(NW * 32, FD_WARPS_MAX / NW)
attn_decode_mma_kernel(const T16* __restrict__ q, const T16* __restrict__ k_cache,
                       const T16* __restrict__ v_cache, const int* __restrict__ seq_slot,
                       const int* __restrict__ slot_pos, T16* __restrict__ out,
                       float* __restrict__ part_o, float* __restrict__ part_ml,
                       int* __restrict__ counters, int* __restrict__ status, int H, int G, int hd,
                       int capacity, int window, int cpc, int max_parts, float scale_log2,
                       const int* __restrict__ page_table, int pps, int n_pages,
                       const fd_fused_args fz) {
  constexpr int NKS = HDP / 16;                              // 16-wide steps over the head size
  constexpr int TILE = FD_UNIT * HDP * 2;                    // K (or V) of one unit, bytes
  constexpr int WARP_RING = FD_STAGES * 2 * TILE;
  constexpr uint32_t FULL = 0xffffffffu;
  constexpr int FD_THREADS = NW * 32;
  extern __shared__ __align__(128) uint8_t fa_smem[];
  __shared__ float wm_s[NW][FD_ROWS];                  // per warp: row max, row sum
  __shared__ float wl_s[NW][FD_ROWS];
  __shared__ float row_m[FD_ROWS], row_l[FD_ROWS];
  __shared__ int last_flag;
  pdl_launch_dependents();
  const int R = H / G;
  const int nhc = (R + FD_ROWS - 1) / FD_ROWS;
  const int g = blockIdx.y / nhc, hchunk = blockIdx.y % nhc;
  const int h0 = g * R + hchunk * FD_ROWS;
  const int nh = min(FD_ROWS, R - hchunk * FD_ROWS);
  const int t = blockIdx.z, part = blockIdx.x;
  const int slot = seq_slot[t];           // written by a host copy, never by a kernel: safe early
  // Positions are written by the advance kernel alone, and that kernel lets nothing start
  // before it has ended: they too may be read while the previous kernel still runs.
  const int pos = slot_pos[slot];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int nkeys = pos - lo + 1;
  const int n_chunks = (nkeys + FD_CHUNK - 1) / FD_CHUNK;
  const int n_parts = (n_chunks + cpc - 1) / cpc;
  if (n_parts > max_parts && part == 0 && threadIdx.x == 0) atomicOr(status, ERR_CONTEXT_RANGE);
  if (part >= n_parts) return;
  constexpr int UPC = FD_CHUNK / FD_UNIT;
  const int u0 = part * cpc * UPC;
  const int u1 = min((nkeys + FD_UNIT - 1) / FD_UNIT, u0 + cpc * UPC);
  const int nks = hd >> 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const uint32_t q_s = smem_u32(fa_smem);                    // [16 heads][HDP]
  const uint32_t ring_s = q_s + FD_ROWS * HDP * 2 + warp * WARP_RING;
  // A head size below HDP: the tiles' columns from hd on are zeroed once (no copy ever writes
  // them), and the products below run over all HDP columns without a test per step.
  if (hd < HDP) {
    constexpr int WORDS = (FD_ROWS * HDP * 2 + NW * WARP_RING) / 16;
    for (int i = threadIdx.x; i < WORDS; i += FD_THREADS)
      reinterpret_cast<uint4*>(fa_smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
  }
  if (FUSED) {
    // the query tile's rows beyond this block's heads stay zero (the copies of the unfused
    // form zero-fill them); the rows of its heads are written after the dependency wait
    for (int i = threadIdx.x; i < FD_ROWS * HDP * 2 / 16; i += FD_THREADS)
      reinterpret_cast<uint4*>(fa_smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  // The page table is written by host copies before the step's first kernel, like the
  // batch's index arrays: it may be read before the dependency wait too.
  const int* my_pages = PAGED ? page_table + (size_t)slot * pps : nullptr;
  const size_t head_off = PAGED ? (size_t)g * n_pages * KV_PAGE * hd
                                : ((size_t)slot * G + g) * capacity * hd;
  const T16* kc = k_cache + head_off;
  const T16* vc = v_cache + head_off;
  // A unit's place in the ring is carried from unit to unit (no division in the loop), and
  // the page that holds its first row is asked for one unit ahead of its use.
  const int ring_step = (NW * FD_UNIT) % capacity;
  auto page_of = [&](int u, int row) { return (PAGED && u < u1) ? my_pages[row / KV_PAGE] : 0; };
  auto load_unit = [&](int u, int stage, int first, int page) {
    const int n = min(FD_UNIT, pos + 1 - (lo + u * FD_UNIT));
    const uint32_t dst = ring_s + stage * 2 * TILE;
    const int in_page = first & (KV_PAGE - 1);
    const bool run = first + FD_UNIT <= capacity && (!PAGED || in_page + FD_UNIT <= KV_PAGE);
    if (run) {
      const size_t off = (PAGED ? (size_t)page * KV_PAGE + in_page : (size_t)first) * hd;
      warp_load_run<HDP>(dst, n, hd, kc + off, lane);
      warp_load_run<HDP>(dst + TILE, n, hd, vc + off, lane);
    } else {
      warp_load_rows<HDP>(dst, n, hd, kc, my_pages, first, capacity, lane);
      warp_load_rows<HDP>(dst + TILE, n, hd, vc, my_pages, first, capacity, lane);
    }
  };
  // FD_STAGES - 1 units are requested before the first is used.  All rows but the newest
  // position's are older than this step: their units are requested before the wait; the
  // unit that holds the newest key (the sequence's last) and the queries come after it.
  const int u_new = (nkeys - 1) / FD_UNIT;
  int u_next = u0 + warp;
  int row_next = (lo + u_next * FD_UNIT) % capacity;
  int row_first[FD_STAGES - 1], page_first[FD_STAGES - 1];
#pragma unroll
  for (int i = 0; i < FD_STAGES - 1; ++i) {
    row_first[i] = row_next;
    page_first[i] = page_of(u_next, row_next);
    u_next += NW;
    row_next += ring_step;
    if (row_next >= capacity) row_next -= capacity;
  }
  int page_next = page_of(u_next, row_next);
#pragma unroll
  for (int i = 0; i < FD_STAGES - 1; ++i) {
    const int u = u0 + warp + i * NW;
    // (fused: the newest key's unit comes now as well; its row for this step's position
    // holds an old key, which is written over below)
    if (u < u1 && (FUSED || u != u_new)) load_unit(u, i, row_first[i], page_first[i]);
    cp_async_commit();
  }
  pdl_wait();
  if (!FUSED) {
    load_tile<HDP, FD_THREADS>(q_s, FD_ROWS, hd, q, [&](int r) -> const T16* {
      return r < nh ? q + ((size_t)t * H + h0 + r) * hd : nullptr;
    });
#pragma unroll
    for (int i = 0; i < FD_STAGES - 1; ++i) {
      const int u = u0 + warp + i * NW;
      if (u < u1 && u == u_new) load_unit(u, i, row_first[i], page_first[i]);
    }
    cp_async_commit();
    cp_async_wait<0>();                                      // this thread's share of Q and of the first units
    __syncthreads();                                         // everybody's
  } else {
    // ---- what the rotary kernel would have done for this block's heads.  Work items of four
    // pairs (q and k: elements i..i+3 and i+half..) or four elements (v); a thread's slices are
    // all asked for before the first is added.
    const int half = hd >> 1;
    const int per_q = half >> 2, per_v = hd >> 2;            // items per query head, of v
    const bool newest_here = u_new >= u0 && u_new < u1;      // this block sees this step's key
    const int n_items = nh * per_q + (newest_here ? per_q + per_v : 0);
    const int row_elems = (H + 2 * G) * hd;
    const float* tok_row = fz.qkv + (size_t)t * row_elems;
    const int r_new = (nkeys - 1) - u_new * FD_UNIT;         // the new key's row in its unit
    const int new_at = u_new - u0;                           // its unit: warp new_at % 4, stage new_at / 4
    const bool staged = newest_here && new_at < (FD_STAGES - 1) * NW;
    const uint32_t new_tile = q_s + FD_ROWS * HDP * 2 + (new_at % NW) * WARP_RING +
                              (new_at / NW) * 2 * TILE;
    const size_t new_row = newest_here
        ? kv_row_offset(page_table, pps, n_pages, slot, g, G, capacity, pos % capacity, hd) : 0;
    cp_async_wait<0>();                                      // this thread's share of the first units
    __syncthreads();                                         // everybody's: their rows may be written over
#pragma unroll 1
    for (int item = threadIdx.x; item < n_items; item += FD_THREADS) {
      int col, i, kind;                                      // kind 0: q, 1: k, 2: v
      int r = 0;
      if (item < nh * per_q) {
        r = item / per_q;
        i = (item - r * per_q) * 4;
        col = (h0 + r) * hd + i;
        kind = 0;
      } else if (item < nh * per_q + per_q) {
        i = (item - nh * per_q) * 4;
        col = (H + g) * hd + i;
        kind = 1;
      } else {
        i = (item - nh * per_q - per_q) * 4;
        col = (H + G + g) * hd + i;
        kind = 2;
      }
      const float* sp = tok_row + col;
      const int second = kind == 2 ? 0 : half;               // v has no partner
      float a[4] = {0.f, 0.f, 0.f, 0.f}, bb[4] = {0.f, 0.f, 0.f, 0.f};
      constexpr int SB = 8;
      for (int p0 = 0; p0 < fz.n_partials; p0 += SB) {
        float4 x[SB], y[SB];
#pragma unroll
        for (int j = 0; j < SB; ++j) {
          const float* pp = sp + (size_t)(p0 + j) * fz.partial_stride;
          const bool live = p0 + j < fz.n_partials;
          x[j] = live ? *reinterpret_cast<const float4*>(pp) : make_float4(0.f, 0.f, 0.f, 0.f);
          y[j] = (live && kind != 2) ? *reinterpret_cast<const float4*>(pp + second)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < SB; ++j) {
          a[0] += x[j].x; a[1] += x[j].y; a[2] += x[j].z; a[3] += x[j].w;
          bb[0] += y[j].x; bb[1] += y[j].y; bb[2] += y[j].z; bb[3] += y[j].w;
        }
      }
      if (kind != 2) {
        const float4* cs = reinterpret_cast<const float4*>(fz.cos_sin + (size_t)t * half + i);
        const float4 c01 = cs[0], c23 = cs[1];               // (cos, sin) of pairs i, i+1 and i+2, i+3
        const float cc[4] = {c01.x, c01.z, c23.x, c23.z}, ss[4] = {c01.y, c01.w, c23.y, c23.w};
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float r0 = rotate_lo(a[v], bb[v], cc[v], ss[v]), r1 = rotate_hi(a[v], bb[v], cc[v], ss[v]);
          a[v] = r0;
          bb[v] = r1;
        }
      }
      const uint2 lo4 = make_uint2(pack2<T16>(a[0], a[1]), pack2<T16>(a[2], a[3]));
      const uint2 hi4 = make_uint2(pack2<T16>(bb[0], bb[1]), pack2<T16>(bb[2], bb[3]));
      if (kind == 0) {
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(tile_addr<HDP>(q_s, r, i >> 3) + (i & 4) * 2),
                     "r"(lo4.x), "r"(lo4.y) : "memory");
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};"
                     ::"r"(tile_addr<HDP>(q_s, r, (i + half) >> 3) + ((i + half) & 4) * 2), "r"(hi4.x), "r"(hi4.y)
                     : "memory");
      } else {
        T16* crow = const_cast<T16*>(kind == 1 ? k_cache : v_cache) + new_row + i;
        *reinterpret_cast<uint2*>(crow) = lo4;
        if (kind == 1) *reinterpret_cast<uint2*>(crow + half) = hi4;
        if (staged) {
          const uint32_t tile = new_tile + (kind == 2 ? TILE : 0);
          asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(tile_addr<HDP>(tile, r_new, i >> 3) + (i & 4) * 2),
                       "r"(lo4.x), "r"(lo4.y) : "memory");
          if (kind == 1)
            asm volatile("st.shared.v2.b32 [%0], {%1, %2};"
                         ::"r"(tile_addr<HDP>(tile, r_new, (i + half) >> 3) + ((i + half) & 4) * 2),
                           "r"(hi4.x), "r"(hi4.y) : "memory");
        }
      }
    }
    // q and the new row are in place for every warp; a unit with the new key that is asked
    // for later in the loop finds the row in the cache (a write of this block, before this barrier)
    __syncthreads();
  }
  // Q^T as the B operand: per 16-wide step two registers for heads 0-7, two for 8-15
  uint32_t qf[NKS][4];
#pragma unroll
  for (int ks = 0; ks < NKS; ++ks)
      ldsm_x4(qf[ks], tile_addr<HDP>(q_s, (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));

  float o[NKS][NT][4];                                       // O^T: 16 features x 8 heads per tile
#pragma unroll
  for (int i = 0; i < NKS; ++i)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][nt][j] = 0.f;
  float m_w[NT][2], l_w[NT][2];                              // per head (column): tig*2, tig*2+1
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    m_w[nt][0] = m_w[nt][1] = -INFINITY;
    l_w[nt][0] = l_w[nt][1] = 0.f;
  }

  // ldmatrix addresses: a lane's row, and its column's swizzle as an exclusive-or
  const uint32_t k_lane = (lane & 15) * (HDP * 2), k_x = (uint32_t)((lane >> 4) ^ (lane & 7)) << 4;
  const uint32_t v_lane = ((lane & 7) + ((lane >> 4) << 3)) * (HDP * 2),
                 v_x = (uint32_t)(((lane >> 3) & 1) ^ (lane & 7)) << 4;
  int it = 0;
  for (int u = u0 + warp; u < u1; u += NW, ++it) {
    const int stage = it % FD_STAGES;
    cp_async_wait<FD_STAGES - 2>();                          // unit u has landed (this lane's share)
    __syncwarp();                                            // ... every lane's; unit u-1 is read out
    if (u_next < u1) load_unit(u_next, (it + FD_STAGES - 1) % FD_STAGES, row_next, page_next);
    u_next += NW;
    row_next += ring_step;
    if (row_next >= capacity) row_next -= capacity;
    page_next = page_of(u_next, row_next);
    cp_async_commit();
    const uint32_t k_s = ring_s + stage * 2 * TILE + k_lane, v_s = ring_s + stage * 2 * TILE + TILE + v_lane;
    const int n = min(FD_UNIT, pos + 1 - (lo + u * FD_UNIT));

    float s[FD_MT][NT][4];                                       // S^T: two tiles of 16 keys x 8 heads
#pragma unroll
    for (int mt = 0; mt < FD_MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[mt][nt][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < NKS; ++ks) {
      {
        const uint32_t a = k_s + ((uint32_t)(ks << 5) ^ k_x);
#pragma unroll
        for (int mt = 0; mt < FD_MT; ++mt) {
          uint32_t kf[4];
          ldsm_x4(kf, a + mt * 16 * HDP * 2);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_16<T16>(s[mt][nt], kf, &qf[ks][2 * nt]);
        }
      }
    }
    if (n < FD_UNIT) {                                       // the sequence's last unit
#pragma unroll
      for (int mt = 0; mt < FD_MT; ++mt)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (mt * 16 + gid + ((j >> 1) << 3) >= n)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) s[mt][nt][j] = -INFINITY;
    }
    // maxima of the raw scores (the scale is positive); every unit has a live key
    bool changed = false;
    float corr[NT][2], m_neg[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float m = fmaxf(s[0][nt][c], s[0][nt][c + 2]);
#pragma unroll
        for (int mt = 1; mt < FD_MT; ++mt) m = fmaxf(m, fmaxf(s[mt][nt][c], s[mt][nt][c + 2]));
        m = fmaxf(m, __shfl_xor_sync(FULL, m, 4));
        m = fmaxf(m, __shfl_xor_sync(FULL, m, 8));
        m = fmaxf(m, __shfl_xor_sync(FULL, m, 16));
        m = fmaxf(m * scale_log2, m_w[nt][c]);
        corr[nt][c] = ex2_approx(m_w[nt][c] - m);
        changed |= m != m_w[nt][c];
        l_w[nt][c] *= corr[nt][c];
        m_w[nt][c] = m;
        m_neg[nt][c] = -m;
      }
    if (__any_sync(FULL, changed)) {                         // rare after the first units
#pragma unroll
      for (int i = 0; i < NKS; ++i)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          o[i][nt][0] *= corr[nt][0]; o[i][nt][1] *= corr[nt][1];
          o[i][nt][2] *= corr[nt][0]; o[i][nt][3] *= corr[nt][1];
        }
    }
    // P^T as the B operand of the second product: each 8x8 block of S^T, transposed
    uint32_t pb[FD_MT][NT][2];
#pragma unroll
    for (int mt = 0; mt < FD_MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          p[j] = ex2_approx(fmaf(s[mt][nt][j], scale_log2, m_neg[nt][j & 1]));
          l_w[nt][j & 1] += p[j];                            // this lane's keys only
        }
        pb[mt][nt][0] = movmatrix_t(pack2<T16>(p[0], p[1]));
        pb[mt][nt][1] = movmatrix_t(pack2<T16>(p[2], p[3]));
      }
#pragma unroll
    for (int i = 0; i < NKS; ++i) {
      {
        const uint32_t a = v_s + ((uint32_t)(i << 5) ^ v_x);
#pragma unroll
        for (int mt = 0; mt < FD_MT; ++mt) {
          uint32_t vf[4];
          ldsm_x4_t(vf, a + mt * 16 * HDP * 2);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_16<T16>(o[i][nt], vf, pb[mt][nt]);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();                                           // Q and every ring are free
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float l = l_w[nt][c];
      l += __shfl_xor_sync(FULL, l, 4);
      l += __shfl_xor_sync(FULL, l, 8);
      l += __shfl_xor_sync(FULL, l, 16);
      if (gid == 0) {
        wm_s[warp][nt * 8 + tig * 2 + c] = m_w[nt][c];
        wl_s[warp][nt * 8 + tig * 2 + c] = l;
      }
    }
  if (NT == 1 && gid == 1) {                                 // heads 8-15 do not exist
    wm_s[warp][8 + tig * 2] = wm_s[warp][9 + tig * 2] = -INFINITY;
    wl_s[warp][8 + tig * 2] = wl_s[warp][9 + tig * 2] = 0.f;
  }
  // merge the four warps (they saw different keys): partial outputs over the staging area
  float* o_s = reinterpret_cast<float*>(fa_smem);            // [warps][hd][FD_OPAD >= 16 heads]
#pragma unroll
  for (int i = 0; i < NKS; ++i) {
    if (i < nks) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float* p0 = o_s + ((size_t)warp * hd + i * 16 + gid) * FD_OPAD + nt * 8 + tig * 2;
        *reinterpret_cast<float2*>(p0) = make_float2(o[i][nt][0], o[i][nt][1]);
        *reinterpret_cast<float2*>(p0 + 8 * FD_OPAD) = make_float2(o[i][nt][2], o[i][nt][3]);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < FD_ROWS) {
    const int r = threadIdx.x;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, wm_s[w][r]);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float f = wm_s[w][r] > -INFINITY ? exp2f(wm_s[w][r] - M) : 0.f;
      wm_s[w][r] = f;                                         // now the warp's weight
      L += wl_s[w][r] * f;
    }
    row_m[r] = M;
    row_l[r] = L;
  }
  __syncthreads();
  const size_t qh = (size_t)t * H + h0;
  for (int idx = threadIdx.x; idx < nh * hd; idx += FD_THREADS) {
    const int d = idx / nh, r = idx - d * nh;
    float O = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) O += o_s[((size_t)w * hd + d) * FD_OPAD + r] * wm_s[w][r];
    if (n_parts == 1) {
      out[(qh + r) * hd + d] = from_float<T16>(O / row_l[r]);
    } else {
      const size_t pi = (qh + r) * max_parts + part;
      part_o[pi * hd + d] = O;
      if (d == 0) { part_ml[pi * 2] = row_m[r]; part_ml[pi * 2 + 1] = row_l[r]; }
    }
  }
  if (n_parts == 1) return;

  // the block that arrives last adds the parts in order
  __threadfence();
  __syncthreads();
  int* counter = counters + (size_t)t * gridDim.y + blockIdx.y;
  if (threadIdx.x == 0) last_flag = (atomicAdd(counter, 1) == n_parts - 1) ? 1 : 0;
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  if (threadIdx.x == 0) *counter = 0;
  // Up to 8 parts: every thread asks for its features' partial sums and its row's maxima and
  // sums at once (one trip to L2, no barrier) and adds them in the order of the parts: 1.5 us
  // less per layer than the two rounds below (7B sizes, 2 to 12 sequences: 1.2-1.6 % of a
  // step).  With 9 to 24 parts at once it is slower than the two rounds (one sequence: +1 %).
  auto merge_at_once = [&](auto width) {
    constexpr int MP = decltype(width)::value;
    for (int idx = threadIdx.x; idx < nh * hd; idx += FD_THREADS) {
      const int r = idx / hd, d = idx - r * hd;
      const float* po = part_o + (qh + r) * max_parts * hd + d;
      const float2* ml = reinterpret_cast<const float2*>(part_ml + (qh + r) * max_parts * 2);
      float v[MP], ms[MP], ls[MP];
#pragma unroll
      for (int j = 0; j < MP; ++j) {
        const bool live = j < n_parts;
        v[j] = live ? __ldcg(po + (size_t)j * hd) : 0.f;
        const float2 x = live ? __ldcg(ml + j) : make_float2(-INFINITY, 0.f);
        ms[j] = x.x;
        ls[j] = x.y;
      }
      float M = ms[0];
#pragma unroll
      for (int j = 1; j < MP; ++j) M = fmaxf(M, ms[j]);
      float O = 0.f, L = 0.f;
#pragma unroll
      for (int j = 0; j < MP; ++j) {
        const float f = ms[j] > -INFINITY ? exp2f(ms[j] - M) : 0.f;
        O = fmaf(v[j], f, O);
        L = fmaf(ls[j], f, L);
      }
      out[(qh + r) * hd + d] = from_float<T16>(O / L);
    }
  };
  if (n_parts <= 8) {
    merge_at_once(std::integral_constant<int, 8>());
    return;
  }
  float* w_s = reinterpret_cast<float*>(fa_smem);            // [n_parts][16 rows]
  for (int r = threadIdx.x >> 3; r < FD_ROWS; r += FD_THREADS / 8) {   // rows x 8 threads
    const int sub = threadIdx.x & 7;
    float M = -INFINITY;
    if (r < nh)
      for (int s2 = sub; s2 < n_parts; s2 += 8)
        M = fmaxf(M, __ldcg(part_ml + ((qh + r) * max_parts + s2) * 2));
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    float L = 0.f;
    if (r < nh)
      for (int s2 = sub; s2 < n_parts; s2 += 8) {
        const float* ml = part_ml + ((qh + r) * max_parts + s2) * 2;
        const float ms = __ldcg(ml);
        const float f = ms > -INFINITY ? exp2f(ms - M) : 0.f;
        L += __ldcg(ml + 1) * f;
        w_s[s2 * FD_ROWS + r] = f;
      }
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
    if (sub == 0 && r < nh) row_l[r] = L;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nh * hd; idx += FD_THREADS) {
    const int r = idx / hd, d = idx - r * hd;
    const float* po = part_o + (qh + r) * max_parts * hd + d;
    float O = 0.f;
    int s2 = 0;
    for (; s2 + 8 <= n_parts; s2 += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __ldcg(po + (size_t)(s2 + j) * hd);
#pragma unroll
      for (int j = 0; j < 8; ++j) O = fmaf(v[j], w_s[(s2 + j) * FD_ROWS + r], O);
    }
    for (; s2 < n_parts; ++s2) O = fmaf(__ldcg(po + (size_t)s2 * hd), w_s[s2 * FD_ROWS + r], O);
    out[(qh + r) * hd + d] = from_float<T16>(O / row_l[r]);
  }
}

template <int HDP, int NT, typename T16, bool PAGED, bool FUSED, int NW>
static int launch_decode_mma(const void* q, const void* k_cache, const void* v_cache,
                             const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                             float* part_ml, int* counters, int* status, int n_seqs, int H, int G,
                             int hd, int capacity, int window, int cpc, int max_parts,
                             const int* page_table, int pps, int n_pages, const fd_fused_args& fz,
                             cudaStream_t stream) {
  // Q, then every warp's ring of (K, V) stages; the merge buffer lies over them
  size_t smem = (size_t)(FD_ROWS + NW * FD_STAGES * 2 * FD_UNIT) * HDP * 2;
  const size_t merge = (size_t)NW * hd * FD_OPAD * 4;
  if (smem < merge) smem = merge;
  static size_t attr_smem = 0;
  if (smem > attr_smem) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<HDP, NT, T16, PAGED, FUSED, NW>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_smem = smem;
  }
  const int nhc = (H / G + FD_ROWS - 1) / FD_ROWS;
  const dim3 grid(max_parts, G * nhc, n_seqs);
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  launch_pdl(attn_decode_mma_kernel<HDP, NT, T16, PAGED, FUSED, NW>, grid, dim3(NW * 32), smem, stream,
             (const T16*)q, (const T16*)k_cache, (const T16*)v_cache,
             seq_slot, slot_pos, (T16*)out, part_o, part_ml, counters, status, H, G, hd,
             capacity, window, cpc, max_parts, scale_log2, page_table, pps, n_pages, fz);
  YALM_LAUNCH_CHECK();
  return 0;
}

template <int HDP, typename T16>
static int launch_prefill(const void* q, const void* kv_step, const void* k_cache,
                          const void* v_cache, const int* q_start, const int* seq_slot,
                          const int* slot_pos, void* out, int n_seqs, int max_q_len, int H, int G,
                          int hd, int capacity, int window, const int* page_table, int pps,
                          int n_pages, cudaStream_t stream) {
  const size_t smem = (size_t)(FA_BM + 4 * FA_BN) * HDP * 2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<HDP, T16>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_prefill_mma_kernel<HDP, T16>,
                             cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const dim3 grid((max_q_len + FA_BM - 1) / FA_BM, H, n_seqs);
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  launch_pdl(attn_prefill_mma_kernel<HDP, T16>, grid, dim3(FP_THREADS), smem, stream,
             (const T16*)q, (const T16*)kv_step, (const T16*)k_cache,
             (const T16*)v_cache, q_start, seq_slot, slot_pos, (T16*)out, H, G,
             hd, capacity, window, scale_log2, page_table, pps, n_pages);
  YALM_LAUNCH_CHECK();
  return 0;
}

// host side of the decode kernel: argument checks and the choice of the instantiation
template <bool FUSED, int NW>
static int decode_mma_dispatch(const void* q, const void* k_cache, const void* v_cache,
                               const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                               float* part_ml, int* counters, int* status, int dtype, int n_seqs, int H,
                               int G, int hd, int capacity, int window, int max_context,
                               int chunks_per_block, const int* page_table,
                               int pages_per_slot, int n_pages, const fd_fused_args* fused,
                               cudaStream_t stream) {
  static_assert(NW == FD_WARPS_MAX || NW == 2, "blocks of four warps, or of two");
  if (n_seqs <= 0) return 0;
  if (dtype != DT_BF16 && dtype != DT_F16) return -3;
  if (hd % 16 != 0 || hd > 128 || hd <= 0) return -2;
  if (G <= 0 || H % G != 0) return -3;
  if (max_context <= 0 || n_seqs > 65535 || chunks_per_block < 1) return -4;
  const int visible = window > 0 && window < max_context ? window : max_context;
  const int max_chunks = (visible + FD_CHUNK - 1) / FD_CHUNK;
  const int max_parts = (max_chunks + chunks_per_block - 1) / chunks_per_block;
  if ((size_t)G * ((H / G + FD_ROWS - 1) / FD_ROWS) > 65535) return -4;
  const bool two = H / G > 8;                                 // a second tile of 8 heads
  const fd_fused_args none = {nullptr, nullptr, 0, 0};
  const fd_fused_args& fz = fused ? *fused : none;
#define YALM_FD_(HDP, NT, T, PAGED)                                                              \
  launch_decode_mma<HDP, NT, T, PAGED, FUSED, NW>(q, k_cache, v_cache, seq_slot, slot_pos, out,  \
                                                  part_o, part_ml, counters, status, n_seqs, H,  \
                                                  G, hd, capacity, window, chunks_per_block,     \
                                                  max_parts, page_table, pages_per_slot,         \
                                                  n_pages, fz, stream)
#define YALM_FD(HDP, NT, T) (page_table ? YALM_FD_(HDP, NT, T, true) : YALM_FD_(HDP, NT, T, false))
  if (dtype == DT_F16) {
    if (hd <= 64) return two ? YALM_FD(64, 2, __half) : YALM_FD(64, 1, __half);
    return two ? YALM_FD(128, 2, __half) : YALM_FD(128, 1, __half);
  }
  if (hd <= 64) return two ? YALM_FD(64, 2, __nv_bfloat16) : YALM_FD(64, 1, __nv_bfloat16);
  return two ? YALM_FD(128, 2, __nv_bfloat16) : YALM_FD(128, 1, __nv_bfloat16);
#undef YALM_FD
#undef YALM_FD_
}

}  // namespace yalm
