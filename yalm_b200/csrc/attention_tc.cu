// Prefill attention on tcgen05: S = Q.K^T and P.V as UMMA instructions with the
// accumulators in tensor memory, operands brought by TMA.
//
// A block takes 128 query tokens of one head of one sequence; 128 threads own one
// query row each.  Per block of 128 keys: the MMA thread issues S = Q.K^T into TMEM;
// every softmax thread reads its row of S (tcgen05.ld), applies scale and mask,
// keeps the running max and sum in 32-bit, writes exp2(s - max) as bfloat16 into a
// swizzled shared-memory tile P; the MMA thread issues P.V (V is the MN-major B
// operand, exactly as TMA lays its rows down); the threads read the product and
// add it to their output row in registers, rescaled when the max moved.  While the
// threads do that, the next block's S is already being computed.
//
// Same mathematics as the reference's attn_dot / attn_softmax / att_mix
// (infer.cu:339-523) and as attention.cu.  Takes the case "all keys are this step's
// own" (prompts from their first token); head sizes 64 and 128.  Every wait on a
// barrier is bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int TA_BM = 128;     // query rows per block
constexpr int TA_BN = 128;     // keys per iteration
constexpr int TA_THREADS = 192;
constexpr int TA_STAGES = 2;

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
__device__ __forceinline__ void ta_umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void ta_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar) : "memory");
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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(TA_THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                       const int* __restrict__ q_start, __nv_bfloat16* __restrict__ out, int H, int G,
                       int window, float scale_log2, int* __restrict__ status) {
  constexpr int SUB = HD / 64;                     // 64-column sub-tiles of a head
  constexpr int Q_BYTES = TA_BM * HD * 2;
  constexpr int KV_BYTES = TA_BN * HD * 2;         // one of K or V
  constexpr int TMEM_COLS = 256;                   // S: 128 columns, P.V: HD columns
  extern __shared__ uint8_t ta_smem[];
  __shared__ __align__(8) uint64_t q_full, s_full, pv_full, p_ready;
  __shared__ __align__(8) uint64_t kv_full[TA_STAGES], kv_empty[TA_STAGES];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int g = h / (H / G);
  const int qs = q_start[b], q_len = q_start[b + 1] - qs;       // written by a host copy: safe early
  const int m0 = (gridDim.x - 1 - blockIdx.x) * TA_BM;          // heaviest tiles first
  if (m0 >= q_len) return;
  const int rows = min(TA_BM, q_len - m0);
  const int p_last = m0 + rows - 1;
  const int k_end = p_last + 1;
  const int k_begin = window > 0 ? max(0, m0 - window + 1) : 0;
  const int kb0 = k_begin / TA_BN, kb1 = (k_end + TA_BN - 1) / TA_BN;
  const int nkb = kb1 - kb0;

  const uint32_t base = (smem_u32(ta_smem) + 1023u) & ~1023u;
  const uint32_t q_s = base;
  const uint32_t kv_s = q_s + Q_BYTES;                          // stages of (K, V)
  const uint32_t p_s = kv_s + TA_STAGES * 2 * KV_BYTES;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), 1);
    mbar_init(smem_u32(&s_full), 1);
    mbar_init(smem_u32(&pv_full), 1);
    mbar_init(smem_u32(&p_ready), TA_BM);
    for (int s = 0; s < TA_STAGES; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
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
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + TA_BN;
  volatile int* abort_p = &abort_flag;
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_kv)) : "memory");
      pdl_wait();
      mbar_expect_tx(smem_u32(&q_full), Q_BYTES);
#pragma unroll
      for (int sub = 0; sub < SUB; ++sub)
        ta_tma_load_2d(q_s + sub * (TA_BM * 128), &map_q, h * HD + sub * 64, qs + m0,
                       smem_u32(&q_full));
      for (int it = 0; it < nkb; ++it) {
        const int s = it % TA_STAGES;
        const uint32_t phase = (it / TA_STAGES) & 1;
        if (!mbar_wait(smem_u32(&kv_empty[s]), phase ^ 1u, abort_p)) break;
        const uint32_t bar = smem_u32(&kv_full[s]);
        mbar_expect_tx(bar, 2 * KV_BYTES);
        const int row = qs + (kb0 + it) * TA_BN;
        const uint32_t k_dst = kv_s + s * 2 * KV_BYTES, v_dst = k_dst + KV_BYTES;
#pragma unroll
        for (int sub = 0; sub < SUB; ++sub) {
          ta_tma_load_2d(k_dst + sub * (TA_BN * 128), &map_kv, g * HD + sub * 64, row, bar);
          ta_tma_load_2d(v_dst + sub * (TA_BN * 128), &map_kv, (G + g) * HD + sub * 64, row, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      // S: M = 128 queries, N = 128 keys, both operands K-major
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TA_BN >> 3) << 17) |
                               ((uint32_t)(TA_BM >> 4) << 24);
      // P.V: M = 128 queries, N = HD, A (P) K-major, B (V) MN-major
      const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TA_BM >> 4) << 24);
      bool ok = mbar_wait(smem_u32(&q_full), 0, abort_p);
      auto issue_s = [&](int it) {
        const int s = it % TA_STAGES;
        const uint32_t k_src = kv_s + s * 2 * KV_BYTES;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks / 4) * (TA_BM * 128) + (ks % 4) * 32;
          ta_umma(tmem_s, ta_desc_k(q_s + off), ta_desc_k(k_src + off), idesc_s, ks > 0 ? 1u : 0u);
        }
        ta_commit(smem_u32(&s_full));
      };
      if (ok && nkb > 0) {
        ok = mbar_wait(smem_u32(&kv_full[0]), 0, abort_p);
        if (ok) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(0);
        }
      }
      for (int it = 0; it < nkb && ok; ++it) {
        const int s = it % TA_STAGES;
        // P of this block is in shared memory and S has been read
        ok = mbar_wait(smem_u32(&p_ready), it & 1, abort_p);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_src = kv_s + s * 2 * KV_BYTES + KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < TA_BN / 16; ++kk) {
          const uint32_t p_off = (kk / 4) * (TA_BM * 128) + (kk % 4) * 32;
          ta_umma(tmem_pv, ta_desc_k(p_s + p_off), ta_desc_mn(v_src + kk * 16 * 128, TA_BN * 128),
                  idesc_pv, kk > 0 ? 1u : 0u);
        }
        ta_commit(smem_u32(&pv_full));
        ta_commit(smem_u32(&kv_empty[s]));                  // K and V of this block are consumed
        if (it + 1 < nkb) {
          const int s2 = (it + 1) % TA_STAGES;
          ok = mbar_wait(smem_u32(&kv_full[s2]), ((it + 1) / TA_STAGES) & 1, abort_p);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(it + 1);                                    // overlaps the threads' work on P.V
        }
      }
    }
  } else {
    // ---------------- softmax and output: one query row per thread
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int p = m0 + row;                                   // this row's position
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    pdl_wait();
    bool ok = true;
    for (int it = 0; it < nkb; ++it) {
      const int j0 = (kb0 + it) * TA_BN;
      mbar_wait(smem_u32(&s_full), it & 1, abort_p);
      asm volatile("bar.sync 1, %0;" ::"n"(TA_BM) : "memory");
      if (*abort_p) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool inside = j0 + TA_BN - 1 <= m0 && (window <= 0 || j0 > p_last - window);
      // pass 1: the row's maximum over this block
      float m_new = m_run;
#pragma unroll 1
      for (int c = 0; c < TA_BN; c += 32) {
        float v[32];
        ta_ld32(tmem_s + lane_addr + c, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = j0 + c + i;
          const bool vis = inside || (key <= p && (window <= 0 || key > p - window));
          m_new = fmaxf(m_new, vis ? v[i] * scale_log2 : -INFINITY);
        }
      }
      const float corr = m_new > -INFINITY ? exp2f(m_run - m_new) : 1.f;
      // pass 2: probabilities into the swizzled P tile, the row's sum
      float l_add = 0.f;
#pragma unroll 1
      for (int c = 0; c < TA_BN; c += 32) {
        float v[32];
        ta_ld32(tmem_s + lane_addr + c, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = j0 + c + i;
          const bool vis = inside || (key <= p && (window <= 0 || key > p - window));
          v[i] = (vis && m_new > -INFINITY) ? exp2f(v[i] * scale_log2 - m_new) : 0.f;
          l_add += v[i];
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {                      // four 16-byte chunks of 8 keys
          uint4 u;
          __nv_bfloat162 t0 = __floats2bfloat162_rn(v[ch * 8 + 0], v[ch * 8 + 1]);
          __nv_bfloat162 t1 = __floats2bfloat162_rn(v[ch * 8 + 2], v[ch * 8 + 3]);
          __nv_bfloat162 t2 = __floats2bfloat162_rn(v[ch * 8 + 4], v[ch * 8 + 5]);
          __nv_bfloat162 t3 = __floats2bfloat162_rn(v[ch * 8 + 6], v[ch * 8 + 7]);
          u.x = *reinterpret_cast<uint32_t*>(&t0);
          u.y = *reinterpret_cast<uint32_t*>(&t1);
          u.z = *reinterpret_cast<uint32_t*>(&t2);
          u.w = *reinterpret_cast<uint32_t*>(&t3);
          const int key_in = c + ch * 8;                      // 0..127
          const int sub = key_in >> 6, chunk = (key_in & 63) >> 3;
          const uint32_t addr = p_s + sub * (TA_BM * 128) + row * 128 + ((chunk ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                       ::"r"(addr), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
        }
      }
      l_run = l_run * corr + l_add;
      m_run = m_new;
      // P is complete for this row and S has been read: let the MMA thread go on
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(smem_u32(&p_ready));
      // the product of this block, added to the row
      mbar_wait(smem_u32(&pv_full), it & 1, abort_p);
      asm volatile("bar.sync 1, %0;" ::"n"(TA_BM) : "memory");
      if (*abort_p) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        float v[32];
        ta_ld32(tmem_pv + lane_addr + c, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = fmaf(o[c + i], corr, v[i]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (ok && row < rows) {
      const float inv = 1.0f / l_run;
      __nv_bfloat16* op = out + ((size_t)(qs + m0 + row) * H + h) * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        uint4 u;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(o[c + 0] * inv, o[c + 1] * inv);
        __nv_bfloat162 t1 = __floats2bfloat162_rn(o[c + 2] * inv, o[c + 3] * inv);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(o[c + 4] * inv, o[c + 5] * inv);
        __nv_bfloat162 t3 = __floats2bfloat162_rn(o[c + 6] * inv, o[c + 7] * inv);
        u.x = *reinterpret_cast<uint32_t*>(&t0);
        u.y = *reinterpret_cast<uint32_t*>(&t1);
        u.z = *reinterpret_cast<uint32_t*>(&t2);
        u.w = *reinterpret_cast<uint32_t*>(&t3);
        *reinterpret_cast<uint4*>(op + c) = u;
      }
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
// rows x cols bfloat16, row-major; box = 128 rows x 64 columns, 128-byte swizzle
static int ta_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols) {
  TaEncodeFn fn = ta_encode_fn();
  if (!fn) return -10;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

template <int HD>
static int launch_prefill_tc(const void* q, const void* kv_step, const int* q_start, void* out,
                             int n_tokens, int n_seqs, int max_q_len, int H, int G, int window,
                             int* status, cudaStream_t stream) {
  CUtensorMap mq, mkv;
  int rc = ta_make_map(&mq, q, n_tokens, (long long)H * HD);
  if (rc) return rc;
  rc = ta_make_map(&mkv, kv_step, n_tokens, (long long)2 * G * HD);
  if (rc) return rc;
  const size_t smem = (size_t)TA_BM * HD * 2 + (size_t)TA_STAGES * 2 * TA_BN * HD * 2 +
                      (size_t)TA_BM * TA_BN * 2 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const dim3 grid((max_q_len + TA_BM - 1) / TA_BM, H, n_seqs);
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
  launch_pdl(attn_prefill_tc_kernel<HD>, grid, dim3(TA_THREADS), smem, stream, mq, mkv, q_start,
             (__nv_bfloat16*)out, H, G, window, scale_log2, status);
  YALM_LAUNCH_CHECK();
  return 0;
}

}  // namespace yalm

using namespace yalm;

// Prefill attention on tcgen05 for sequences that start at their first token (every
// key is in kv_step).  q [n_tokens, H*hd], kv_step [n_tokens, 2, G, hd], out like q;
// bfloat16; hd 64 or 128.  q_start [n_seqs + 1] must be in place before the launch
// (it is read before the wait on the previous kernel).
extern "C" int yalm_attention_prefill_tc(const void* q, const void* kv_step, const int* q_start,
                                         void* out, int n_tokens, int n_seqs, int max_q_len, int H,
                                         int G, int hd, int window, int* status,
                                         cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0 || n_tokens <= 0) return 0;
  if (hd != 64 && hd != 128) return -2;
  if (G <= 0 || H % G != 0) return -3;
  if (H > 65535 || n_seqs > 65535) return -4;
  if (((uintptr_t)q | (uintptr_t)kv_step | (uintptr_t)out) & 15) return -6;
  if (hd == 64)
    return launch_prefill_tc<64>(q, kv_step, q_start, out, n_tokens, n_seqs, max_q_len, H, G,
                                 window, status, stream);
  return launch_prefill_tc<128>(q, kv_step, q_start, out, n_tokens, n_seqs, max_q_len, H, G,
                                window, status, stream);
}
