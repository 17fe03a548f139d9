// out[M,N] = A[M,K] * W[N,K]^T on the Blackwell tensor cores: bfloat16 or float16
// operands brought into shared memory by TMA (128-byte swizzle), tcgen05.mma
// issued by one thread, 32-bit accumulators in tensor memory (TMEM), read back
// with tcgen05.ld for a fused epilogue.
//
// The WEIGHT tile sits on the 128-row side of the instruction and the tokens on
// its N side (16..256), so the same kernel serves decode (a handful of tokens:
// the step is a stream of weights, optionally split over K so that all SMs pull
// from HBM) and prefill (256 tokens per tile: compute bound).  In TMEM a lane is
// an output feature and a column is a token.
//
// The reference's counterparts are its one-token GEMV kernels: matmul_wide
// infer.cu:250-268, fused_matmul_add_residuals infer.cu:270-288 (mode 1 here),
// fused_qkv_matmul_clip infer.cu:290-337, fused_ffn_w1_w3_glu_act
// infer.cu:610-634 (mode 2 here: two accumulators, gate and up, one epilogue).
//
// Every wait on a barrier is bounded: after about two seconds a role gives up,
// raises ERR_WAIT_TIMEOUT in the status word, and the block frees its TMEM and
// returns.
#include <cuda.h>

#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int TC_BM = 128;      // weight rows (output features) per tile = UMMA M
constexpr int TC_BK = 64;       // k per stage: 64 16-bit elements = one 128-byte swizzle row
constexpr int TC_UMMA_K = 16;
constexpr int TC_THREADS = 192; // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue

// The producers, like the issuers below, run as whole warps with one lane (`issue` set)
// executing the copy or the arrival, so that addresses and coordinates are uniform values.
__device__ __forceinline__ void tma_load_2d_by(uint32_t issue, uint32_t dst, const CUtensorMap* map,
                                               int x, int y, uint32_t bar) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %5, 0;\n"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];\n}"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "r"(issue)
      : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_by(uint32_t issue, uint32_t bar, uint32_t bytes) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %2, 0;\n"
      "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n}"
      ::"r"(bar), "r"(bytes), "r"(issue) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (64 16-bit elements) with the 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address
  d |= (uint64_t)1 << 16;                                // leading byte offset (unused here)
  d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
  return d;
}
// A product issued from a whole warp: every lane runs the (uniform) descriptor arithmetic,
// which can then stay in uniform registers, and the lane whose `issue` is set issues the
// instruction.  (In a branch that one lane takes, each operand goes from a vector register
// to a uniform one, a transfer at a time: about 80 clocks per instruction.)
__device__ __forceinline__ void umma_f16_by(uint32_t issue, uint32_t tmem_d, uint64_t adesc,
                                             uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
__device__ __forceinline__ void umma_commit_by(uint32_t issue, uint32_t bar) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %1, 0;\n"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}"
      ::"r"(bar), "r"(issue) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Instruction descriptor of tcgen05.mma kind::f16: 32-bit accumulator, both operands
// K-major unless b_mn_major, operand format bfloat16 or float16, N and M of the tile.
__device__ __forceinline__ uint32_t umma_idesc(int ab_dtype, int n, int m, bool b_mn_major = false) {
  const uint32_t fmt = ab_dtype == DT_BF16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn_major ? (1u << 16) : 0u) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int BT, int NACC> struct TcCfg {
  static constexpr int W_BYTES = TC_BM * TC_BK * 2;              // 16 KiB per weight tile
  static constexpr int A_BYTES = BT * TC_BK * 2;
  static constexpr int STAGE_BYTES = NACC * W_BYTES + A_BYTES;
  // two blocks per SM wherever the stages stay deep enough: a grid of up to 2 x SMs
  // tiles (or K slices) is then resident at once instead of running as two waves
  static constexpr int BUDGET = (BT <= 32 || (NACC == 1 && BT <= 128)) ? 110 * 1024 : 200 * 1024;
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;       // + slack to align to 1024
  static constexpr int TMEM_COLS_RAW = NACC * BT;
  static constexpr int TMEM_COLS = TMEM_COLS_RAW <= 32 ? 32 : (TMEM_COLS_RAW <= 64 ? 64 :
                                   (TMEM_COLS_RAW <= 128 ? 128 : (TMEM_COLS_RAW <= 256 ? 256 : 512)));
};

// mode 0: store, 1: add into float32 out, 2: silu(gate)*up (NACC == 2), 3: split-K partials,
// 4: silu(gate)*up with gate and up rows interleaved in groups of 16 (out is [M, N/2])
template <int BT, int NACC>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
               void* __restrict__ out, int out_dtype, int ab_dtype, int M, int N, int K, int mode,
               int splits, int* __restrict__ status) {
  using Cfg = TcCfg<BT, NACC>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[Cfg::STAGES];
  __shared__ __align__(8) uint64_t empty_bar[Cfg::STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  // (broadcasts from lane 0: the compiler then knows these are the same in every lane)
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int n_out = mode == 2 ? N / 2 : N;                   // features this grid covers
  const int feat0 = blockIdx.x * TC_BM;
  const int tok0 = blockIdx.y * BT;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  const int per = (nkb + splits - 1) / splits;
  const int kb_lo = blockIdx.z * per;
  const int kb_hi = min(nkb, kb_lo + per);
  const int nk = max(0, kb_hi - kb_lo);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&acc_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_slot, 0);
  volatile int* abort_p = &abort_flag;
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer: the whole warp runs the loop, lane 0 issues
    if (nk > 0) {
      const uint32_t issue = lane == 0 ? 1u : 0u;
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
      // weights do not depend on the previous kernel: the first stages' weight
      // tiles are requested before the wait, the activations after it
      const int pre = nk < Cfg::STAGES ? nk : Cfg::STAGES;
      for (int it = 0; it < pre; ++it) {
        const uint32_t stage = tiles + it * Cfg::STAGE_BYTES;
        const uint32_t bar = smem_u32(&full_bar[it]);
        mbar_expect_tx_by(issue, bar, Cfg::STAGE_BYTES);
        const int kx = (kb_lo + it) * TC_BK;
        tma_load_2d_by(issue, stage, &map_w, kx, feat0, bar);
        if (NACC == 2) tma_load_2d_by(issue, stage + Cfg::W_BYTES, &map_w, kx, n_out + feat0, bar);
      }
      pdl_wait();
      for (int it = 0; it < pre; ++it)
        tma_load_2d_by(issue, tiles + it * Cfg::STAGE_BYTES + NACC * Cfg::W_BYTES, &map_a,
                    (kb_lo + it) * TC_BK, tok0, smem_u32(&full_bar[it]));
      for (int it = pre; it < nk; ++it) {
        const int s = it % Cfg::STAGES;
        const uint32_t phase = (it / Cfg::STAGES) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&empty_bar[s]), phase ^ 1u, abort_p))) break;
        const uint32_t stage = tiles + s * Cfg::STAGE_BYTES;
        const uint32_t bar = smem_u32(&full_bar[s]);
        mbar_expect_tx_by(issue, bar, Cfg::STAGE_BYTES);
        const int kx = (kb_lo + it) * TC_BK;
        tma_load_2d_by(issue, stage, &map_w, kx, feat0, bar);
        if (NACC == 2) tma_load_2d_by(issue, stage + Cfg::W_BYTES, &map_w, kx, n_out + feat0, bar);
        tma_load_2d_by(issue, stage + NACC * Cfg::W_BYTES, &map_a, kx, tok0, bar);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: the whole warp runs the loop, lane 0 issues
    if (nk > 0) {
      const uint32_t issue = lane == 0 ? 1u : 0u;
      const uint32_t idesc = umma_idesc(ab_dtype, BT, TC_BM);
      bool ok = true;
      for (int it = 0; it < nk && ok; ++it) {
        const int s = it % Cfg::STAGES;
        const uint32_t phase = (it / Cfg::STAGES) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s]), phase, abort_p));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t stage = tiles + s * Cfg::STAGE_BYTES;
        const uint64_t wdesc = umma_desc_k_sw128(stage);
        const uint64_t adesc = umma_desc_k_sw128(stage + NACC * Cfg::W_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          const uint64_t koff = (uint64_t)((k * TC_UMMA_K * 2) >> 4);   // 32 bytes per k-step
          umma_f16_by(issue, tmem_base, wdesc + koff, adesc + koff, idesc, acc);
          if (NACC == 2) {
            const uint64_t w2 = umma_desc_k_sw128(stage + Cfg::W_BYTES);
            umma_f16_by(issue, tmem_base + BT, w2 + koff, adesc + koff, idesc, acc);
          }
        }
        umma_commit_by(issue, smem_u32(&empty_bar[s]));     // frees the stage once these MMAs are done
      }
      if (ok) umma_commit_by(issue, smem_u32(&acc_bar));    // accumulators complete
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> global
    const int quarter = warp & 3;                 // the TMEM lanes this warp may read
    const int f = feat0 + quarter * 32 + lane;    // output feature of this thread
    bool ok = true;
    pdl_wait();                                   // `out` may be read or written by the previous kernel
    if (nk > 0) ok = mbar_wait(smem_u32(&acc_bar), 0, abort_p);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      float* outf = reinterpret_cast<float*>(out);
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 16) {
        if (tok0 + c0 >= M) break;                // uniform over the warp
        float v[16];
        if (nk > 0) {
          tmem_ld16(taddr + c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
        if (NACC == 2) {
          float u[16];
          tmem_ld16(taddr + BT + c0, u);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu_times_fast(v[j], u[j]);
        }
        if (mode == 4) {
          // weight rows come as 16 gate rows followed by the 16 up rows of the same features
          float r[8];
          silu_pairs_of_chunk(v, lane, r);
          const int fo = (feat0 >> 1) + quarter * 16 + (lane & 15);
          if (fo < (N >> 1))
            store_eight_tokens(out_dtype, out, r, fo, tok0 + c0 + (lane < 16 ? 0 : 8), M, N >> 1);
          continue;
        }
        if (f < n_out && mode == 1) {
          // residual add as reductions at the memory: nothing to wait for (see sk_store_chunk)
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + c0 + j;
            if (tok < M) atomicAdd(&outf[(size_t)tok * n_out + f], v[j]);
          }
        } else if (f < n_out) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + c0 + j;
            if (tok < M) {
              if (mode == 3) {
                outf[((size_t)blockIdx.z * M + tok) * n_out + f] = v[j];
              } else if (out_dtype == DT_F32) {
                outf[(size_t)tok * n_out + f] = v[j];
              } else {
                store16_rt(out_dtype, out, (size_t)tok * n_out + f, v[j]);
              }
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_flag) {
    // a wait ran out: let copies in flight land before the block leaves
    if (threadIdx.x == 0) atomicOr(status, ERR_WAIT_TIMEOUT);
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rows x K of a 16-bit type, row-major; box = box_rows x 64 with the 128-byte swizzle
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows, int dtype) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                  2, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

// out [rows, cols] of float32 or a 16-bit type, row-major; box = 16 rows x box_cols columns,
// no swizzle: what the two-SM kernel's epilogue stages token-major in shared memory
static int make_out_map(CUtensorMap* map, void* ptr, int rows, int cols, int dtype, int box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  const int esz = dtype == DT_F32 ? 4 : 2;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * esz};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, 16};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType t = dtype == DT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                : dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(map, t, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

template <int BT, int NACC>
static int launch_tc(const CUtensorMap& mw, const void* A, void* out, int out_dtype, int ab_dtype,
                     int M, int N, int K, int mode, int splits, int* status, cudaStream_t stream) {
  using Cfg = TcCfg<BT, NACC>;
  static_assert(Cfg::STAGES >= 2, "pipeline needs two stages");
  CUtensorMap ma;
  int rc = make_map(&ma, A, M, K, BT, ab_dtype);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BT, NACC>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int n_out = mode == 2 ? N / 2 : N;
  const dim3 grid((n_out + TC_BM - 1) / TC_BM, (M + BT - 1) / BT, splits);
  if (grid.y > 65535 || grid.z > 65535) return -4;
  launch_pdl(gemm_tc_kernel<BT, NACC>, dim3(grid), dim3(TC_THREADS), Cfg::SMEM, stream, mw, ma, out,
             out_dtype, ab_dtype, M, N, K, mode, splits, status);
  YALM_LAUNCH_CHECK();
  return 0;
}


// Shared by the kernels below: tiles are ordered in bands of 8 weight tiles with the
// token tile running fastest inside a band, so blocks that run together share
// operands in L2.
constexpr int SK_BAND = 8;
constexpr int SK_EPI_THREADS = 128;

// One 16-column chunk of the epilogue for the thread that owns feature f.
__device__ __forceinline__ void sk_store_chunk(int mode, int out_dtype, void* __restrict__ out,
                                               const float* v, int f, int tok_first, int M,
                                               int n_out) {
  float* outf = reinterpret_cast<float*>(out);
  if (f >= n_out) return;
  if (mode == 1) {
    // out += v as reductions at the memory (no value comes back, so the chunk does not wait
    // for a round trip as a load, add and store would: 10 us less at the tail of a product of
    // 2,048 tokens).  Every element is added to once per launch, so the sum is the same.
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int tok = tok_first + j;
      if (tok < M) atomicAdd(&outf[(size_t)tok * n_out + f], v[j]);
    }
  } else if (out_dtype == DT_F32) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int tok = tok_first + j;
      if (tok < M) outf[(size_t)tok * n_out + f] = v[j];
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int tok = tok_first + j;
      if (tok < M) store16_rt(out_dtype, out, (size_t)tok * n_out + f, v[j]);
    }
  }
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 1;
  }
  return n;
}

// ===========================================================================
// The two-SM kernel for many tokens.
//
// A cluster of two blocks on neighbouring SMs computes one 256-feature x BT-token
// tile with tcgen05.mma.cta_group::2: each block brings its own 128 weight rows and
// its own half of the token tile into its shared memory, the first block's MMA
// thread issues one instruction that reads both halves, and each block's tensor
// memory receives its 128 rows of the result.  Per byte that leaves L2 the pair does
// 1.5 times the arithmetic of two single-SM 128x256 tiles, which is what the
// single-SM kernels are short of at these sizes.
//
// Barriers: the "full" barrier of a stage lives in the first block and counts the
// bytes of both blocks' TMA loads; "empty" and "accumulator full" barriers live in
// both blocks and are signalled by multicast commits; "accumulator empty" lives in
// the first block and counts the epilogue warps of both.  Persistent: a pair walks
// through tiles pair, pair + n_pairs, ...; two accumulator buffers in TMEM.
constexpr int G2_STAGE_LIMIT = 196 * 1024;

template <int BT, int NACC> struct G2Cfg {
  static constexpr int W_BYTES = TC_BM * TC_BK * 2;            // this block's 128 weight rows
  static constexpr int A_BYTES = (BT / 2) * TC_BK * 2;         // this block's half of the tokens
  static constexpr int STAGE_BYTES = NACC * W_BYTES + A_BYTES;
  static constexpr int STAGES_RAW = G2_STAGE_LIMIT / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;
  static constexpr int ACC_COLS = NACC * BT;
  static constexpr int ACC_STRIDE = (ACC_COLS + 63) / 64 * 64;  // the second buffer's first column
  static constexpr int TMEM_COLS = 512;
  static_assert(2 * ACC_STRIDE <= 512, "two accumulator buffers must fit into TMEM");
  static_assert(BT % 16 == 0 && BT <= 256 && STAGE_BYTES % 1024 == 0, "token tile of the pair");
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion bytes are counted on a barrier that may live in the peer block
__device__ __forceinline__ void tma_load_2d_pair_by(uint32_t issue, uint32_t dst, const CUtensorMap* map,
                                                    int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %5, 0;\n"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];\n}"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr), "r"(issue)
      : "memory");
}
// The pair's product, issued like umma_f16_by (whole warp, one issuing lane).
__device__ __forceinline__ void umma_f16_pair_by(uint32_t issue, uint32_t tmem_d, uint64_t adesc,
                                                  uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(issue)
      : "memory");
}
// arrives on the barrier at this offset in both blocks once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair_by(uint32_t issue, uint32_t bar) {
  asm volatile(
      "{\n.reg .pred q;\nsetp.ne.b32 q, %1, 0;\n"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %2;\n}"
      ::"r"(bar), "r"(issue), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];"
               ::"r"(bar_cluster_addr) : "memory");
}

// mode 0: store, 1: add into float32 out, 2: silu(gate)*up (NACC == 2), 4: silu(gate)*up
// with gate and up rows interleaved in groups of 16
template <int BT, int NACC, bool SPLIT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS)
gemm_2sm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                const __grid_constant__ CUtensorMap map_out, int out_tma,
                void* __restrict__ out, int out_dtype, int ab_dtype, int M, int N, int K, int mode,
                int splits, int* __restrict__ status, const yalm_rope_args rope) {
  using Cfg = G2Cfg<BT, NACC>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[Cfg::STAGES];
  __shared__ __align__(8) uint64_t empty_bar[Cfg::STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  // mode 5 (rotary epilogue): a 16-token chunk of the block's 128 features, so that a
  // feature finds its rotation partner, and each token's position and cache row
  // The epilogues' staging area: for mode 5 rope_ex [128][17] floats and rope_out [16][136]
  // 16-bit (a rotated chunk, token-major); for stores through TMA two buffers of a 16-token
  // chunk of the block's 128 features, token-major ([16][128] of the output type).
  constexpr int EPI_BYTES = NACC == 1 ? 16384 : 16;
  constexpr int ROPE_OUT_AT = TC_BM * 17 * 4;
  static_assert(NACC != 1 || ROPE_OUT_AT + 16 * (TC_BM + 8) * 2 <= EPI_BYTES, "staging area");
  __shared__ __align__(128) uint8_t epi_smem[EPI_BYTES];
  float (*rope_ex)[17] = reinterpret_cast<float(*)[17]>(epi_smem);
  uint16_t (*rope_out)[TC_BM + 8] = reinterpret_cast<uint16_t(*)[TC_BM + 8]>(epi_smem + (NACC == 1 ? ROPE_OUT_AT : 0));
  __shared__ int rope_row[NACC == 1 ? BT : 1], rope_where[NACC == 1 ? BT : 1];

  // (broadcasts from lane 0: the compiler then knows these are the same in every lane)
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const uint32_t rank = __shfl_sync(0xffffffffu, cluster_rank(), 0);
  const bool leader = rank == 0;
  const uint32_t tiles_smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int n_out = mode == 2 ? N / 2 : N;
  const int n_feat_tiles = (n_out + 2 * TC_BM - 1) / (2 * TC_BM);     // tiles of 256 features
  const int n_tok_tiles = (M + BT - 1) / BT;
  const int n_tiles = n_feat_tiles * n_tok_tiles;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  // work items: (tile, slice of K); compiled without slices (every mode but 3) an item is a tile
  const int n_items = SPLIT ? n_tiles * splits : n_tiles;
  const int k_per = SPLIT ? (nkb + splits - 1) / splits : nkb;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc_full[b]), 1);
      mbar_init(smem_u32(&acc_empty[b]), 2 * (SK_EPI_THREADS / 32));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                        // both blocks' barriers exist
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_slot, 0);
  volatile int* abort_p = &abort_flag;
  pdl_launch_dependents();

  // tile -> (first feature of the pair's 256, first token); bands of 8 feature tiles
  auto tile_of = [&](int t, int& feat0, int& tok0) {
    const int band_tiles = SK_BAND * n_tok_tiles;
    const int band = t / band_tiles;
    const int in_band = t - band * band_tiles;
    const int band_w = min(SK_BAND, n_feat_tiles - band * SK_BAND);
    feat0 = (band * SK_BAND + in_band % band_w) * 2 * TC_BM;
    tok0 = (in_band / band_w) * BT;
  };

  // item -> its tile's place and its k-blocks [kb_lo, kb_hi): slices of one tile lie n_tiles apart
  auto item_of = [&](int t, int& feat0, int& tok0, int& kb_lo, int& kb_hi) {
    const int slice = SPLIT ? t / n_tiles : 0;
    tile_of(t - slice * n_tiles, feat0, tok0);
    kb_lo = slice * k_per;
    kb_hi = SPLIT ? min(nkb, kb_lo + k_per) : nkb;
    return slice;
  };

  if (warp == 0) {
    // ---------------- TMA producer (warp 0 of each block runs the loop, its lane 0 issues)
    if (pair < n_items) {
      const uint32_t issue = lane == 0 ? 1u : 0u;
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
      // weights do not depend on the previous kernel: the first tile's first stages of them
      // are requested before the wait, the tokens of those stages after it
      int pre;
      {
        int feat0, tok0, kb_lo, kb_hi;
        item_of(pair, feat0, tok0, kb_lo, kb_hi);
        pre = kb_hi - kb_lo < Cfg::STAGES ? kb_hi - kb_lo : Cfg::STAGES;
        const int my_feat = feat0 + (int)rank * TC_BM;
        for (int i = 0; i < pre; ++i) {
          const uint32_t stage = tiles_smem + i * Cfg::STAGE_BYTES;
          const uint32_t bar0 = map_to_rank(smem_u32(&full_bar[i]), 0);
          mbar_expect_tx_by(leader ? issue : 0u, smem_u32(&full_bar[i]), 2 * Cfg::STAGE_BYTES);
          tma_load_2d_pair_by(issue, stage, &map_w, (kb_lo + i) * TC_BK, my_feat, bar0);
          if (NACC == 2)
            tma_load_2d_pair_by(issue, stage + Cfg::W_BYTES, &map_w, (kb_lo + i) * TC_BK, n_out + my_feat, bar0);
        }
        pdl_wait();
        const int my_tok = tok0 + (int)rank * (BT / 2);
        for (int i = 0; i < pre; ++i)
          tma_load_2d_pair_by(issue, tiles_smem + i * Cfg::STAGE_BYTES + NACC * Cfg::W_BYTES, &map_a,
                              (kb_lo + i) * TC_BK, my_tok, map_to_rank(smem_u32(&full_bar[i]), 0));
      }
      int it = 0;
      bool ok = true;
      for (int t = pair; t < n_items && ok; t += n_pairs) {
        int feat0, tok0, kb_lo, kb_hi;
        item_of(t, feat0, tok0, kb_lo, kb_hi);
        const int my_feat = feat0 + (int)rank * TC_BM;
        const int my_tok = tok0 + (int)rank * (BT / 2);
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          if (it < pre) continue;                             // requested above
          const int s = it % Cfg::STAGES;
          const uint32_t phase = (it / Cfg::STAGES) & 1;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&empty_bar[s]), phase ^ 1u, abort_p));
          if (!ok) break;
          const uint32_t stage = tiles_smem + s * Cfg::STAGE_BYTES;
          const uint32_t bar0 = map_to_rank(smem_u32(&full_bar[s]), 0);   // the first block's
          mbar_expect_tx_by(leader ? issue : 0u, smem_u32(&full_bar[s]), 2 * Cfg::STAGE_BYTES);
          const int kx = kb * TC_BK;
          tma_load_2d_pair_by(issue, stage, &map_w, kx, my_feat, bar0);
          if (NACC == 2) tma_load_2d_pair_by(issue, stage + Cfg::W_BYTES, &map_w, kx, n_out + my_feat, bar0);
          tma_load_2d_pair_by(issue, stage + NACC * Cfg::W_BYTES, &map_a, kx, my_tok, bar0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: warp 1 of the first block runs the loop, its lane 0 issues for the pair
    if (leader && pair < n_items) {
      const uint32_t issue = lane == 0 ? 1u : 0u;
      const uint32_t idesc = umma_idesc(ab_dtype, BT, 2 * TC_BM);
      bool ok = true;
      int it = 0, part = 0;
      for (int t = pair; t < n_items && ok; t += n_pairs, ++part) {
        const int buf = part & 1;
        const int k_lo = SPLIT ? (t / n_tiles) * k_per : 0, k_hi = SPLIT ? min(nkb, k_lo + k_per) : nkb;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&acc_empty[buf]), (((uint32_t)part >> 1) & 1u) ^ 1u, abort_p));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc_addr = tmem_base + (uint32_t)(buf * Cfg::ACC_STRIDE);
        for (int kb = k_lo; kb < k_hi && ok; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t phase = (it / Cfg::STAGES) & 1;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s]), phase, abort_p));
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t stage = tiles_smem + s * Cfg::STAGE_BYTES;
          const uint64_t wdesc = umma_desc_k_sw128(stage);
          const uint64_t adesc = umma_desc_k_sw128(stage + NACC * Cfg::W_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
            const uint32_t acc = (kb > k_lo || k > 0) ? 1u : 0u;
            const uint64_t koff = (uint64_t)((k * TC_UMMA_K * 2) >> 4);
            umma_f16_pair_by(issue, acc_addr, wdesc + koff, adesc + koff, idesc, acc);
            if (NACC == 2) {
              const uint64_t w2 = umma_desc_k_sw128(stage + Cfg::W_BYTES);
              umma_f16_pair_by(issue, acc_addr + BT, w2 + koff, adesc + koff, idesc, acc);
            }
          }
          umma_commit_pair_by(issue, smem_u32(&empty_bar[s]));           // frees the stage in both blocks
        }
        if (ok) umma_commit_pair_by(issue, smem_u32(&acc_full[buf]));    // both blocks' epilogues may read
      }
    }
  } else {
    // ---------------- epilogue warps of both blocks: this block's 128 features
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    bool ok = true;
    int part = 0, stage_it = 0;
    pdl_wait();
    for (int t = pair; t < n_items && ok; t += n_pairs, ++part) {
      const int buf = part & 1;
      int feat0, tok0, kb_lo, kb_hi;
      const int slice = item_of(t, feat0, tok0, kb_lo, kb_hi);
      const int f = feat0 + (int)rank * TC_BM + row;
      mbar_wait(smem_u32(&acc_full[buf]), ((uint32_t)part >> 1) & 1u, abort_p);
      asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
      if (*abort_p) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                             (uint32_t)(buf * Cfg::ACC_STRIDE);
      const int ncols = min(BT, M - tok0);
      if (NACC == 1 && mode == 5) {
        // ---- rotary encoding and cache write on the way out (rows are q, k, v heads)
        for (int j = row; j < ncols; j += SK_EPI_THREADS) {
          const int tok = tok0 + j;
          const int b = rope.token_seq[tok];
          const int slot = rope.seq_slot[b];
          const int qs = rope.q_start[b], qe = rope.q_start[b + 1];
          const int past = rope.slot_pos[slot];
          const int pos = past + (tok - qs);
          const bool keep = rope.write_cache && pos >= past + (qe - qs) - rope.capacity;
          const int r = pos % rope.capacity;
          rope_row[j] = keep ? r : -1;
          rope_where[j] = rope.page_table ? rope.page_table[(size_t)slot * rope.pages_per_slot + r / KV_PAGE]
                                          : slot;
        }
        const int hd = rope.hd, half = hd >> 1, H = rope.H, G = rope.G;
        const bool live = f < N;
        const int head = live ? f / hd : 0, i = live ? f - head * hd : 0;
        const bool upper = i >= half, rotates = head < H + G;
        const int partner = upper ? row - half : row + half;
        // cosine and sine of (token, pair) come from a table made once per step for all layers
        const float2* cs_col = reinterpret_cast<const float2*>(rope.cos_sin) + (upper ? i - half : i);
        asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
        // A chunk's cosines and sines are asked for one chunk ahead: their round trip to L2
        // then runs under the previous chunk's exchange and stores (asked for in the chunk
        // itself, fifteen such round trips per tile made this epilogue longer than the next
        // tile's main loop).
        auto load_cs = [&](int c0, float2* cs) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            cs[j] = (live && rotates && c0 + j < ncols)
                        ? __ldg(cs_col + (size_t)(tok0 + c0 + j) * half) : make_float2(1.f, 0.f);
        };
        float2 cs[16], cs_next[16];
        load_cs(0, cs);
#pragma unroll 1
        for (int c0 = 0; c0 < ncols; c0 += 16) {
          float v[16];
          tmem_ld16(taddr + c0, v);
          load_cs(c0 + 16, cs_next);                          // nothing is loaded past the tile's last column
#pragma unroll
          for (int j = 0; j < 16; ++j) rope_ex[row][j] = v[j];
          asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
          if (live) {
            if (rotates) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float o = rope_ex[partner][j];
                v[j] = upper ? rotate_hi(o, v[j], cs[j].x, cs[j].y) : rotate_lo(v[j], o, cs[j].x, cs[j].y);
              }
            }
          }
          // token-major in shared memory, so that a thread stores 16 features of one token
          // (32 bytes) instead of one feature of 16 tokens
#pragma unroll
          for (int j = 0; j < 16; ++j) rope_out[j][row] = bits16_rt(ab_dtype, v[j]);
          asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
          {
            const int j = row >> 3, fl = (row & 7) * 16;        // this thread's token and features
            const int f0 = feat0 + (int)rank * TC_BM + fl;
            if (c0 + j < ncols && f0 < N) {
              const int tok = tok0 + c0 + j;
              const int head0 = f0 / hd, i0 = f0 - head0 * hd;
              const uint4 lo = *reinterpret_cast<const uint4*>(&rope_out[j][fl]);
              const uint4 hi = *reinterpret_cast<const uint4*>(&rope_out[j][fl + 8]);
              uint16_t* dst;
              if (head0 < H) {
                dst = reinterpret_cast<uint16_t*>(rope.q_out) + (size_t)tok * H * hd + f0;
              } else {
                const bool v_row = head0 >= H + G;
                const int g0 = head0 - H - (v_row ? G : 0);
                dst = reinterpret_cast<uint16_t*>(rope.kv_step) +
                      ((size_t)tok * 2 * G + (v_row ? G : 0) + g0) * hd + i0;
                const int r = rope_row[c0 + j];
                if (r >= 0) {
                  const int w = rope_where[c0 + j];
                  const size_t at = rope.page_table
                      ? (((size_t)g0 * rope.n_pages + w) * KV_PAGE + (r % KV_PAGE)) * hd + i0
                      : (((size_t)w * G + g0) * rope.capacity + r) * hd + i0;
                  uint16_t* c = reinterpret_cast<uint16_t*>(v_row ? rope.v_cache : rope.k_cache) + at;
                  reinterpret_cast<uint4*>(c)[0] = lo;
                  reinterpret_cast<uint4*>(c)[1] = hi;
                }
              }
              reinterpret_cast<uint4*>(dst)[0] = lo;
              reinterpret_cast<uint4*>(dst)[1] = hi;
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) cs[j] = cs_next[j];
          asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
        }
      } else if (NACC == 1 && out_tma && mode == 4) {
        // ---- SiLU(gate).up of interleaved rows, stored through TMA: the block's 128 rows are
        // 64 output features; a chunk goes token-major ([16][64] of the 16-bit type) into one
        // of two staging buffers (see the store below)
        const int x = (feat0 + (int)rank * TC_BM) >> 1;
        const bool issuer = row == 0 && x < (N >> 1);
#pragma unroll 1
        for (int c0 = 0; c0 < ncols; c0 += 16, ++stage_it) {
          float v[16];
          tmem_ld16(taddr + c0, v);
          float r[8];
          silu_pairs_of_chunk(v, lane, r);
          const uint32_t st = smem_u32(epi_smem) + (uint32_t)((stage_it & 1) * 16 * 64 * 2);
          if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
          const uint32_t mine = st + (uint32_t)(((lane < 16 ? 0 : 8) * 64 + quarter * 16 + (lane & 15)) * 2);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(mine + (uint32_t)(j * 64 * 2)),
                         "h"(bits16_rt(out_dtype, r[j])) : "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
          if (issuer) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(reinterpret_cast<uint64_t>(&map_out)), "r"(st), "r"(x), "r"(tok0 + c0) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      } else if (NACC == 1 && out_tma && mode <= 1) {
        // ---- store (mode 0) or add into float32 out (mode 1) through TMA: a chunk of 16
        // tokens goes token-major into one of two staging buffers and one thread hands it
        // to the copy engine (one store per thread and column instead, 64-128 bytes per
        // warp instruction, kept a tile's last epilogue 5-6 us long; tokens beyond M are
        // clipped by the tensor map)
        const int x = feat0 + (int)rank * TC_BM;
        const bool issuer = row == 0 && x < n_out;           // (a block whose features lie beyond N copies nothing)
        const int esz = out_dtype == DT_F32 ? 4 : 2;
#pragma unroll 1
        for (int c0 = 0; c0 < ncols; c0 += 16, ++stage_it) {
          float v[16];
          tmem_ld16(taddr + c0, v);
          const uint32_t st = smem_u32(epi_smem) + (uint32_t)((stage_it & 1) * 16 * TC_BM * esz);
          // the copy that read this buffer two chunks ago has read it
          if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
          if (out_dtype == DT_F32) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              asm volatile("st.shared.f32 [%0], %1;" ::"r"(st + (uint32_t)((j * TC_BM + row) * 4)), "f"(v[j]) : "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              asm volatile("st.shared.u16 [%0], %1;" ::"r"(st + (uint32_t)((j * TC_BM + row) * 2)),
                           "h"(bits16_rt(out_dtype, v[j])) : "memory");
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 1, %0;" ::"n"(SK_EPI_THREADS) : "memory");
          if (issuer) {
            if (mode == 1)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(reinterpret_cast<uint64_t>(&map_out)), "r"(st), "r"(x), "r"(tok0 + c0) : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(reinterpret_cast<uint64_t>(&map_out)), "r"(st), "r"(x), "r"(tok0 + c0) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      } else
#pragma unroll 1
      for (int c0 = 0; c0 < ncols; c0 += 16) {
        float v[16];
        tmem_ld16(taddr + c0, v);
        if (NACC == 2) {
          float g2[16];
          tmem_ld16(taddr + BT + c0, g2);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu_times_fast(v[j], g2[j]);
        }
        if (mode == 4) {
          // rows interleaved in groups of 16: gate and up of a feature in lanes l and l + 16
          float r[8];
          silu_pairs_of_chunk(v, lane, r);
          const int fo = ((feat0 + (int)rank * TC_BM) >> 1) + quarter * 16 + (lane & 15);
          if (fo < (N >> 1))
            store_eight_tokens(out_dtype, out, r, fo, tok0 + c0 + (lane < 16 ? 0 : 8), M, N >> 1);
        } else if (SPLIT && mode == 3) {
          // this slice's 32-bit partial sums, [slice, M, N]
          sk_store_chunk(0, DT_F32, reinterpret_cast<float*>(out) + (size_t)slice * M * n_out, v, f,
                         tok0 + c0, M, n_out);
        } else {
          sk_store_chunk(mode, out_dtype, out, v, f, tok0 + c0, M, n_out);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty[buf]), 0));
    }
    // the copies this thread handed to the copy engine are done before the block ends
    if (row == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) atomicOr(status, ERR_WAIT_TIMEOUT);
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();                  // nobody touches the peer's barriers or TMEM after this
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
  }
}

template <int BT, int NACC, bool SPLIT = false>
static int launch_2sm(const void* A, const void* W, void* out, int out_dtype, int ab_dtype, int M,
                      int N, int K, int mode, int splits, int* status, cudaStream_t stream,
                      const yalm_rope_args& rope) {
  using Cfg = G2Cfg<BT, NACC>;
  static_assert(Cfg::STAGES >= 3, "pipeline depth");
  CUtensorMap mw, ma, mo;
  int rc = make_map(&mw, W, N, K, TC_BM, ab_dtype);
  if (rc) return rc;
  rc = make_map(&ma, A, M, K, BT / 2, ab_dtype);
  if (rc) return rc;
  // stores and residual adds of whole rows go through TMA where its rules allow (a 16-byte
  // aligned base and row pitch); else, and for the other epilogues, threads store
  int out_tma = 0;
  mo = ma;
  if (NACC == 1 && mode <= 1 && out != nullptr) {
    const int esz = out_dtype == DT_F32 ? 4 : 2;
    if (((uintptr_t)out & 15) == 0 && ((long long)N * esz) % 16 == 0 &&
        make_out_map(&mo, out, M, N, out_dtype, TC_BM) == 0)
      out_tma = 1;
  } else if (NACC == 1 && mode == 4 && out != nullptr && out_dtype != DT_F32) {
    if (((uintptr_t)out & 15) == 0 && ((long long)(N / 2) * 2) % 16 == 0 &&
        make_out_map(&mo, out, M, N / 2, out_dtype, TC_BM / 2) == 0)
      out_tma = 1;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_2sm_kernel<BT, NACC, SPLIT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int n_out = mode == 2 ? N / 2 : N;
  const long long tiles = (long long)((n_out + 2 * TC_BM - 1) / (2 * TC_BM)) * ((M + BT - 1) / BT);
  long long pairs = sm_count() / 2;
  if (pairs > tiles * splits) pairs = tiles * splits;
  if (pairs < 1) return -4;
  launch_pdl(gemm_2sm_kernel<BT, NACC, SPLIT>, dim3((unsigned)(2 * pairs)), dim3(TC_THREADS), Cfg::SMEM,
             stream, mw, ma, mo, out_tma, out, out_dtype, ab_dtype, M, N, K, mode, splits, status, rope);
  YALM_LAUNCH_CHECK();
  return 0;
}

// The pair's token tile, 256 or 240: the one whose waves of tiles over the SM pairs cost
// less (waves x tile width).  At 2,048 tokens a 4,096-feature product is 128 tiles of 256
// tokens on 74 pairs (two waves, the second 73 % full) or 144 tiles of 240 (two fuller,
// shorter waves: 6 % less time); a 28,672-feature product stays with 256.
static int two_sm_token_tile(int M, int n_out, int splits) {
  const long long pairs = sm_count() / 2 > 0 ? sm_count() / 2 : 1;
  const long long feats = (n_out + 2 * TC_BM - 1) / (2 * TC_BM);
  long long best = 0;
  int best_bt = 256;
  for (int bt : {256, 240}) {
    const long long tiles = feats * ((M + bt - 1) / bt) * splits;
    const long long cost = ((tiles + pairs - 1) / pairs) * bt;
    if (best == 0 || cost < best) {
      best = cost;
      best_bt = bt;
    }
  }
  return best_bt;
}

}  // namespace yalm

using namespace yalm;

extern "C" int yalm_gemm_tc_available(void) { return encode_fn() ? 0 : -10; }

extern "C" int yalm_gemm_tc(const void* A, const void* W, int ab_dtype, void* out, int out_dtype,
                            int M, int N, int K, int mode, int splits, int* status,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (ab_dtype != DT_BF16 && ab_dtype != DT_F16) return -3;
  if (out_dtype != DT_F32 && out_dtype != ab_dtype) return -3;
  if (K <= 0 || K % 8 != 0) return -2;               // TMA: rows must be 16-byte multiples
  if (((uintptr_t)A | (uintptr_t)W) & 15) return -6; // TMA: 16-byte aligned bases
  if (mode < 0 || mode > 4) return -3;
  if (mode == 2 && (N % 2 != 0)) return -3;
  if (mode == 4 && (N % 32 != 0)) return -3;
  if ((mode == 1 || mode == 3) && out_dtype != DT_F32) return -3;
  const int nkb = (K + TC_BK - 1) / TC_BK;
  if (mode != 3) splits = 1;
  if (splits < 1 || splits > nkb) return -5;
  {
    const int per = (nkb + splits - 1) / splits;
    if ((splits - 1) * per >= nkb) return -5;        // no empty slice of K
  }
  CUtensorMap mw;
  int rc = make_map(&mw, W, N, K, TC_BM, ab_dtype);
  if (rc) return rc;
#define YALM_TC(BT, NACC) \
  return launch_tc<BT, NACC>(mw, A, out, out_dtype, ab_dtype, M, N, K, mode, splits, status, stream)
  if (mode == 2) {
    if (M <= 16) YALM_TC(16, 2);
    if (M <= 32) YALM_TC(32, 2);
    if (M <= 64) YALM_TC(64, 2);
    if (M <= 128) YALM_TC(128, 2);
    YALM_TC(256, 2);
  }
  if (M <= 16) YALM_TC(16, 1);
  if (M <= 32) YALM_TC(32, 1);
  if (M <= 64) YALM_TC(64, 1);
  if (M <= 128) YALM_TC(128, 1);
  YALM_TC(256, 1);
#undef YALM_TC
}

// Two-SM variant for many tokens (see gemm_2sm_kernel): mode 0 store, 1 add into
// float32 out, 2 silu(gate)*up, 4 the same with interleaved rows, 3 `splits` slices of K as
// 32-bit partial sums [splits, M, N] (for token counts whose tiles leave SM pairs idle).
extern "C" int yalm_gemm_2sm(const void* A, const void* W, int ab_dtype, void* out, int out_dtype,
                             int M, int N, int K, int mode, int splits, int* status,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (ab_dtype != DT_BF16 && ab_dtype != DT_F16) return -3;
  if (out_dtype != DT_F32 && out_dtype != ab_dtype) return -3;
  if (K <= 0 || K % 8 != 0) return -2;
  if (((uintptr_t)A | (uintptr_t)W) & 15) return -6;
  if (mode < 0 || mode > 4) return -3;
  if (mode == 2 && (N % 2 != 0)) return -3;
  if (mode == 4 && (N % 32 != 0)) return -3;
  if ((mode == 1 || mode == 3) && out_dtype != DT_F32) return -3;
  if (mode != 3) splits = 1;
  {
    const int nkb = (K + TC_BK - 1) / TC_BK;
    if (splits < 1 || splits > nkb) return -5;
    const int per = (nkb + splits - 1) / splits;
    if ((splits - 1) * per >= nkb) return -5;        // no empty slice of K
  }
  yalm_rope_args none = {};
  if (mode == 2)
    return launch_2sm<128, 2>(A, W, out, out_dtype, ab_dtype, M, N, K, mode, 1, status, stream, none);
  if (mode == 3) {
    if (two_sm_token_tile(M, N, splits) == 240)
      return launch_2sm<240, 1, true>(A, W, out, out_dtype, ab_dtype, M, N, K, mode, splits, status, stream, none);
    return launch_2sm<256, 1, true>(A, W, out, out_dtype, ab_dtype, M, N, K, mode, splits, status, stream, none);
  }
  if (two_sm_token_tile(M, N, 1) == 240)
    return launch_2sm<240, 1>(A, W, out, out_dtype, ab_dtype, M, N, K, mode, 1, status, stream, none);
  return launch_2sm<256, 1>(A, W, out, out_dtype, ab_dtype, M, N, K, mode, 1, status, stream, none);
}

// The token tile that yalm_gemm_2sm takes for these sizes (256 or 240): callers that plan a
// split of K weigh it against the tiles this gives.
extern "C" int yalm_gemm_2sm_token_tile(int M, int N, int splits) {
  return two_sm_token_tile(M, N, splits < 1 ? 1 : splits);
}

// The q/k/v product of a prompt with the rotary encoding and the cache write in its
// epilogue: W's rows are the q heads, then the k heads, then the v heads; nothing but
// rotated q (q_out), this step's keys and values (kv_step) and the cache rows is written.
extern "C" int yalm_gemm_2sm_rope(const void* A, const void* W, int ab_dtype, int M, int N, int K,
                                  const yalm_rope_args* rope, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (rope == nullptr) return -3;
  if (ab_dtype != DT_BF16 && ab_dtype != DT_F16) return -3;
  if (K <= 0 || K % 8 != 0) return -2;
  if (((uintptr_t)A | (uintptr_t)W) & 15) return -6;
  const int hd = rope->hd;
  if (hd <= 0 || hd % 2 != 0 || TC_BM % hd != 0) return -2;        // a block's 128 rows hold whole heads
  if (N != (rope->H + 2 * rope->G) * hd || rope->capacity <= 0) return -2;
  if (!rope->cos_sin || !rope->token_seq || !rope->q_start || !rope->seq_slot || !rope->slot_pos ||
      !rope->q_out || !rope->kv_step || !rope->k_cache || !rope->v_cache)
    return -3;
  if (two_sm_token_tile(M, N, 1) == 240)
    return launch_2sm<240, 1>(A, W, nullptr, ab_dtype, ab_dtype, M, N, K, 5, 1, status, stream, *rope);
  return launch_2sm<256, 1>(A, W, nullptr, ab_dtype, ab_dtype, M, N, K, 5, 1, status, stream, *rope);
}
