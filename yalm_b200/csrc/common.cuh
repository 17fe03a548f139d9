// Shared device helpers of the sm_100a kernels: storage types, conversions and
// block reductions.  Every kernel computes in 32-bit floats; only storage is
// bfloat16 or float16 on the 16-bit paths.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace yalm {

// dtype codes of the C interface
enum : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };

// error bits a kernel may set in the status word it is given
enum : int {
  ERR_TOKEN_RANGE = 1,    // a token id outside the vocabulary
  ERR_WAIT_TIMEOUT = 2,   // a bounded wait on a barrier gave up
  ERR_SLOT_RANGE = 4,     // a slot index outside the cache
  ERR_CONTEXT_RANGE = 8,  // a sequence longer than the bound the launch was sized for
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// Two floats rounded into one 32-bit word of the 16-bit type T (low half first).
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// The same with the type chosen at run time (dtype code DT_BF16 or DT_F16).
__device__ __forceinline__ uint32_t pack2_rt(int dtype, float lo, float hi) {
  return dtype == DT_F16 ? pack2<__half>(lo, hi) : pack2<__nv_bfloat16>(lo, hi);
}
__device__ __forceinline__ uint16_t bits16_rt(int dtype, float v) {
  return dtype == DT_F16 ? __half_as_ushort(__float2half_rn(v))
                         : __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void store16_rt(int dtype, void* base, size_t index, float v) {
  if (dtype == DT_F16) reinterpret_cast<__half*>(base)[index] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(v);
}

// silu(g) * u where the result is rounded to a 16-bit type: 2^x and the division are the
// special-function unit's approximations (relative error about 2^-22, far below that
// rounding); the float32 path keeps expf and the IEEE division.
__device__ __forceinline__ float silu_times_fast(float g, float u) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
  return __fdividef(g * u, 1.0f + e);
}
// The SiLU.up epilogue of a product whose weight rows come as 16 gate rows followed by the
// 16 up rows of the same features: of an accumulator chunk of 16 token columns, lane l < 16
// holds the gate and lane l + 16 the up value of feature l.  The halves swap eight columns
// each, so that every lane computes eight results: r[j] is token column j (lanes 0-15) or
// 8 + j (lanes 16-31) of feature lane & 15.
__device__ __forceinline__ void silu_pairs_of_chunk(const float* v, int lane, float* r) {
  const bool lo = lane < 16;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float got = __shfl_xor_sync(0xffffffffu, lo ? v[8 + j] : v[j], 16);
    r[j] = silu_times_fast(lo ? v[j] : got, lo ? got : v[8 + j]);
  }
}
// ... and its store: eight tokens from tok_first on (those below M) of feature f, row pitch n_out
__device__ __forceinline__ void store_eight_tokens(int out_dtype, void* __restrict__ out, const float* r,
                                                   int f, int tok_first, int M, int n_out) {
  if (out_dtype == DT_F32) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (tok_first + j < M) reinterpret_cast<float*>(out)[(size_t)(tok_first + j) * n_out + f] = r[j];
  } else if (out_dtype == DT_F16) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (tok_first + j < M)
        reinterpret_cast<__half*>(out)[(size_t)(tok_first + j) * n_out + f] = __float2half_rn(r[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (tok_first + j < M)
        reinterpret_cast<__nv_bfloat16*>(out)[(size_t)(tok_first + j) * n_out + f] = __float2bfloat16_rn(r[j]);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 33 floats of shared memory.  The order of additions depends only
// on the block size, never on the data or on other blocks.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---- the rotation of one pair ----------------------------------------------
// (a, b) -> (a c - b s, a s + b c) with the roundings spelled out, so that every kernel
// that rotates gives the same bits whatever the compiler would have fused.
__device__ __forceinline__ float rotate_lo(float a, float b, float c, float s) {
  return __fmaf_rn(a, c, -__fmul_rn(b, s));
}
__device__ __forceinline__ float rotate_hi(float a, float b, float c, float s) {
  return __fmaf_rn(a, s, __fmul_rn(b, c));
}

// ---- where a cached row lives --------------------------------------------
// The cache of one layer run is either contiguous per sequence,
// [slots][kv heads][capacity][head size], or made of pages of KV_PAGE positions,
// [kv heads][pages][KV_PAGE][head size], with a table [slots][pages_per_slot] that
// names the page of rows 64 p .. 64 p + 63 of each sequence (page_table != null).
// Row r is a position modulo the capacity in both.  With the kv head outermost the
// rows of one head in pages that follow one another are one run of memory, which is
// what a sequence that grew without interruption has.
constexpr int KV_PAGE = 64;
__device__ __forceinline__ size_t kv_row_offset(const int* __restrict__ page_table,
                                                int pages_per_slot, int n_pages, int slot, int g,
                                                int G, int capacity, int row, int hd) {
  if (page_table == nullptr) return (((size_t)slot * G + g) * capacity + row) * hd;
  const int page = page_table[(size_t)slot * pages_per_slot + (row / KV_PAGE)];
  return (((size_t)g * n_pages + page) * KV_PAGE + (row % KV_PAGE)) * hd;
}

// ---- shared-memory barriers with bounded waits --------------------------
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Bounded wait; false after the time limit or once another role has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long limit_ns = WAIT_LIMIT_NS) {
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 255u) == 255u) {
      if (*abort_flag) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) { *abort_flag = 1; return false; }
    }
  }
}
// Plain (untiled) bulk copy global -> shared; both addresses and the size are
// multiples of 16 bytes.  Completion is counted on the barrier in bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// ---- programmatic dependent launch ---------------------------------------
// Every kernel of the library is launched so that its blocks may start while
// the previous kernel of the stream is still draining.  A kernel first lets its
// own successor do the same (pdl_launch_dependents) and then waits until the
// previous kernel has completed and its writes are visible (pdl_wait) before it
// touches anything that kernel may have written or may still read.  Only data
// that no kernel of a step writes (weights) is read before the wait.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

extern int g_pdl_enabled;     // defined in elementwise.cu; yalm_set_pdl switches it

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace yalm

#define YALM_LAUNCH_CHECK()                         \
  do {                                              \
    cudaError_t e__ = cudaGetLastError();           \
    if (e__ != cudaSuccess) return (int)e__;        \
  } while (0)
