// Row-wise kernels of the step: embedding gather, RMSNorm (with the residual
// sum of pending split-K partials folded in), SiLU(gate)*up, rotary position
// encoding fused with the cache write, and the position advance.
//
// Reference counterparts (plain SIMT kernels for one token of one sequence):
// copy_embedding_* infer.cu:636-658, rmsnorm infer.cu:525-539,
// fused_rope_and_cache_update infer.cu:660-705, act<SILU> infer.cu:601-604.
// Here every kernel takes a ragged batch of tokens and reads each sequence's
// position from the cache's per-slot state on the device.
#include <type_traits>

#include "api.h"
#include "common.cuh"

namespace yalm {

int g_pdl_enabled = 1;

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ x, int dim, int vocab, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, ERR_TOKEN_RANGE);
    tok = tok < 0 ? 0 : vocab - 1;
  }
  const T* row = table + (size_t)tok * dim;
  float* out = x + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] = to_float(row[i]);
}

// ------------------------------------------------------------------ rmsnorm
// One block per output row.  v = x[src] + sum_s partial[s][src]; the sum is
// written back to x when there are partials and no row gather (it is the
// residual stream's new value).  out = v * (1/sqrt(mean(v^2)+eps)) * w.
template <typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ partials,
                               int n_partials, long long partial_stride,
                               const int* __restrict__ rows, const float* __restrict__ weight,
                               TO* __restrict__ out, int dim, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * dim;
  const bool write_back = n_partials > 0 && rows == nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = xr[i];
    for (int s = 0; s < n_partials; ++s)
      v += partials[(size_t)s * partial_stride + (size_t)src * dim + i];
    if (write_back) xr[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* o = out + (size_t)r * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = xr[i];
    if (n_partials > 0 && !write_back)
      for (int s = 0; s < n_partials; ++s)
        v += partials[(size_t)s * partial_stride + (size_t)src * dim + i];
    o[i] = from_float<TO>(v * scale * weight[i]);
  }
}

// The same with the row held in registers as VPT float4 vectors per thread:
// every load of a pass is in flight at once, which is what a decode step's
// handful of rows needs (the kernel is a chain of memory round trips).
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <typename T16>
__device__ __forceinline__ void store4(T16* p, float4 v) {
  uint2 u;
  u.x = pack2<T16>(v.x, v.y);
  u.y = pack2<T16>(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TO, int VPT>
__global__ void __launch_bounds__(VPT <= 2 ? 1024 : 512)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ partials,
                   int n_partials, long long partial_stride,
                   const int* __restrict__ rows, const float* __restrict__ weight,
                   TO* __restrict__ out, int dim, float eps) {
  pdl_launch_dependents();
  const int nvec = dim >> 2;
  // the norm's weights do not depend on the previous kernel
  float4 w[VPT];
  {
    const float4* wr = reinterpret_cast<const float4*>(weight);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      w[k] = c < nvec ? wr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float4* xr = reinterpret_cast<float4*>(x + (size_t)src * dim);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    v[k] = c < nvec ? xr[c] : zero;
  }
  // several slices at a time, so that their loads are in flight together: a decode
  // step's row (one or two vectors per thread) takes up to eight slices in one round trip
  constexpr int SB = VPT <= 2 ? 8 : 4;
  for (int s0 = 0; s0 < n_partials; s0 += SB) {
    float4 p[SB][VPT];
#pragma unroll
    for (int j = 0; j < SB; ++j) {
      const float4* pr = reinterpret_cast<const float4*>(
          partials + (size_t)(s0 + j) * partial_stride + (size_t)src * dim);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        p[j][k] = (s0 + j < n_partials && c < nvec) ? pr[c] : zero;
      }
    }
#pragma unroll
    for (int j = 0; j < SB; ++j)
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        v[k].x += p[j][k].x; v[k].y += p[j][k].y; v[k].z += p[j][k].z; v[k].w += p[j][k].w;
      }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (n_partials > 0 && rows == nullptr && c < nvec) xr[c] = v[k];
    ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* o = out + (size_t)r * dim;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < nvec)
      store4(o + 4 * c, make_float4(v[k].x * scale * w[k].x, v[k].y * scale * w[k].y,
                                    v[k].z * scale * w[k].z, v[k].w * scale * w[k].w));
  }
}

// ---------------------------------------------------------------- silu * up
// gu: [rows, 2F] in 32-bit, possibly as n_partials split-K slices.  Columns are
// (gate | up), or with `paired` groups of 16 gate columns each followed by the 16
// up columns of the same features.
template <typename TO>
__global__ void silu_mul_kernel(const float* __restrict__ gu, int n_partials,
                                long long partial_stride, TO* __restrict__ out, int rows, int F,
                                int paired) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)rows * F;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / F, f = idx % F;
    const size_t gc = paired ? (f >> 4) * 32 + (f & 15) : f;
    const size_t uc = paired ? gc + 16 : F + f;
    float g = 0.f, u = 0.f;
    for (int s = 0; s < n_partials; ++s) {
      const float* p = gu + (size_t)s * partial_stride + r * 2 * F;
      g += p[gc];
      u += p[uc];
    }
    // the 16-bit paths round the result anyway: the same approximations as the products' epilogues
    if (std::is_same<TO, float>::value) out[idx] = from_float<TO>(g / (1.0f + expf(-g)) * u);
    else out[idx] = from_float<TO>(silu_times_fast(g, u));
  }
}

// ------------------------------------------------- rotary + cache write
// One block per (token, group of heads); one thread per (head, VEC rotary pairs).
// qkv: [N, (H+2G)*hd] in 32-bit (n_partials slices are summed).  Pair
// (i, i+hd/2) of every q and k head is rotated by the angle pos * inv_freq[i],
// all in 32-bit.  Rotated q goes to q_out [N, H*hd]; rotated k and plain v go
// to kv_step [N, 2, G, hd] (this step's keys and values in token order) and,
// for the positions that the ring keeps, to the cache [slots, G, capacity, hd]
// at row pos % capacity.  VEC = 4 when hd/2 is a multiple of 4 (16-byte loads,
// 8- or 16-byte stores), else 1.
template <typename T, int VEC> struct RopeIO;
template <> struct RopeIO<float, 4> {
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct RopeIO<__nv_bfloat16, 4> {
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    store4(p, make_float4(v[0], v[1], v[2], v[3]));
  }
};
template <> struct RopeIO<__half, 4> {
  static __device__ __forceinline__ void store(__half* p, const float* v) {
    store4(p, make_float4(v[0], v[1], v[2], v[3]));
  }
};
template <typename T> struct RopeIO<T, 1> {
  static __device__ __forceinline__ void store(T* p, const float* v) { p[0] = from_float<T>(v[0]); }
};

// Rotation of one thread's pairs (q and k heads only) and the stores that follow.
template <typename T, int VEC>
__device__ __forceinline__ void rope_rotate_store(float* a, float* bb, const float* fr, int t, int head,
                                                  int i, int pos, bool keep, int slot,
                                                  T* __restrict__ q_out, T* __restrict__ kv_step,
                                                  T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                  int H, int G, int hd, size_t cache_row) {
  const int half = hd >> 1;
  if (head < H + G) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const float ang = (float)pos * fr[v];
      const float c = cosf(ang), s = sinf(ang);
      const float r0 = rotate_lo(a[v], bb[v], c, s), r1 = rotate_hi(a[v], bb[v], c, s);
      a[v] = r0;
      bb[v] = r1;
    }
  }
  if (head < H) {
    T* o = q_out + ((size_t)t * H + head) * hd + i;
    RopeIO<T, VEC>::store(o, a);
    RopeIO<T, VEC>::store(o + half, bb);
    return;
  }
  const bool is_v = head >= H + G;
  const int g = head - H - (is_v ? G : 0);
  T* o = kv_step + ((size_t)t * 2 * G + (is_v ? G : 0) + g) * hd + i;
  RopeIO<T, VEC>::store(o, a);
  RopeIO<T, VEC>::store(o + half, bb);
  if (keep) {
    T* c = (is_v ? v_cache : k_cache) + cache_row + i;
    RopeIO<T, VEC>::store(c, a);
    RopeIO<T, VEC>::store(c + half, bb);
  }
}

template <typename T, int VEC>
__global__ void rope_store_kernel(const float* __restrict__ qkv, int n_partials,
                                  long long partial_stride, const float* __restrict__ inv_freq,
                                  const int* __restrict__ token_seq, const int* __restrict__ q_start,
                                  const int* __restrict__ seq_slot, const int* __restrict__ slot_pos,
                                  T* __restrict__ q_out, T* __restrict__ kv_step,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int G,
                                  int hd, int capacity, int write_cache, int heads_per_block,
                                  const int* __restrict__ page_table, int pps, int n_pages) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int half = hd >> 1;
  const int lanes = half / VEC;                             // threads per head
  const int i = (threadIdx.x % lanes) * VEC;
  const int head = blockIdx.y * heads_per_block + threadIdx.x / lanes;
  // the batch's index arrays are written by host copies, never by a kernel: they may be
  // read while the previous kernel still runs; positions and the product may not
  const int b = token_seq[t];
  const int slot = seq_slot[b];
  const int qs = q_start[b];
  const int q_end = q_start[b + 1];
  float fr[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) fr[v] = inv_freq[i + v];
  const int past = slot_pos[slot];                        // written by the advance kernel alone (see there)
  const int pos = past + (t - qs);
  const int end = past + (q_end - qs);                     // positions after this step
  const bool keep = write_cache && pos >= end - capacity;
  // where the row goes in the cache (the page table too is written by host copies only)
  size_t cache_row = 0;
  if (keep && head >= H && head < H + 2 * G)
    cache_row = kv_row_offset(page_table, pps, n_pages, slot, (head - H) % G, G, capacity,
                              pos % capacity, hd);
  pdl_wait();
  if (head >= H + 2 * G) return;
  const int row_elems = (H + 2 * G) * hd;
  const float* sp = qkv + (size_t)t * row_elems + head * hd + i;
  float a[VEC], bb[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) { a[v] = 0.f; bb[v] = 0.f; }
  if (VEC == 4) {
    // eight slices at a time, so that their loads are in flight together
    constexpr int SB = 8;
    for (int p0 = 0; p0 < n_partials; p0 += SB) {
      float4 x[SB], y[SB];
#pragma unroll
      for (int j = 0; j < SB; ++j) {
        const float* pp = sp + (size_t)(p0 + j) * partial_stride;
        const bool live = p0 + j < n_partials;
        x[j] = live ? *reinterpret_cast<const float4*>(pp) : make_float4(0.f, 0.f, 0.f, 0.f);
        y[j] = live ? *reinterpret_cast<const float4*>(pp + half) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < SB; ++j) {
        a[0] += x[j].x; a[VEC > 1 ? 1 : 0] += x[j].y; a[VEC > 2 ? 2 : 0] += x[j].z; a[VEC > 3 ? 3 : 0] += x[j].w;
        bb[0] += y[j].x; bb[VEC > 1 ? 1 : 0] += y[j].y; bb[VEC > 2 ? 2 : 0] += y[j].z; bb[VEC > 3 ? 3 : 0] += y[j].w;
      }
    }
  } else {
    for (int p = 0; p < n_partials; ++p) {
      const float* pp = sp + (size_t)p * partial_stride;
      a[0] += pp[0];
      bb[0] += pp[half];
    }
  }
  rope_rotate_store<T, VEC>(a, bb, fr, t, head, i, pos, keep, slot, q_out, kv_step, k_cache, v_cache, H, G, hd,
                            cache_row);
}

// The same for many tokens whose product is a single slice (a prompt): a block takes
// TPB tokens, and the index chains and the loads of all of them are in flight together.
template <typename T, int TPB>
__global__ void rope_store_many_kernel(const float* __restrict__ qkv, const float* __restrict__ inv_freq,
                                       const int* __restrict__ token_seq, const int* __restrict__ q_start,
                                       const int* __restrict__ seq_slot, const int* __restrict__ slot_pos,
                                       T* __restrict__ q_out, T* __restrict__ kv_step,
                                       T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int G,
                                       int hd, int capacity, int write_cache, int heads_per_block,
                                       int n_tokens, const int* __restrict__ page_table, int pps, int n_pages) {
  pdl_launch_dependents();
  const int half = hd >> 1;
  const int lanes = half / 4;
  const int i = (threadIdx.x % lanes) * 4;
  const int head = blockIdx.y * heads_per_block + threadIdx.x / lanes;
  const int t0 = blockIdx.x * TPB;
  int b[TPB], slot[TPB], qs[TPB], qe[TPB];
#pragma unroll
  for (int k = 0; k < TPB; ++k) b[k] = token_seq[min(t0 + k, n_tokens - 1)];
#pragma unroll
  for (int k = 0; k < TPB; ++k) {
    slot[k] = seq_slot[b[k]];
    qs[k] = q_start[b[k]];
    qe[k] = q_start[b[k] + 1];
  }
  float fr[4];
#pragma unroll
  for (int v = 0; v < 4; ++v) fr[v] = inv_freq[i + v];
  int past[TPB];
#pragma unroll
  for (int k = 0; k < TPB; ++k) past[k] = slot_pos[slot[k]];
  pdl_wait();
  if (head >= H + 2 * G) return;
  const int row_elems = (H + 2 * G) * hd;
  float4 x[TPB], y[TPB];
#pragma unroll
  for (int k = 0; k < TPB; ++k) {
    const float* sp = qkv + (size_t)min(t0 + k, n_tokens - 1) * row_elems + head * hd + i;
    x[k] = *reinterpret_cast<const float4*>(sp);
    y[k] = *reinterpret_cast<const float4*>(sp + half);
  }
#pragma unroll
  for (int k = 0; k < TPB; ++k) {
    const int t = t0 + k;
    if (t >= n_tokens) break;
    const int pos = past[k] + (t - qs[k]);
    const int end = past[k] + (qe[k] - qs[k]);
    const bool keep = write_cache && pos >= end - capacity;
    float a[4] = {x[k].x, x[k].y, x[k].z, x[k].w}, bb[4] = {y[k].x, y[k].y, y[k].z, y[k].w};
    size_t cache_row = 0;
    if (keep && head >= H)
      cache_row = kv_row_offset(page_table, pps, n_pages, slot[k], (head - H) % G, G, capacity,
                                pos % capacity, hd);
    rope_rotate_store<T, 4>(a, bb, fr, t, head, i, pos, keep, slot[k], q_out, kv_step, k_cache, v_cache, H, G,
                            hd, cache_row);
  }
}

// cos_sin[t][i] = (cos, sin)(pos(t) * inv_freq[i]) with the angle in 32 bits, exactly as
// rope_store_kernel computes it: the table a product with a rotary epilogue reads.
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ token_seq,
                                  const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                  const int* __restrict__ slot_pos, float2* __restrict__ cos_sin,
                                  int n_tokens, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const int pos = slot_pos[seq_slot[b]] + (t - q_start[b]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float ang = (float)pos * inv_freq[i];
    cos_sin[(size_t)t * half + i] = make_float2(cosf(ang), sinf(ang));
  }
}

// ------------------------------------------------- ring rows from the step's buffer
// Copies this step's keys and values (kv_step [N, 2, G, hd], already rotated) into
// the cache ring for the positions the ring keeps: what rope_store does on the way
// when it may write at once.  Used when the ring may only be written after the
// attention (several tokens on top of a ring that already wrapped).  One block per
// token; 16-byte copies when rows allow it.
template <typename T>
__global__ void cache_write_kernel(const T* __restrict__ kv_step, const int* __restrict__ token_seq,
                                   const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                                   const int* __restrict__ slot_pos, T* __restrict__ k_cache,
                                   T* __restrict__ v_cache, int G, int hd, int capacity, int vec,
                                   const int* __restrict__ page_table, int pps, int n_pages) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const int slot = seq_slot[b];
  const int qs = q_start[b], q_end = q_start[b + 1];
  const int past = slot_pos[slot];
  const int pos = past + (t - qs);
  if (pos < past + (q_end - qs) - capacity) return;          // the ring keeps only the last rows
  const int row = pos % capacity;
  const T* src = kv_step + (size_t)t * 2 * G * hd;
  if (vec) {
    constexpr int E = 16 / sizeof(T);
    const int per_head = hd / E;
    for (int i = threadIdx.x; i < 2 * G * per_head; i += blockDim.x) {
      const int kv = i / (G * per_head), g = (i / per_head) % G, c = i % per_head;
      T* dst = (kv ? v_cache : k_cache) + kv_row_offset(page_table, pps, n_pages, slot, g, G, capacity, row, hd);
      reinterpret_cast<uint4*>(dst)[c] =
          reinterpret_cast<const uint4*>(src + ((size_t)kv * G + g) * hd)[c];
    }
  } else {
    for (int i = threadIdx.x; i < 2 * G * hd; i += blockDim.x) {
      const int kv = i / (G * hd), g = (i / hd) % G, c = i % hd;
      T* dst = (kv ? v_cache : k_cache) + kv_row_offset(page_table, pps, n_pages, slot, g, G, capacity, row, hd);
      dst[c] = src[((size_t)kv * G + g) * hd + c];
    }
  }
}

__global__ void advance_kernel(const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                               int* __restrict__ slot_pos, int n_seqs) {
  // No early start for what follows: this is the one kernel that writes the positions, and
  // other kernels read them before their own dependency wait.
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < n_seqs) slot_pos[seq_slot[b]] += q_start[b + 1] - q_start[b];
}

// The bounded wait of common.cuh on its own: one thread waits on a barrier that nobody
// arrives on, gives up after limit_ns, and raises ERR_WAIT_TIMEOUT in the status word,
// exactly as a kernel's role does when a copy or a product never completes.  It returns by
// itself; nothing is trapped and nothing waits without a limit.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int* __restrict__ status) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    volatile int* abort_p = &abort_flag;
    if (!mbar_wait(smem_u32(&bar), 0, abort_p, limit_ns)) atomicOr(status, ERR_WAIT_TIMEOUT);
  }
}

}  // namespace yalm

using namespace yalm;

// For tests of the status path: a kernel whose bounded wait runs out after limit_ns
// (at most 100 ms) and reports it in `status`.
extern "C" int yalm_wait_probe(unsigned long long limit_ns, int* status, cudaStream_t stream) {
  if (limit_ns == 0 || limit_ns > 100000000ull) return -2;
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_ns, status);
  YALM_LAUNCH_CHECK();
  return 0;
}

// Programmatic dependent launch on (1, the default) or off (0: every kernel starts
// only after the previous one has ended, as a plain stream launch does).
extern "C" int yalm_set_pdl(int on) {
  g_pdl_enabled = on ? 1 : 0;
  return 0;
}

// Host <-> device copies of a decode step's few tokens without a tensor library in
// between: `to_device` 1 copies host (pinned) to device, 0 device to host; both are
// asynchronous on the stream.  yalm_stream_wait blocks the host until the stream is idle.
extern "C" int yalm_copy_async(void* dst, const void* src, long long bytes, int to_device,
                               cudaStream_t stream) {
  if (bytes <= 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, (size_t)bytes,
                              to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, stream);
}
extern "C" int yalm_stream_wait(cudaStream_t stream) { return (int)cudaStreamSynchronize(stream); }

extern "C" int yalm_embed(const int* tokens, const void* table, int table_dtype, float* x,
                          int n_tokens, int dim, int vocab, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int threads = dim >= 1024 ? 256 : 128;
  if (table_dtype == DT_F32)
    launch_pdl(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table, x, dim,
                                                          vocab, status);
  else if (table_dtype == DT_BF16)
    launch_pdl(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream,
               tokens, (const __nv_bfloat16*)table, x, dim, vocab, status);
  else if (table_dtype == DT_F16)
    launch_pdl(embed_kernel<__half>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
               (const __half*)table, x, dim, vocab, status);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

template <typename TO>
static void launch_rmsnorm(float* x, const float* partials, int n_partials,
                           long long partial_stride, const int* rows, const float* weight, TO* out,
                           int n_rows, int dim, float eps, cudaStream_t stream) {
  const bool vec = dim % 4 == 0 && partial_stride % 4 == 0 &&
                   ((((uintptr_t)x) | ((uintptr_t)partials) | ((uintptr_t)weight) |
                     ((uintptr_t)out)) & 15) == 0;
  const int nvec = dim / 4;
  if (vec && nvec <= 8 * 512) {
    // A few rows (a decode step; up to 256, which is one wave of such blocks): few vectors
    // per thread, because the kernel is then a chain of memory round trips.  Many rows (a prompt): blocks of 256 threads with the
    // row in four vectors per thread stream at the memory's rate.
    int threads;
    if (n_rows <= 256) threads = nvec <= 1024 ? (nvec + 31) / 32 * 32 : (nvec <= 2048 ? 1024 : 512);
    else threads = nvec <= 128 ? 128 : (nvec <= 1024 ? 256 : 512);
    const int vpt = (nvec + threads - 1) / threads;
#define YALM_RMS(V)                                                                          \
  launch_pdl(rmsnorm_vec_kernel<TO, V>, dim3(n_rows), dim3(threads), 0, stream, x, partials, n_partials,          \
                                                           partial_stride, rows, weight, out, \
                                                           dim, eps)
    if (vpt <= 1) YALM_RMS(1);
    else if (vpt <= 2) YALM_RMS(2);
    else if (vpt <= 4) YALM_RMS(4);
    else YALM_RMS(8);
#undef YALM_RMS
    return;
  }
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  launch_pdl(rmsnorm_kernel<TO>, dim3(n_rows), dim3(threads), 0, stream, x, partials, n_partials, partial_stride, rows,
                                                     weight, out, dim, eps);
}

extern "C" int yalm_rmsnorm(float* x, const float* partials, int n_partials,
                            long long partial_stride, const int* rows, const float* weight,
                            void* out, int out_dtype, int n_rows, int dim, float eps,
                            cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (out_dtype == DT_F32)
    launch_rmsnorm<float>(x, partials, n_partials, partial_stride, rows, weight, (float*)out,
                          n_rows, dim, eps, stream);
  else if (out_dtype == DT_BF16)
    launch_rmsnorm<__nv_bfloat16>(x, partials, n_partials, partial_stride, rows, weight,
                                  (__nv_bfloat16*)out, n_rows, dim, eps, stream);
  else if (out_dtype == DT_F16)
    launch_rmsnorm<__half>(x, partials, n_partials, partial_stride, rows, weight, (__half*)out,
                           n_rows, dim, eps, stream);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_silu_mul(const float* gu, int n_partials, long long partial_stride, void* out,
                             int out_dtype, int rows, int F, int paired, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (paired && F % 16 != 0) return -2;
  const size_t total = (size_t)rows * F;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (out_dtype == DT_F32)
    launch_pdl(silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, gu, n_partials, partial_stride,
                                                               (float*)out, rows, F, paired);
  else if (out_dtype == DT_BF16)
    launch_pdl(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream,
               gu, n_partials, partial_stride, (__nv_bfloat16*)out, rows, F, paired);
  else if (out_dtype == DT_F16)
    launch_pdl(silu_mul_kernel<__half>, dim3((int)blocks), dim3(threads), 0, stream, gu,
               n_partials, partial_stride, (__half*)out, rows, F, paired);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_rope_store(const float* qkv, int n_partials, long long partial_stride,
                               const float* inv_freq, const int* token_seq, const int* q_start,
                               const int* seq_slot, const int* slot_pos, void* q_out,
                               void* kv_step, void* k_cache, void* v_cache, int dtype,
                               int n_tokens, int H, int G, int hd, int capacity, int write_cache,
                               const int* page_table, int pages_per_slot, int n_pages, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd % 2 != 0 || hd / 2 > 512 || hd <= 0) return -2;
  if (dtype != DT_F32 && dtype != DT_BF16 && dtype != DT_F16) return -3;
  const int half = hd / 2;
  const bool vec = half % 4 == 0 && partial_stride % 4 == 0 &&
                   ((((uintptr_t)qkv) | ((uintptr_t)q_out) | ((uintptr_t)kv_step) |
                     ((uintptr_t)k_cache) | ((uintptr_t)v_cache)) & 15) == 0;
  const int lanes = vec ? half / 4 : half;                  // threads per head
  int hpb = 512 / lanes;                                    // heads per block
  if (hpb > 16) hpb = 16;
  if (hpb < 1) hpb = 1;
  if (hpb > H + 2 * G) hpb = H + 2 * G;
  const dim3 grid(n_tokens, (H + 2 * G + hpb - 1) / hpb);
  const int threads = lanes * hpb;
  if (grid.y > 65535 || threads > 1024) return -4;
  if (vec && n_partials == 1 && n_tokens >= 512) {
    constexpr int TPB = 4;
    const dim3 grid4((n_tokens + TPB - 1) / TPB, grid.y);
    if (dtype == DT_F32)
      launch_pdl(rope_store_many_kernel<float, TPB>, grid4, dim3(threads), 0, stream, qkv, inv_freq, token_seq,
                 q_start, seq_slot, slot_pos, (float*)q_out, (float*)kv_step, (float*)k_cache, (float*)v_cache,
                 H, G, hd, capacity, write_cache, hpb, n_tokens, page_table, pages_per_slot, n_pages);
    else if (dtype == DT_BF16)
      launch_pdl(rope_store_many_kernel<__nv_bfloat16, TPB>, grid4, dim3(threads), 0, stream, qkv, inv_freq,
                 token_seq, q_start, seq_slot, slot_pos, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv_step,
                 (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, H, G, hd, capacity, write_cache, hpb,
                 n_tokens, page_table, pages_per_slot, n_pages);
    else
      launch_pdl(rope_store_many_kernel<__half, TPB>, grid4, dim3(threads), 0, stream, qkv, inv_freq,
                 token_seq, q_start, seq_slot, slot_pos, (__half*)q_out, (__half*)kv_step,
                 (__half*)k_cache, (__half*)v_cache, H, G, hd, capacity, write_cache, hpb, n_tokens,
                 page_table, pages_per_slot, n_pages);
    YALM_LAUNCH_CHECK();
    return 0;
  }
#define YALM_ROPE(T, V)                                                                        \
  launch_pdl(rope_store_kernel<T, V>, grid, dim3(threads), 0, stream, qkv, n_partials,         \
             partial_stride, inv_freq, token_seq, q_start, seq_slot, slot_pos, (T*)q_out,      \
             (T*)kv_step, (T*)k_cache, (T*)v_cache, H, G, hd, capacity, write_cache, hpb,      \
             page_table, pages_per_slot, n_pages)
  if (dtype == DT_F32) {
    if (vec) YALM_ROPE(float, 4); else YALM_ROPE(float, 1);
  } else if (dtype == DT_BF16) {
    if (vec) YALM_ROPE(__nv_bfloat16, 4); else YALM_ROPE(__nv_bfloat16, 1);
  } else {
    if (vec) YALM_ROPE(__half, 4); else YALM_ROPE(__half, 1);
  }
#undef YALM_ROPE
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_rope_table(const float* inv_freq, const int* token_seq, const int* q_start,
                               const int* seq_slot, const int* slot_pos, float* cos_sin,
                               int n_tokens, int half, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (half <= 0 || (((uintptr_t)cos_sin) & 7)) return -2;
  launch_pdl(rope_table_kernel, dim3(n_tokens), dim3(half >= 64 ? 64 : 32), 0, stream, inv_freq, token_seq,
             q_start, seq_slot, slot_pos, reinterpret_cast<float2*>(cos_sin), n_tokens, half);
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_cache_write(const void* kv_step, const int* token_seq, const int* q_start,
                                const int* seq_slot, const int* slot_pos, void* k_cache,
                                void* v_cache, int dtype, int n_tokens, int G, int hd,
                                int capacity, const int* page_table, int pages_per_slot, int n_pages,
                                cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (G <= 0 || hd <= 0 || capacity <= 0) return -2;
  const int esz = dtype == DT_F32 ? 4 : 2;
  const int vec = (hd * esz) % 16 == 0 &&
                  ((((uintptr_t)kv_step) | ((uintptr_t)k_cache) | ((uintptr_t)v_cache)) & 15) == 0;
  const dim3 grid(n_tokens), block(128);
  if (dtype == DT_F32)
    launch_pdl(cache_write_kernel<float>, grid, block, 0, stream, (const float*)kv_step, token_seq,
               q_start, seq_slot, slot_pos, (float*)k_cache, (float*)v_cache, G, hd, capacity, vec,
               page_table, pages_per_slot, n_pages);
  else if (dtype == DT_BF16 || dtype == DT_F16)          // 16-bit rows are copied as they are
    launch_pdl(cache_write_kernel<uint16_t>, grid, block, 0, stream, (const uint16_t*)kv_step,
               token_seq, q_start, seq_slot, slot_pos, (uint16_t*)k_cache, (uint16_t*)v_cache, G,
               hd, capacity, vec, page_table, pages_per_slot, n_pages);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_advance(const int* q_start, const int* seq_slot, int* slot_pos, int n_seqs,
                            cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  launch_pdl(advance_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, q_start, seq_slot, slot_pos, n_seqs);
  YALM_LAUNCH_CHECK();
  return 0;
}
