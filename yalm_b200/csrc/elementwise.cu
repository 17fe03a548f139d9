// Row-wise kernels of the step: embedding gather, RMSNorm (with the residual
// sum of pending split-K partials folded in), SiLU(gate)*up, rotary position
// encoding fused with the cache write, and the position advance.
//
// Reference counterparts (plain SIMT kernels for one token of one sequence):
// copy_embedding_* infer.cu:636-658, rmsnorm infer.cu:525-539,
// fused_rope_and_cache_update infer.cu:660-705, act<SILU> infer.cu:601-604.
// Here every kernel takes a ragged batch of tokens and reads each sequence's
// position from the cache's per-slot state on the device.
#include "api.h"
#include "common.cuh"

namespace yalm {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ x, int dim, int vocab, int* status) {
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

// ---------------------------------------------------------------- silu * up
// gu: [rows, 2F] (gate | up) in 32-bit, possibly as n_partials split-K slices.
template <typename TO>
__global__ void silu_mul_kernel(const float* __restrict__ gu, int n_partials,
                                long long partial_stride, TO* __restrict__ out, int rows, int F) {
  const size_t total = (size_t)rows * F;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / F, f = idx % F;
    float g = 0.f, u = 0.f;
    for (int s = 0; s < n_partials; ++s) {
      const float* p = gu + (size_t)s * partial_stride + r * 2 * F;
      g += p[f];
      u += p[F + f];
    }
    out[idx] = from_float<TO>(g / (1.0f + expf(-g)) * u);
  }
}

// ------------------------------------------------- rotary + cache write
// One block per token.  qkv: [N, (H+2G)*hd] in 32-bit (n_partials slices are
// summed).  Pair (i, i+hd/2) of every q and k head is rotated by the angle
// pos * inv_freq[i], all in 32-bit.  Rotated q goes to q_out [N, H*hd]; rotated
// k and plain v go to kv_step [N, 2, G, hd] (this step's keys and values in
// token order) and, for the positions that the ring keeps, to the cache
// [slots, G, capacity, hd] at row pos % capacity.
template <typename T>
__global__ void rope_store_kernel(const float* __restrict__ qkv, int n_partials,
                                  long long partial_stride, const float* __restrict__ inv_freq,
                                  const int* __restrict__ token_seq, const int* __restrict__ q_start,
                                  const int* __restrict__ seq_slot, const int* __restrict__ slot_pos,
                                  T* __restrict__ q_out, T* __restrict__ kv_step,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int G,
                                  int hd, int capacity, int write_cache) {
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const int slot = seq_slot[b];
  const int past = slot_pos[slot];
  const int pos = past + (t - q_start[b]);
  const int end = past + (q_start[b + 1] - q_start[b]);   // positions after this step
  const bool keep = write_cache && pos >= end - capacity;
  const int half = hd >> 1;
  const int i = threadIdx.x % half;
  const int group = threadIdx.x / half;
  const int ngroups = blockDim.x / half;
  if (group >= ngroups) return;
  const float ang = (float)pos * inv_freq[i];
  const float c = cosf(ang), s = sinf(ang);
  const int row_elems = (H + 2 * G) * hd;
  const float* src = qkv + (size_t)t * row_elems;
  const int ring = pos % capacity;
  for (int head = group; head < H + 2 * G; head += ngroups) {
    float a = 0.f, bb = 0.f;
    for (int p = 0; p < n_partials; ++p) {
      const float* sp = src + (size_t)p * partial_stride + head * hd;
      a += sp[i];
      bb += sp[i + half];
    }
    if (head < H) {
      T* o = q_out + (size_t)t * H * hd + head * hd;
      o[i] = from_float<T>(a * c - bb * s);
      o[i + half] = from_float<T>(a * s + bb * c);
    } else if (head < H + G) {
      const int g = head - H;
      const T r0 = from_float<T>(a * c - bb * s), r1 = from_float<T>(a * s + bb * c);
      T* o = kv_step + ((size_t)t * 2 * G + g) * hd;
      o[i] = r0;
      o[i + half] = r1;
      if (keep) {
        T* kc = k_cache + (((size_t)slot * G + g) * capacity + ring) * hd;
        kc[i] = r0;
        kc[i + half] = r1;
      }
    } else {
      const int g = head - H - G;
      const T r0 = from_float<T>(a), r1 = from_float<T>(bb);
      T* o = kv_step + ((size_t)t * 2 * G + G + g) * hd;
      o[i] = r0;
      o[i + half] = r1;
      if (keep) {
        T* vc = v_cache + (((size_t)slot * G + g) * capacity + ring) * hd;
        vc[i] = r0;
        vc[i + half] = r1;
      }
    }
  }
}

__global__ void advance_kernel(const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                               int* __restrict__ slot_pos, int n_seqs) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < n_seqs) slot_pos[seq_slot[b]] += q_start[b + 1] - q_start[b];
}

}  // namespace yalm

using namespace yalm;

extern "C" int yalm_embed(const int* tokens, const void* table, int table_dtype, float* x,
                          int n_tokens, int dim, int vocab, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int threads = dim >= 1024 ? 256 : 128;
  if (table_dtype == DT_F32)
    embed_kernel<float><<<n_tokens, threads, 0, stream>>>(tokens, (const float*)table, x, dim,
                                                          vocab, status);
  else
    embed_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        tokens, (const __nv_bfloat16*)table, x, dim, vocab, status);
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_rmsnorm(float* x, const float* partials, int n_partials,
                            long long partial_stride, const int* rows, const float* weight,
                            void* out, int out_dtype, int n_rows, int dim, float eps,
                            cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
  if (out_dtype == DT_F32)
    rmsnorm_kernel<float><<<n_rows, threads, 0, stream>>>(x, partials, n_partials, partial_stride,
                                                          rows, weight, (float*)out, dim, eps);
  else
    rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(
        x, partials, n_partials, partial_stride, rows, weight, (__nv_bfloat16*)out, dim, eps);
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_silu_mul(const float* gu, int n_partials, long long partial_stride, void* out,
                             int out_dtype, int rows, int F, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t total = (size_t)rows * F;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (out_dtype == DT_F32)
    silu_mul_kernel<float><<<(int)blocks, threads, 0, stream>>>(gu, n_partials, partial_stride,
                                                               (float*)out, rows, F);
  else
    silu_mul_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
        gu, n_partials, partial_stride, (__nv_bfloat16*)out, rows, F);
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_rope_store(const float* qkv, int n_partials, long long partial_stride,
                               const float* inv_freq, const int* token_seq, const int* q_start,
                               const int* seq_slot, const int* slot_pos, void* q_out,
                               void* kv_step, void* k_cache, void* v_cache, int dtype,
                               int n_tokens, int H, int G, int hd, int capacity, int write_cache,
                               cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd % 2 != 0 || hd / 2 > 256) return -2;
  const int half = hd / 2;
  int threads = 128;
  if (threads < half) threads = 256;
  if (dtype == DT_F32)
    rope_store_kernel<float><<<n_tokens, threads, 0, stream>>>(
        qkv, n_partials, partial_stride, inv_freq, token_seq, q_start, seq_slot, slot_pos,
        (float*)q_out, (float*)kv_step, (float*)k_cache, (float*)v_cache, H, G, hd, capacity,
        write_cache);
  else
    rope_store_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        qkv, n_partials, partial_stride, inv_freq, token_seq, q_start, seq_slot, slot_pos,
        (__nv_bfloat16*)q_out, (__nv_bfloat16*)kv_step, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, H, G, hd, capacity, write_cache);
  YALM_LAUNCH_CHECK();
  return 0;
}

extern "C" int yalm_advance(const int* q_start, const int* seq_slot, int* slot_pos, int n_seqs,
                            cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  advance_kernel<<<(n_seqs + 127) / 128, 128, 0, stream>>>(q_start, seq_slot, slot_pos, n_seqs);
  YALM_LAUNCH_CHECK();
  return 0;
}
