// Causal grouped-query attention over the cache, one query token per block
// column, for prefill and decode alike, in 32-bit arithmetic on bfloat16, float16 or
// 32-bit storage.
//
// The reference computes the same thing for one token of one sequence with
// three kernels (attn_dot infer.cu:339-362, attn_softmax infer.cu:364-396,
// att_mix infer.cu:398-523): scores (q.k)/sqrt(hd) over kv_len keys, a
// max-subtracted softmax, the weighted sum of values.  Here one kernel does
// all three with an online softmax; the query heads that share a kv head
// share its loads; the keys of one query can be split over several blocks
// (split-KV) whose partial results a second kernel merges.
//
// Where a key lives: position j of a sequence is in this step's own buffer
// (kv_step) when j >= past (the sequence's length before the step), else in
// the cache ring at row j % capacity.  A prompt longer than the ring therefore
// still sees all of its own keys during prefill.
#include "api.h"
#include "common.cuh"
#include "no_alloc.h"

namespace yalm {

constexpr int ATT_RT = 4;        // query heads per block (of those sharing one kv head)
constexpr int ATT_WARPS = 4;
constexpr int ATT_EPL = 8;       // elements of a head that one lane owns
constexpr int ATT_U = 4;         // keys in flight per lane group

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  typedef uint4 Raw;
  static __device__ __forceinline__ Raw zero() { return make_uint4(0u, 0u, 0u, 0u); }
  static __device__ __forceinline__ Raw load_raw(const __nv_bfloat16* p) {
    return *reinterpret_cast<const uint4*>(p);
  }
  static __device__ __forceinline__ void unpack(const Raw& u, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    unpack(load_raw(p), f);
  }
};
template <> struct Vec8<__half> {
  typedef uint4 Raw;
  static __device__ __forceinline__ Raw zero() { return make_uint4(0u, 0u, 0u, 0u); }
  static __device__ __forceinline__ Raw load_raw(const __half* p) {
    return *reinterpret_cast<const uint4*>(p);
  }
  static __device__ __forceinline__ void unpack(const Raw& u, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __half22float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  static __device__ __forceinline__ void load(const __half* p, float* f) { unpack(load_raw(p), f); }
};
template <> struct Vec8<float> {
  struct Raw { float4 a, b; };
  static __device__ __forceinline__ Raw zero() {
    Raw r;
    r.a = make_float4(0.f, 0.f, 0.f, 0.f);
    r.b = r.a;
    return r;
  }
  static __device__ __forceinline__ Raw load_raw(const float* p) {
    Raw r;
    r.a = *reinterpret_cast<const float4*>(p);
    r.b = *reinterpret_cast<const float4*>(p + 4);
    return r;
  }
  static __device__ __forceinline__ void unpack(const Raw& r, float* f) {
    f[0] = r.a.x; f[1] = r.a.y; f[2] = r.a.z; f[3] = r.a.w;
    f[4] = r.b.x; f[5] = r.b.y; f[6] = r.b.z; f[7] = r.b.w;
  }
  static __device__ __forceinline__ void load(const float* p, float* f) { unpack(load_raw(p), f); }
};

// LPK lanes share one key (LPK*8 >= hd); a warp handles 32/LPK keys at a time.
template <typename T, int LPK>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_token_kernel(const T* __restrict__ q, const T* __restrict__ kv_step,
                  const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                  const int* __restrict__ token_seq, const int* __restrict__ q_start,
                  const int* __restrict__ seq_slot, const int* __restrict__ slot_pos,
                  T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                  int H, int G, int hd, int capacity, int window, int nsplit, float scale, int t0,
                  const int* __restrict__ page_table, int pps, int n_pages) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int KPW = 32 / LPK;                 // keys per warp per iteration
  constexpr int GROUPS = ATT_WARPS * KPW;       // key groups per block
  __shared__ float m_s[GROUPS][ATT_RT];
  __shared__ float l_s[GROUPS][ATT_RT];
  __shared__ float o_s[ATT_RT * GROUPS * LPK * ATT_EPL];   // [RT][GROUPS][LPK*8]

  const int R = H / G;
  const int nchunks = (R + ATT_RT - 1) / ATT_RT;
  const int g = blockIdx.y / nchunks;
  const int chunk = blockIdx.y % nchunks;
  const int h0 = g * R + chunk * ATT_RT;
  const int nh = min(ATT_RT, R - chunk * ATT_RT);
  const int t = t0 + blockIdx.z;
  const int split = blockIdx.x;

  const int b = token_seq[t];
  const int slot = seq_slot[b];
  const int past = slot_pos[slot];
  const int qs = q_start[b];
  const int pos = past + (t - qs);
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int nkeys = pos - lo + 1;
  const int per = (nkeys + nsplit - 1) / nsplit;
  const int s_lo = lo + split * per;
  const int s_hi = min(lo + (split + 1) * per, pos + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPK, kg = lane / LPK;
  const int e0 = sub * ATT_EPL;
  const bool lane_on = e0 < hd;

  float qreg[ATT_RT][ATT_EPL];
#pragma unroll
  for (int r = 0; r < ATT_RT; ++r) {
    if (r < nh && lane_on) {
      Vec8<T>::load(q + ((size_t)t * H + h0 + r) * hd + e0, qreg[r]);
    } else {
#pragma unroll
      for (int e = 0; e < ATT_EPL; ++e) qreg[r][e] = 0.f;
    }
  }
  float m[ATT_RT], l[ATT_RT], o[ATT_RT][ATT_EPL];
#pragma unroll
  for (int r = 0; r < ATT_RT; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int e = 0; e < ATT_EPL; ++e) o[r][e] = 0.f;
  }

  const size_t step_row = (size_t)2 * G * hd;

  // ATT_U keys per lane group are loaded before any is used: the loop is a
  // stream of independent 16-byte loads, which is what hides HBM latency
  for (int base = s_lo + warp * KPW; base < s_hi; base += GROUPS * ATT_U) {
    typename Vec8<T>::Raw kraw[ATT_U], vraw[ATT_U];
    bool valid[ATT_U];
#pragma unroll
    for (int u = 0; u < ATT_U; ++u) {
      const int key = base + u * GROUPS + kg;
      valid[u] = key < s_hi;
      if (valid[u] && lane_on) {
        const T *kp, *vp;
        if (key >= past) {
          kp = kv_step + (size_t)(qs + key - past) * step_row + (size_t)g * hd + e0;
          vp = kp + (size_t)G * hd;
        } else {
          const size_t row = kv_row_offset(page_table, pps, n_pages, slot, g, G, capacity, key % capacity, hd) + e0;
          kp = k_cache + row;
          vp = v_cache + row;
        }
        kraw[u] = Vec8<T>::load_raw(kp);
        vraw[u] = Vec8<T>::load_raw(vp);
      } else {
        kraw[u] = Vec8<T>::zero();
        vraw[u] = Vec8<T>::zero();
      }
    }
    float s[ATT_U][ATT_RT];
#pragma unroll
    for (int u = 0; u < ATT_U; ++u) {
      float kf[ATT_EPL];
      Vec8<T>::unpack(kraw[u], kf);
#pragma unroll
      for (int r = 0; r < ATT_RT; ++r) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < ATT_EPL; ++e) d = fmaf(qreg[r][e], kf[e], d);
#pragma unroll
        for (int off = LPK / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        s[u][r] = valid[u] ? d * scale : -INFINITY;
      }
    }
    float mn[ATT_RT], corr[ATT_RT];
#pragma unroll
    for (int r = 0; r < ATT_RT; ++r) {
      float x = m[r];
#pragma unroll
      for (int u = 0; u < ATT_U; ++u) x = fmaxf(x, s[u][r]);
      mn[r] = x;
      corr[r] = x > -INFINITY ? expf(m[r] - x) : 1.f;     // exp(-inf) = 0 on the first key
      l[r] *= corr[r];
#pragma unroll
      for (int e = 0; e < ATT_EPL; ++e) o[r][e] *= corr[r];
      m[r] = x;
    }
#pragma unroll
    for (int u = 0; u < ATT_U; ++u) {
      if (valid[u]) {
        float vf[ATT_EPL];
        Vec8<T>::unpack(vraw[u], vf);
#pragma unroll
        for (int r = 0; r < ATT_RT; ++r) {
          const float p = expf(s[u][r] - mn[r]);
          l[r] += p;
#pragma unroll
          for (int e = 0; e < ATT_EPL; ++e) o[r][e] = fmaf(p, vf[e], o[r][e]);
        }
      }
    }
  }

  // merge the key groups of the block
  const int grp = warp * KPW + kg;
#pragma unroll
  for (int r = 0; r < ATT_RT; ++r) {
    if (sub == 0) { m_s[grp][r] = m[r]; l_s[grp][r] = l[r]; }
#pragma unroll
    for (int e = 0; e < ATT_EPL; ++e)
      o_s[((size_t)r * GROUPS + grp) * (LPK * ATT_EPL) + e0 + e] = o[r][e];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nh * hd; idx += blockDim.x) {
    const int r = idx / hd, d = idx % hd;
    float M = -INFINITY;
    for (int gi = 0; gi < GROUPS; ++gi) M = fmaxf(M, m_s[gi][r]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
      for (int gi = 0; gi < GROUPS; ++gi) {
        const float w = expf(m_s[gi][r] - M);
        L += l_s[gi][r] * w;
        O += o_s[((size_t)r * GROUPS + gi) * (LPK * ATT_EPL) + d] * w;
      }
    }
    const int h = h0 + r;
    if (nsplit == 1) {
      out[((size_t)t * H + h) * hd + d] = from_float<T>(O / L);
    } else {
      const size_t pi = ((size_t)t * H + h) * nsplit + split;
      part_o[pi * hd + d] = O;
      if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
    }
  }
}

// Merges the nsplit partial results of one (token, head): block per (token, head).
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ part_o,
                                  const float* __restrict__ part_ml, T* __restrict__ out, int hd,
                                  int nsplit) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t th = blockIdx.x;
  const float* ml = part_ml + th * nsplit * 2;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ml[2 * s]);
  float L = 0.f;
  for (int s = 0; s < nsplit; ++s)
    if (ml[2 * s] > -INFINITY) L += ml[2 * s + 1] * expf(ml[2 * s] - M);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float O = 0.f;
    for (int s = 0; s < nsplit; ++s)
      if (ml[2 * s] > -INFINITY) O += part_o[(th * nsplit + s) * hd + d] * expf(ml[2 * s] - M);
    out[th * hd + d] = from_float<T>(O / L);
  }
}

// ---------------------------------------------------------------------------
// Decode attention: one query token per sequence, every key and value in the
// cache (the step's own row was written by the rotary kernel just before).
// A block takes one chunk of `chunk` consecutive positions of one (sequence,
// kv head, group of query heads).  It brings the chunk's K and V rows into
// shared memory with bulk asynchronous copies (one thread issues at most four:
// K and V, twice if the chunk wraps around the ring), so the memory system sees
// few large requests instead of thousands of 16-byte loads, and then computes
// from shared memory exactly as attn_token_kernel does from global memory.
// Chunks of one query are merged by the block that finishes last (a counter per
// query and head group; partial results in scratch, added in chunk order), so
// there is no second kernel.  Blocks whose chunk lies beyond the sequence's
// length leave at once.
constexpr int ATT_MAX_CHUNK = 128;

template <typename T, int LPK>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                   const T* __restrict__ v_cache, const int* __restrict__ seq_slot,
                   const int* __restrict__ slot_pos, T* __restrict__ out,
                   float* __restrict__ part_o, float* __restrict__ part_ml,
                   int* __restrict__ counters, int* __restrict__ status, int H, int G, int hd,
                   int capacity, int window, int chunk, int max_chunks, float scale,
                   const int* __restrict__ page_table, int pps, int n_pages) {
  static_assert(ATT_WARPS == ATT_RT, "one warp per query head in the softmax pass");
  constexpr int KPW = 32 / LPK;
  constexpr int GROUPS = ATT_WARPS * KPW;
  extern __shared__ __align__(128) uint8_t att_smem[];      // K rows, V rows; later the o partials
  __shared__ float sc_s[ATT_RT][ATT_MAX_CHUNK];             // scores, then probabilities
  __shared__ float m_s[GROUPS][ATT_RT];                     // scratch of the final merge
  __shared__ float l_s[GROUPS][ATT_RT];
  __shared__ float ml_s[2][ATT_RT];                         // this chunk's max and sum per head
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  __shared__ int last_flag;
  pdl_launch_dependents();
  pdl_wait();

  const int R = H / G;
  const int nchunks = (R + ATT_RT - 1) / ATT_RT;
  const int g = blockIdx.y / nchunks;
  const int hchunk = blockIdx.y % nchunks;
  const int h0 = g * R + hchunk * ATT_RT;
  const int nh = min(ATT_RT, R - hchunk * ATT_RT);
  const int t = blockIdx.z;
  const int c = blockIdx.x;

  const int slot = seq_slot[t];
  const int pos = slot_pos[slot];                           // the query's position
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int nkeys = pos - lo + 1;
  const int n_active = (nkeys + chunk - 1) / chunk;
  if (n_active > max_chunks && c == 0 && threadIdx.x == 0) atomicOr(status, ERR_CONTEXT_RANGE);
  if (c >= n_active) return;
  const int k_lo = lo + c * chunk;
  const int n = min(chunk, pos + 1 - k_lo);

  T* ks = reinterpret_cast<T*>(att_smem);
  T* vs = ks + (size_t)chunk * hd;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const size_t row_bytes = (size_t)hd * sizeof(T);
    // consecutive rows in runs that end where the ring wraps or a page ends
    mbar_expect_tx(smem_u32(&bar), (uint32_t)(2 * n * row_bytes));
    for (int done = 0; done < n;) {
      const int row = (k_lo + done) % capacity;
      int run = min(n - done, capacity - row);
      if (page_table != nullptr) run = min(run, KV_PAGE - row % KV_PAGE);
      const size_t off = kv_row_offset(page_table, pps, n_pages, slot, g, G, capacity, row, hd);
      bulk_load(smem_u32(ks + (size_t)done * hd), k_cache + off, (uint32_t)(run * row_bytes),
                smem_u32(&bar));
      bulk_load(smem_u32(vs + (size_t)done * hd), v_cache + off, (uint32_t)(run * row_bytes),
                smem_u32(&bar));
      done += run;
    }
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPK, kg = lane / LPK;
  const int e0 = sub * ATT_EPL;
  const bool lane_on = e0 < hd;
  float qreg[ATT_RT][ATT_EPL];
#pragma unroll
  for (int r = 0; r < ATT_RT; ++r) {
    if (r < nh && lane_on) {
      Vec8<T>::load(q + ((size_t)t * H + h0 + r) * hd + e0, qreg[r]);
    } else {
#pragma unroll
      for (int e = 0; e < ATT_EPL; ++e) qreg[r][e] = 0.f;
    }
  }
  __syncthreads();                                           // the barrier is initialised
  const bool arrived = mbar_wait(smem_u32(&bar), 0, &abort_flag);
  if (!arrived) {
    // never expected: give the copies time to land, report, and go on without a result
    if (threadIdx.x == 0) atomicOr(status, ERR_WAIT_TIMEOUT);
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }

  // pass 1: scores of the chunk's keys
  for (int base = warp * KPW; base < n; base += GROUPS) {
    const int i = base + kg;
    const bool valid = i < n;
    float kf[ATT_EPL];
    if (valid && lane_on) {
      Vec8<T>::load(ks + (size_t)i * hd + e0, kf);
    } else {
#pragma unroll
      for (int e = 0; e < ATT_EPL; ++e) kf[e] = 0.f;
    }
#pragma unroll
    for (int r = 0; r < ATT_RT; ++r) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < ATT_EPL; ++e) d = fmaf(qreg[r][e], kf[e], d);
#pragma unroll
      for (int off = LPK / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
      if (valid && sub == 0) sc_s[r][i] = d * scale;
    }
  }
  __syncthreads();
  // softmax numerators of the chunk: warp r owns head r
  {
    float mx = -INFINITY;
    for (int i = lane; i < n; i += 32) mx = fmaxf(mx, sc_s[warp][i]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) {
      const float p = expf(sc_s[warp][i] - mx);
      sc_s[warp][i] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    if (lane == 0) { ml_s[0][warp] = mx; ml_s[1][warp] = sum; }
  }
  __syncthreads();
  // pass 2: weighted sum of the values
  float o[ATT_RT][ATT_EPL];
#pragma unroll
  for (int r = 0; r < ATT_RT; ++r)
#pragma unroll
    for (int e = 0; e < ATT_EPL; ++e) o[r][e] = 0.f;
  for (int base = warp * KPW; base < n; base += GROUPS) {
    const int i = base + kg;
    if (i < n && lane_on) {
      float vf[ATT_EPL];
      Vec8<T>::load(vs + (size_t)i * hd + e0, vf);
#pragma unroll
      for (int r = 0; r < ATT_RT; ++r) {
        const float p = sc_s[r][i];
#pragma unroll
        for (int e = 0; e < ATT_EPL; ++e) o[r][e] = fmaf(p, vf[e], o[r][e]);
      }
    }
  }
  __syncthreads();                                           // K and V are no longer read
  float* o_s = reinterpret_cast<float*>(att_smem);           // [RT][GROUPS][LPK*8] over the K/V area
  const int grp = warp * KPW + kg;
#pragma unroll
  for (int r = 0; r < ATT_RT; ++r)
#pragma unroll
    for (int e = 0; e < ATT_EPL; ++e)
      o_s[((size_t)r * GROUPS + grp) * (LPK * ATT_EPL) + e0 + e] = o[r][e];
  __syncthreads();
  const size_t qh = (size_t)t * H + h0;                       // first (token, head) of this block
  for (int idx = threadIdx.x; idx < nh * hd; idx += blockDim.x) {
    const int r = idx / hd, d = idx % hd;
    float O = 0.f;
#pragma unroll
    for (int gi = 0; gi < GROUPS; ++gi) O += o_s[((size_t)r * GROUPS + gi) * (LPK * ATT_EPL) + d];
    if (n_active == 1) {
      out[(qh + r) * hd + d] = from_float<T>(O / ml_s[1][r]);
    } else {
      const size_t pi = (qh + r) * max_chunks + c;
      part_o[pi * hd + d] = O;
      if (d == 0) { part_ml[pi * 2] = ml_s[0][r]; part_ml[pi * 2 + 1] = ml_s[1][r]; }
    }
  }
  if (n_active == 1) return;

  // the block that arrives last adds the chunks in order
  __threadfence();
  __syncthreads();
  int* counter = counters + (size_t)t * gridDim.y + blockIdx.y;
  if (threadIdx.x == 0) last_flag = (atomicAdd(counter, 1) == n_active - 1) ? 1 : 0;
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  if (threadIdx.x == 0) *counter = 0;
  // weights of the chunks first (the small (max, sum) records, spread over all
  // threads), then the weighted sum of the partial outputs, eight loads in flight
  float* w_s = o_s;                                          // [n_active][ATT_RT], reuses o_s
  constexpr int W_CAP = (GROUPS * LPK * ATT_EPL);            // chunks whose weights fit (1024)
  if (n_active <= W_CAP) {
    float mloc[ATT_RT], lloc[ATT_RT];
#pragma unroll
    for (int r = 0; r < ATT_RT; ++r) {
      mloc[r] = -INFINITY;
      if (r < nh) {
        const float* ml = part_ml + (qh + r) * max_chunks * 2;
        for (int s2 = threadIdx.x; s2 < n_active; s2 += blockDim.x)
          mloc[r] = fmaxf(mloc[r], __ldcg(ml + 2 * s2));
      }
      mloc[r] = warp_max(mloc[r]);
      if (lane == 0) m_s[warp][r] = mloc[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < ATT_RT; ++r) {
      float M = -INFINITY;
#pragma unroll
      for (int wp = 0; wp < ATT_WARPS; ++wp) M = fmaxf(M, m_s[wp][r]);
      lloc[r] = 0.f;
      if (r < nh) {
        const float* ml = part_ml + (qh + r) * max_chunks * 2;
        for (int s2 = threadIdx.x; s2 < n_active; s2 += blockDim.x) {
          const float ms = __ldcg(ml + 2 * s2);
          const float w = ms > -INFINITY ? expf(ms - M) : 0.f;
          lloc[r] += __ldcg(ml + 2 * s2 + 1) * w;
          w_s[s2 * ATT_RT + r] = w;
        }
      }
      lloc[r] = warp_sum(lloc[r]);
      if (lane == 0) l_s[warp][r] = lloc[r];
    }
    __syncthreads();
    if (threadIdx.x < ATT_RT) {
      float L = 0.f;
#pragma unroll
      for (int wp = 0; wp < ATT_WARPS; ++wp) L += l_s[wp][threadIdx.x];
      ml_s[1][threadIdx.x] = L;                              // the total over all chunks
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nh * hd; idx += blockDim.x) {
      const int r = idx / hd, d = idx % hd;
      const float* po = part_o + (qh + r) * max_chunks * hd + d;
      float O = 0.f;
      int s = 0;
      for (; s + 8 <= n_active; s += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __ldcg(po + (size_t)(s + j) * hd);
#pragma unroll
        for (int j = 0; j < 8; ++j) O = fmaf(v[j], w_s[(s + j) * ATT_RT + r], O);
      }
      for (; s < n_active; ++s) O = fmaf(__ldcg(po + (size_t)s * hd), w_s[s * ATT_RT + r], O);
      out[(qh + r) * hd + d] = from_float<T>(O / ml_s[1][r]);
    }
    return;
  }
  for (int idx = threadIdx.x; idx < nh * hd; idx += blockDim.x) {
    const int r = idx / hd, d = idx % hd;
    const float* ml = part_ml + (qh + r) * max_chunks * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_active; ++s) M = fmaxf(M, __ldcg(ml + 2 * s));
    float L = 0.f, O = 0.f;
    for (int s = 0; s < n_active; ++s) {
      const float ms = __ldcg(ml + 2 * s);
      if (ms > -INFINITY) {
        const float w = expf(ms - M);
        L += __ldcg(ml + 2 * s + 1) * w;
        O += __ldcg(part_o + ((qh + r) * max_chunks + s) * hd + d) * w;
      }
    }
    out[(qh + r) * hd + d] = from_float<T>(O / L);
  }
}

template <typename T>
static int launch_attention(const void* q, const void* kv_step, const void* k_cache,
                            const void* v_cache, const int* token_seq, const int* q_start,
                            const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                            float* part_ml, int n_tokens, int H, int G, int hd, int capacity,
                            int window, int nsplit, const int* page_table, int pps, int n_pages,
                            cudaStream_t stream) {
  const int R = H / G;
  const int nchunks = (R + ATT_RT - 1) / ATT_RT;
  const dim3 block(ATT_WARPS * 32);
  const float scale = 1.0f / sqrtf((float)hd);
  // gridDim.z is limited to 65535: tokens run in slices
  for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
  const dim3 grid(nsplit, G * nchunks, n_tokens - t0 < 65535 ? n_tokens - t0 : 65535);
#define YALM_ATT_CASE(LPK)                                                                      \
  launch_pdl(attn_token_kernel<T, LPK>, dim3(grid), dim3(block), 0, stream,                                         \
      (const T*)q, (const T*)kv_step, (const T*)k_cache, (const T*)v_cache, token_seq, q_start, \
      seq_slot, slot_pos, (T*)out, part_o, part_ml, H, G, hd, capacity, window, nsplit, scale, t0, \
      page_table, pps, n_pages)
  if (hd <= 16) YALM_ATT_CASE(2);
  else if (hd <= 32) YALM_ATT_CASE(4);
  else if (hd <= 64) YALM_ATT_CASE(8);
  else if (hd <= 128) YALM_ATT_CASE(16);
  else YALM_ATT_CASE(32);
#undef YALM_ATT_CASE
  YALM_LAUNCH_CHECK();
  }
  if (nsplit > 1) {
    const int threads = hd >= 128 ? 128 : (hd >= 64 ? 64 : 32);
    launch_pdl(attn_merge_kernel<T>, dim3(n_tokens * H), dim3(threads), 0, stream, part_o, part_ml, (T*)out, hd,
                                                               nsplit);
    YALM_LAUNCH_CHECK();
  }
  return 0;
}

}  // namespace yalm

using namespace yalm;

// part_o: [n_tokens, H, nsplit, hd] floats, part_ml: [n_tokens, H, nsplit, 2]
// floats; both are needed only when nsplit > 1.
extern "C" int yalm_attention(const void* q, const void* kv_step, const void* k_cache,
                              const void* v_cache, const int* token_seq, const int* q_start,
                              const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                              float* part_ml, int dtype, int n_tokens, int H, int G, int hd,
                              int capacity, int window, int nsplit, const int* page_table,
                              int pages_per_slot, int n_pages, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd % 8 != 0 || hd > 256 || hd <= 0) return -2;     // head sizes: multiples of 8 up to 256
  if (G <= 0 || H % G != 0) return -3;
  if (nsplit < 1 || nsplit > 65535) return -4;
  if ((size_t)G * ((H / G + ATT_RT - 1) / ATT_RT) > 65535) return -5;
  if (dtype == DT_F32)
    return launch_attention<float>(q, kv_step, k_cache, v_cache, token_seq, q_start, seq_slot,
                                   slot_pos, out, part_o, part_ml, n_tokens, H, G, hd, capacity,
                                   window, nsplit, page_table, pages_per_slot, n_pages, stream);
  if (dtype == DT_F16)
    return launch_attention<__half>(q, kv_step, k_cache, v_cache, token_seq, q_start, seq_slot,
                                    slot_pos, out, part_o, part_ml, n_tokens, H, G, hd, capacity,
                                    window, nsplit, page_table, pages_per_slot, n_pages, stream);
  if (dtype != DT_BF16) return -3;
  return launch_attention<__nv_bfloat16>(q, kv_step, k_cache, v_cache, token_seq, q_start,
                                         seq_slot, slot_pos, out, part_o, part_ml, n_tokens, H, G,
                                         hd, capacity, window, nsplit, page_table, pages_per_slot, n_pages,
                                         stream);
}

// Decode attention (see attn_decode_kernel).  Every query is the newest token of
// its sequence and its own key/value row is already in the cache.  chunk: keys
// per block; max_context: upper bound of any sequence's visible keys in this
// call (it sizes the grid).  part_o [n, H, max_chunks, hd], part_ml
// [n, H, max_chunks, 2] floats with max_chunks = ceil(max_context / chunk);
// counters: n * G * ceil((H/G)/4) ints, zero before the first launch.
extern "C" int yalm_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                                     const int* seq_slot, const int* slot_pos, void* out,
                                     float* part_o, float* part_ml, int* counters, int* status,
                                     int dtype, int n_seqs, int H, int G, int hd, int capacity,
                                     int window, int chunk, int max_context,
                                     const int* page_table, int pages_per_slot, int n_pages,
                                     cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (hd % 8 != 0 || hd > 256 || hd <= 0) return -2;
  if (G <= 0 || H % G != 0) return -3;
  if (chunk <= 0 || max_context <= 0 || n_seqs > 65535) return -4;
  const size_t esz = dtype == DT_F32 ? 4 : 2;
  if (chunk > ATT_MAX_CHUNK) return -2;
  size_t smem = (size_t)2 * chunk * hd * esz;
  if (smem < 16 * 1024) smem = 16 * 1024;                    // the merge reuses it for partials
  if (smem > 160 * 1024) return -2;
  const int R = H / G;
  const int nchunks = (R + ATT_RT - 1) / ATT_RT;
  if ((size_t)G * nchunks > 65535) return -4;
  const int visible = window > 0 && window < max_context ? window : max_context;
  const int max_chunks = (visible + chunk - 1) / chunk;
  const dim3 grid(max_chunks, G * nchunks, n_seqs);
  const dim3 block(ATT_WARPS * 32);
  const float scale = 1.0f / sqrtf((float)hd);
#define YALM_DEC_CASE(T, LPK)                                                                  \
  do {                                                                                         \
    static size_t attr_smem = 0;                                                               \
    if (smem > attr_smem) {                                                                    \
      cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<T, LPK>,                         \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                           (int)smem);                                         \
      if (e != cudaSuccess) return (int)e;                                                     \
      attr_smem = smem;                                                                        \
    }                                                                                          \
    launch_pdl(attn_decode_kernel<T, LPK>, grid, block, smem, stream, (const T*)q,             \
               (const T*)k_cache, (const T*)v_cache, seq_slot, slot_pos, (T*)out, part_o,      \
               part_ml, counters, status, H, G, hd, capacity, window, chunk, max_chunks,       \
               scale, page_table, pages_per_slot, n_pages);                                             \
  } while (0)
#define YALM_DEC_T(T)                                  \
  do {                                                 \
    if (hd <= 16) YALM_DEC_CASE(T, 2);                 \
    else if (hd <= 32) YALM_DEC_CASE(T, 4);            \
    else if (hd <= 64) YALM_DEC_CASE(T, 8);            \
    else if (hd <= 128) YALM_DEC_CASE(T, 16);          \
    else YALM_DEC_CASE(T, 32);                         \
  } while (0)
  if (dtype == DT_F32) YALM_DEC_T(float);
  else if (dtype == DT_F16) YALM_DEC_T(__half);
  else if (dtype == DT_BF16) YALM_DEC_T(__nv_bfloat16);
  else return -3;
#undef YALM_DEC_T
#undef YALM_DEC_CASE
  YALM_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// yalm_attention_no_alloc: the same attention for callers that cannot allocate.
// (Declared in no_alloc.h; the reference has nothing like it.)
//
// Split-KV attention needs scratch for the partial results of each key slice.
// yalm_attention takes that scratch from its caller.  Some callers have no way
// to provide it: a host program that gave all device memory to an arena of its
// own at start-up, or code running inside another runtime's callback where
// cudaMalloc is off limits because it synchronises the whole device.  For them
// the scratch lives in the array below, which is part of the loaded library
// image: every GPU that loads the library holds these 8 MiB until the process
// exits, whether or not this entry point is ever called.
//
// Rules of use:
//  * n_tokens * H * nsplit * (hd + 2) floats must fit into the array; a larger
//    request is refused with -7 and nothing is launched.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and remembers it; make
//    that first call outside any stream capture.  The address is kept per
//    device in a plain host table: `stream` must belong to the device that is
//    current at the call (the array used is the current device's), and when
//    several host threads make the first call together each may do the look-up
//    and store the same value, which is harmless.
//  * All calls share the one array, and it keeps whatever the last call left.
//    Nothing in it has to start at zero: every slice that is read was written
//    by the same call (an empty slice writes max = -inf, sum = 0).  Two calls
//    that overlap on the GPU (different streams) race on it; keep calls on one
//    stream or order them with events.
//  * No cudaMalloc, cudaFree or other allocating routine is called.
namespace yalm {
constexpr size_t NO_ALLOC_SCRATCH_FLOATS = (size_t)2 * 1024 * 1024;      // 8 MiB
static __device__ __align__(256) float g_attention_scratch[NO_ALLOC_SCRATCH_FLOATS];
constexpr int NO_ALLOC_MAX_DEVICES = 64;
static float* g_attention_scratch_addr[NO_ALLOC_MAX_DEVICES];            // per device, host side
}  // namespace yalm

extern "C" long long yalm_attention_no_alloc_capacity(void) {
  return (long long)yalm::NO_ALLOC_SCRATCH_FLOATS;
}

extern "C" int yalm_attention_no_alloc(const void* q, const void* kv_step, const void* k_cache,
                                       const void* v_cache, const int* token_seq,
                                       const int* q_start, const int* seq_slot,
                                       const int* slot_pos, void* out, int dtype, int n_tokens,
                                       int H, int G, int hd, int capacity, int window, int nsplit,
                                       cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  // the same refusals, in the same order, as yalm_attention; then the capacity
  if (hd % 8 != 0 || hd > 256 || hd <= 0) return -2;
  if (G <= 0 || H <= 0 || H % G != 0) return -3;
  if (nsplit < 1 || nsplit > 65535) return -4;
  const size_t need = (size_t)n_tokens * H * nsplit * ((size_t)hd + 2);
  if (nsplit > 1 && need > yalm::NO_ALLOC_SCRATCH_FLOATS) return -7;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= yalm::NO_ALLOC_MAX_DEVICES) return -8;
  if (yalm::g_attention_scratch_addr[dev] == nullptr) {
    // the array's name is a host-side handle here, not a device address
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, yalm::g_attention_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return -9;
    yalm::g_attention_scratch_addr[dev] = p;
  }
  float* base = yalm::g_attention_scratch_addr[dev];
  float* part_o = base;                                              // [tokens, H, nsplit, hd]
  float* part_ml = base + (size_t)n_tokens * H * nsplit * hd;        // [tokens, H, nsplit, 2]
  return yalm_attention(q, kv_step, k_cache, v_cache, token_seq, q_start, seq_slot, slot_pos, out,
                        part_o, part_ml, dtype, n_tokens, H, G, hd, capacity, window, nsplit,
                        nullptr, 0, 0, stream);            // a contiguous cache only
}
