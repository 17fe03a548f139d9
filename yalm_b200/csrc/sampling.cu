// Sampling on the device, one block per row of logits.
//
// Greedy: the first maximal index (sampler.cpp:27-38).  Temperature: with
// e_i = exp((l_i - max)/T), the first i whose running sum of e reaches
// r * sum(e), the last index if none does (sampler.cpp:44-64, where r is
// rand()/RAND_MAX).  Here r comes from a counter-based generator keyed by
// (seed, the request's key, the position the new token will take), so a
// request's tokens do not depend on what else is in the batch.
#include "api.h"
#include "common.cuh"

namespace yalm {

__host__ __device__ inline unsigned long long mix64(unsigned long long x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}
__host__ __device__ inline float uniform01(unsigned long long seed, unsigned key,
                                           unsigned counter) {
  unsigned long long x = mix64(seed ^ ((unsigned long long)key * 0x9E3779B97F4A7C15ull));
  x = mix64(x ^ ((unsigned long long)counter * 0xD1B54A32D192ED03ull));
  return (float)(x >> 40) * (1.0f / 16777216.0f);   // 24 bits: [0, 1)
}

// a row is read once or twice: what matters is how many loads are in flight
constexpr int SAMPLE_THREADS = 1024;
static_assert(SAMPLE_THREADS == 1024, "the scan over the warps' sums assumes 32 warps");

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, float temperature,
              unsigned long long seed, const unsigned long long* __restrict__ params,
              const int* __restrict__ row_key, const int* __restrict__ seq_slot,
              const int* __restrict__ slot_pos, int* __restrict__ out_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  if (params != nullptr) {
    // seed and temperature from device memory (written by a host copy): a captured
    // launch then serves every seed and temperature
    seed = params[0];
    temperature = __uint_as_float((unsigned)params[1]);
  }
  __shared__ float red_v[SAMPLE_THREADS];
  __shared__ int red_i[SAMPLE_THREADS];
  __shared__ int result;
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* l = logits + (size_t)row * vocab;

  // first maximal index
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  int i = tid;
  for (; i + 3 * SAMPLE_THREADS < vocab; i += 4 * SAMPLE_THREADS) {   // four loads in flight
    const float v0 = l[i], v1 = l[i + SAMPLE_THREADS], v2 = l[i + 2 * SAMPLE_THREADS],
                v3 = l[i + 3 * SAMPLE_THREADS];
    if (v0 > bv) { bv = v0; bi = i; }
    if (v1 > bv) { bv = v1; bi = i + SAMPLE_THREADS; }
    if (v2 > bv) { bv = v2; bi = i + 2 * SAMPLE_THREADS; }
    if (v3 > bv) { bv = v3; bi = i + 3 * SAMPLE_THREADS; }
  }
  for (; i < vocab; i += SAMPLE_THREADS) {
    const float v = l[i];
    if (v > bv) { bv = v; bi = i; }
  }
  red_v[tid] = bv;
  red_i[tid] = bi;
  __syncthreads();
  for (int s = SAMPLE_THREADS / 2; s > 0; s >>= 1) {
    if (tid < s) {
      const float ov = red_v[tid + s];
      const int oi = red_i[tid + s];
      if (ov > red_v[tid] || (ov == red_v[tid] && oi < red_i[tid])) {
        red_v[tid] = ov;
        red_i[tid] = oi;
      }
    }
    __syncthreads();
  }
  const float maxv = red_v[0];
  const int argmax = red_i[0] == 0x7fffffff ? 0 : red_i[0];
  if (temperature == 0.0f) {
    if (tid == 0) out_tokens[row] = argmax;
    return;
  }

  // each thread owns a contiguous chunk of the vocabulary
  const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int c0 = min(tid * chunk, vocab), c1 = min(c0 + chunk, vocab);
  float mine = 0.f;
  for (int i = c0; i < c1; ++i) mine += expf((l[i] - maxv) / temperature);
  // running sums over the threads' chunks: a scan inside each warp, then over the warps
  const int lane = tid & 31, warp = tid >> 5;
  float incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  float excl = __shfl_up_sync(0xffffffffu, incl, 1);
  if (lane == 0) excl = 0.f;
  __syncthreads();                                   // red_v is free again
  if (lane == 31) red_v[warp] = incl;
  if (tid == 0) result = vocab - 1;
  __syncthreads();
  if (warp == 0) {
    float w = red_v[lane];                           // SAMPLE_THREADS / 32 == 32 warps
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += n;
    }
    red_v[lane] = w;
  }
  __syncthreads();
  // a warp's last running sum is, to the bit, the next warp's first exclusive sum
  const float base = warp > 0 ? red_v[warp - 1] : 0.f;
  incl = lane == 31 ? red_v[warp] : incl + base;
  excl += base;
  const float total = red_v[SAMPLE_THREADS / 32 - 1];
  const unsigned counter = (unsigned)slot_pos[seq_slot[row]];
  const float target = uniform01(seed, (unsigned)row_key[row], counter) * total;
  if (c1 > c0 && incl >= target && (tid == 0 || excl < target)) {
    float cum = excl;
    int pick = c1 - 1;
    for (int i = c0; i < c1; ++i) {
      cum += expf((l[i] - maxv) / temperature);
      if (cum >= target) { pick = i; break; }
    }
    result = pick;
  }
  __syncthreads();
  if (tid == 0) out_tokens[row] = result;
}

}  // namespace yalm

using namespace yalm;

// params: null, or two 64-bit words on the device that replace the arguments: the seed, and
// the temperature's 32 bits in the low half of the second word.
extern "C" int yalm_sample(const float* logits, int n_rows, int vocab, float temperature,
                           unsigned long long seed, const unsigned long long* params,
                           const int* row_key, const int* seq_slot, const int* slot_pos,
                           int* out_tokens, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0 || temperature < 0.f) return -2;
  launch_pdl(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, vocab,
             temperature, seed, params, row_key, seq_slot, slot_pos, out_tokens);
  YALM_LAUNCH_CHECK();
  return 0;
}

// The same generator on the host, for tests and for callers that sample on the CPU.
extern "C" float yalm_uniform01(unsigned long long seed, unsigned key, unsigned counter) {
  return uniform01(seed, key, counter);
}
