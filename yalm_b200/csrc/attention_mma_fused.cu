// The decode attention compiled with the rotary kernel's work inside (attention_mma.cuh): a
// translation unit of its own, so that its instantiations compile beside the others.
#include "attention_mma.cuh"

using namespace yalm;

// The same with the rotary kernel's work done inside: instead of rotated queries and a cache
// that already holds this step's row, it takes the q/k/v product of this step (n_partials
// 32-bit slices [slice][n_seqs][(H + 2 G) hd], partial_stride elements apart) and the step's
// cosines and sines cos_sin [n_seqs][hd / 2][2], and writes the new cache rows itself.
extern "C" int yalm_attention_decode_mma_fused(const float* qkv, int n_partials, long long partial_stride,
                                               const float* cos_sin, void* k_cache, void* v_cache,
                                               const int* seq_slot, const int* slot_pos, void* out,
                                               float* part_o, float* part_ml, int* counters,
                                               int* status, int dtype, int n_seqs, int H, int G, int hd,
                                               int capacity, int window, int max_context,
                                               int chunks_per_block, const int* page_table,
                                               int pages_per_slot, int n_pages, cudaStream_t stream) {
  if (qkv == nullptr || cos_sin == nullptr || n_partials < 1) return -3;
  if (((uintptr_t)qkv | (uintptr_t)cos_sin) & 15 || (partial_stride & 3)) return -6;
  const fd_fused_args fz = {qkv, reinterpret_cast<const float2*>(cos_sin), partial_stride, n_partials};
  return decode_mma_dispatch<true, FD_WARPS_MAX>(nullptr, k_cache, v_cache, seq_slot, slot_pos, out, part_o,
                                                 part_ml, counters, status, dtype, n_seqs, H, G, hd, capacity,
                                                 window, max_context, chunks_per_block, page_table,
                                                 pages_per_slot, n_pages, &fz, stream);
}
