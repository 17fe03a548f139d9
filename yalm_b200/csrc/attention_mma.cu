// Attention on mma.sync tensor-core tiles: the entry point of the decode kernel (the kernels
// themselves: attention_mma.cuh; the prefill kernel's entry: attention_mma_prefill.cu).
#include "attention_mma.cuh"

using namespace yalm;

// Decode attention on tensor cores (dtype: bfloat16 or float16): one query per sequence over the
// cache.  A block walks through `chunks_per_block` chunks of 64 positions; a
// sequence needs parts = ceil(ceil(visible / 64) / chunks_per_block) blocks, with
// visible = min(max_context, window).  part_o [n, H, parts, hd] and part_ml
// [n, H, parts, 2] floats; counters: n * G * ceil((H/G)/16) ints, zero before the
// first launch.  Head sizes: multiples of 16 up to 128.  `warps`: 4, one block of four
// warps to an SM; or 2, two blocks of two warps, each warp with the same ring as before, so
// that one block's start and end run under the other's copies (for grids of several waves
// of whole sequences).
extern "C" int yalm_attention_decode_mma(const void* q, const void* k_cache, const void* v_cache,
                                         const int* seq_slot, const int* slot_pos, void* out,
                                         float* part_o, float* part_ml, int* counters, int* status,
                                         int dtype, int n_seqs, int H, int G, int hd, int capacity,
                                         int window, int max_context, int chunks_per_block,
                                         int warps, const int* page_table, int pages_per_slot,
                                         int n_pages, cudaStream_t stream) {
  if (warps == 2)                     // compiled in a translation unit of its own
    return yalm_attention_decode_mma_two_warps(q, k_cache, v_cache, seq_slot, slot_pos, out, part_o,
                                               part_ml, counters, status, dtype, n_seqs, H, G, hd,
                                               capacity, window, max_context, chunks_per_block,
                                               page_table, pages_per_slot, n_pages, stream);
  if (warps != FD_WARPS_MAX) return -4;
  return decode_mma_dispatch<false, FD_WARPS_MAX>(q, k_cache, v_cache, seq_slot, slot_pos, out, part_o,
                                                  part_ml, counters, status, dtype, n_seqs, H, G, hd,
                                                  capacity, window, max_context, chunks_per_block,
                                                  page_table, pages_per_slot, n_pages, nullptr, stream);
}
