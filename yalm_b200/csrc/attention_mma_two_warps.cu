// The decode attention compiled with two warps per block (attention_mma.cuh): two such blocks
// share an SM.  A translation unit of its own, so that its instantiations compile beside the
// others; reached through yalm_attention_decode_mma(..., warps = 2, ...).
#include "attention_mma.cuh"

using namespace yalm;

extern "C" int yalm_attention_decode_mma_two_warps(const void* q, const void* k_cache, const void* v_cache,
                                                   const int* seq_slot, const int* slot_pos, void* out,
                                                   float* part_o, float* part_ml, int* counters,
                                                   int* status, int dtype, int n_seqs, int H, int G, int hd,
                                                   int capacity, int window, int max_context,
                                                   int chunks_per_block, const int* page_table,
                                                   int pages_per_slot, int n_pages, cudaStream_t stream) {
  return decode_mma_dispatch<false, 2>(q, k_cache, v_cache, seq_slot, slot_pos, out, part_o, part_ml,
                                       counters, status, dtype, n_seqs, H, G, hd, capacity, window,
                                       max_context, chunks_per_block, page_table, pages_per_slot, n_pages,
                                       nullptr, stream);
}
