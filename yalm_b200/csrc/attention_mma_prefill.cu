// Attention on mma.sync tensor-core tiles: the entry point of the prefill kernel
// (attention_mma.cuh), in a translation unit of its own so that it compiles beside the others.
#include "attention_mma.cuh"

using namespace yalm;

// Prefill attention on tensor cores (dtype: bfloat16 or float16).  Sequences are given by q_start
// [n_seqs + 1]; max_q_len is the longest of them (it sizes the grid).  Head sizes:
// multiples of 16 up to 128 (others: use yalm_attention).
extern "C" int yalm_attention_prefill_mma(const void* q, const void* kv_step, const void* k_cache,
                                          const void* v_cache, const int* q_start,
                                          const int* seq_slot, const int* slot_pos, void* out,
                                          int dtype, int n_seqs, int max_q_len, int H, int G,
                                          int hd, int capacity, int window, const int* page_table,
                                          int pages_per_slot, int n_pages, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  if (dtype != DT_BF16 && dtype != DT_F16) return -3;
  if (hd % 16 != 0 || hd > 128 || hd <= 0) return -2;
  if (G <= 0 || H % G != 0) return -3;
  if (H > 65535 || n_seqs > 65535) return -4;
#define YALM_FP(HDP, T)                                                                          \
  return launch_prefill<HDP, T>(q, kv_step, k_cache, v_cache, q_start, seq_slot, slot_pos, out,  \
                                n_seqs, max_q_len, H, G, hd, capacity, window, page_table,        \
                                pages_per_slot, n_pages, stream)
  if (dtype == DT_F16) {
    if (hd <= 64) YALM_FP(64, __half);
    YALM_FP(128, __half);
  }
  if (hd <= 64) YALM_FP(64, __nv_bfloat16);
  YALM_FP(128, __nv_bfloat16);
#undef YALM_FP
}
