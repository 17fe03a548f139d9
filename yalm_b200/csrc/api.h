// C interface of the sm_100a kernel library.  Every function launches on the
// given stream and returns 0, a cudaError_t of the launch, or a negative code
// for arguments it refuses (a size the kernel does not take).  Pointers are
// device pointers unless said otherwise.  dtype codes: 0 = float32, 1 = bfloat16,
// 2 = float16.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// a kernel whose bounded barrier wait runs out after limit_ns (<= 100 ms) and raises
// ERR_WAIT_TIMEOUT in *status: the status path, for tests
int yalm_wait_probe(unsigned long long limit_ns, int* status, cudaStream_t stream);
int yalm_copy_async(void* dst, const void* src, long long bytes, int to_device, cudaStream_t stream);
int yalm_stream_wait(cudaStream_t stream);
int yalm_embed(const int* tokens, const void* table, int table_dtype, float* x, int n_tokens,
               int dim, int vocab, int* status, cudaStream_t stream);

int yalm_rmsnorm(float* x, const float* partials, int n_partials, long long partial_stride,
                 const int* rows, const float* weight, void* out, int out_dtype, int n_rows,
                 int dim, float eps, cudaStream_t stream);

int yalm_silu_mul(const float* gu, int n_partials, long long partial_stride, void* out,
                  int out_dtype, int rows, int F, int paired, cudaStream_t stream);

// The cache of a layer run, wherever it is an argument: contiguous per sequence,
// [slots][G][capacity][hd] (page_table null), or pages of 64 positions,
// [pages][G][64][hd], with page_table [slots][pages_per_slot] naming the page of rows
// 64 p .. 64 p + 63 of each sequence.  A row is a position modulo the capacity.
int yalm_rope_store(const float* qkv, int n_partials, long long partial_stride,
                    const float* inv_freq, const int* token_seq, const int* q_start,
                    const int* seq_slot, const int* slot_pos, void* q_out, void* kv_step,
                    void* k_cache, void* v_cache, int dtype, int n_tokens, int H, int G, int hd,
                    int capacity, int write_cache, const int* page_table, int pages_per_slot, int n_pages,
                    cudaStream_t stream);

// kv_step [N, 2, G, hd] -> the ring rows of the positions the ring keeps (the cache
// write of yalm_rope_store, on its own: for a ring that may only be written after the
// attention has read the rows that are replaced)
int yalm_cache_write(const void* kv_step, const int* token_seq, const int* q_start,
                     const int* seq_slot, const int* slot_pos, void* k_cache, void* v_cache,
                     int dtype, int n_tokens, int G, int hd, int capacity, const int* page_table,
                     int pages_per_slot, int n_pages, cudaStream_t stream);

int yalm_advance(const int* q_start, const int* seq_slot, int* slot_pos, int n_seqs,
                 cudaStream_t stream);

int yalm_attention(const void* q, const void* kv_step, const void* k_cache, const void* v_cache,
                   const int* token_seq, const int* q_start, const int* seq_slot,
                   const int* slot_pos, void* out, float* part_o, float* part_ml, int dtype,
                   int n_tokens, int H, int G, int hd, int capacity, int window, int nsplit,
                   const int* page_table, int pages_per_slot, int n_pages, cudaStream_t stream);

int yalm_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                          const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                          float* part_ml, int* counters, int* status, int dtype, int n_seqs, int H,
                          int G, int hd, int capacity, int window, int chunk, int max_context,
                          const int* page_table, int pages_per_slot, int n_pages, cudaStream_t stream);

// 16-bit attention on tensor cores (attention_mma_prefill.cu, attention_mma.cu; dtype 1 or 2): head sizes in steps of
// 16 up to 128
int yalm_attention_prefill_mma(const void* q, const void* kv_step, const void* k_cache,
                               const void* v_cache, const int* q_start, const int* seq_slot,
                               const int* slot_pos, void* out, int dtype, int n_seqs,
                               int max_q_len, int H, int G, int hd, int capacity, int window,
                               const int* page_table, int pages_per_slot, int n_pages, cudaStream_t stream);
int yalm_attention_decode_mma(const void* q, const void* k_cache, const void* v_cache,
                              const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                              float* part_ml, int* counters, int* status, int dtype, int n_seqs,
                              int H, int G, int hd, int capacity, int window, int max_context,
                              int chunks_per_block, int warps, const int* page_table, int pages_per_slot,
                              int n_pages, cudaStream_t stream);
// ... compiled with two warps per block (attention_mma_two_warps.cu); yalm_attention_decode_mma
// calls it for warps = 2
int yalm_attention_decode_mma_two_warps(const void* q, const void* k_cache, const void* v_cache,
                                        const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                                        float* part_ml, int* counters, int* status, int dtype, int n_seqs,
                                        int H, int G, int hd, int capacity, int window, int max_context,
                                        int chunks_per_block, const int* page_table, int pages_per_slot,
                                        int n_pages, cudaStream_t stream);
// ... with the rotary kernel's work inside (attention_mma_fused.cu): takes this step's q/k/v product
// as n_partials 32-bit slices and the step's cosines and sines, writes the new cache rows
int yalm_attention_decode_mma_fused(const float* qkv, int n_partials, long long partial_stride,
                                    const float* cos_sin, void* k_cache, void* v_cache,
                                    const int* seq_slot, const int* slot_pos, void* out, float* part_o,
                                    float* part_ml, int* counters, int* status, int dtype, int n_seqs,
                                    int H, int G, int hd, int capacity, int window, int max_context,
                                    int chunks_per_block, const int* page_table, int pages_per_slot,
                                    int n_pages, cudaStream_t stream);

// 16-bit prefill attention on tcgen05 (attention_tc.cu; dtype 1 or 2): sequences that start
// at their first token, head size 64 or 128
int yalm_attention_prefill_tc(const void* q, const void* kv_step, const int* q_start, void* out,
                              int dtype, int n_tokens, int n_seqs, int max_q_len, int H, int G,
                              int hd, int window, int* status, cudaStream_t stream);
// ... for sequences that go on from slot_pos, no one wrapping around its ring in this step:
// every key (this step's too) from the layer's cache, paged or one block per sequence
int yalm_attention_prefill_tc_cache(const void* q, const void* k_cache, const void* v_cache,
                                    const int* q_start, const int* seq_slot, const int* slot_pos,
                                    void* out, int dtype, int n_tokens, int n_seqs, int max_q_len,
                                    int n_slots, int H, int G, int hd, int capacity, int window,
                                    const int* page_table, int pages_per_slot, int n_pages, int* status,
                                    cudaStream_t stream);

int yalm_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* out,
                   int out_dtype, int M, int N, int K, int accumulate, cudaStream_t stream);

// params: null, or two 64-bit words on the device that replace `seed` and `temperature`
// (the temperature's float bits in the low half of the second word)
int yalm_sample(const float* logits, int n_rows, int vocab, float temperature,
                unsigned long long seed, const unsigned long long* params, const int* row_key,
                const int* seq_slot, const int* slot_pos, int* out_tokens, cudaStream_t stream);

float yalm_uniform01(unsigned long long seed, unsigned key, unsigned counter);

// tcgen05 / TMA matrix product (operands of ab_dtype 1 or 2, 32-bit accumulation in TMEM;
// out_dtype is 0 or ab_dtype):
//   mode 0: out[M,N]  = A W^T             (out_dtype 0 or 1)
//   mode 1: out[M,N] += A W^T             (out float32: the residual stream)
//   mode 2: out[M,N/2] = silu(A Wg^T) * (A Wu^T), W = [Wg; Wu] with N rows in all
//   mode 3: out[s][M,N] = partial products of `splits` slices of K (float32 scratch)
// status: a device int that receives ERR_WAIT_TIMEOUT if a bounded wait gave up.
int yalm_gemm_tc(const void* A, const void* W, int ab_dtype, void* out, int out_dtype, int M,
                 int N, int K, int mode, int splits, int* status, cudaStream_t stream);
// 0 if the driver's tensor-map encoder was found (host-side set-up of yalm_gemm_tc).
int yalm_gemm_tc_available(void);

// cos_sin[t][i] = (cos, sin) of position(t) * inv_freq[i], positions as yalm_rope_store
// derives them: the table that yalm_gemm_2sm_rope reads, made once per step for all layers
int yalm_rope_table(const float* inv_freq, const int* token_seq, const int* q_start,
                    const int* seq_slot, const int* slot_pos, float* cos_sin, int n_tokens, int half,
                    cudaStream_t stream);

// What the rotary epilogue of yalm_gemm_2sm_rope needs: the arguments of yalm_rope_store,
// with the table of yalm_rope_table in place of the frequencies.
typedef struct yalm_rope_args {
  const float* cos_sin;      // [M][hd/2][2]
  const int* token_seq;      // [M]
  const int* q_start;        // [n_seqs + 1]
  const int* seq_slot;       // [n_seqs]
  const int* slot_pos;       // [slots]
  void* q_out;               // [M, H*hd]
  void* kv_step;             // [M, 2, G, hd]
  void* k_cache;
  void* v_cache;
  const int* page_table;     // null: a cache that is one block per sequence
  int pages_per_slot, n_pages;
  int H, G, hd, capacity, write_cache;
} yalm_rope_args;

// Two-SM (cta_group::2) variant for many tokens: mode 0 store, 1 add, 2 silu(gate)*up, 4 the
// same with interleaved rows, 3 `splits` slices of K as 32-bit partial sums [splits, M, N].
int yalm_gemm_2sm(const void* A, const void* W, int ab_dtype, void* out, int out_dtype, int M,
                  int N, int K, int mode, int splits, int* status, cudaStream_t stream);
// the token tile (256 or 240) it takes for these sizes
int yalm_gemm_2sm_token_tile(int M, int N, int splits);

// The q/k/v product of many tokens with rotary encoding and cache write in its epilogue
// (head sizes that divide 128).
int yalm_gemm_2sm_rope(const void* A, const void* W, int ab_dtype, int M, int N, int K,
                       const yalm_rope_args* rope, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
