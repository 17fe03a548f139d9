// An entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference: its kernels take every buffer from
// the engine that owns them.  Here the split-KV attention kernel normally gets
// its scratch (the partial result of every key slice) from the caller.  A
// caller that has no allocator to ask -- one that handed all device memory to
// its own arena at start-up, or one running inside another runtime's callback
// where cudaMalloc is forbidden because it synchronises the device -- can call
// yalm_attention_no_alloc instead: the arguments are those of yalm_attention
// (api.h) without the two scratch pointers and without a page table (the cache
// is one block per sequence, [slots][G][capacity][hd]), and the scratch is a fixed array
// of yalm_attention_no_alloc_capacity() floats (8 MiB) inside the library.
//
// Returns 0, a cudaError_t, or a refusal: -7 if n_tokens * H * nsplit *
// (hd + 2) floats exceed the capacity, -8 for a device index beyond 63, the
// codes of yalm_attention otherwise.  The first call on a device looks up the
// array's address and should come before any stream capture; `stream` must
// belong to the device that is current at the call, because the array used is
// the current device's.  The addresses are kept in a host table without a
// lock: host threads that make a device's first call together may each do the
// look-up and store the same value.  Calls share the array: calls that overlap
// on the GPU race.  See the comment at the definition in attention.cu for the
// full rules.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long yalm_attention_no_alloc_capacity(void);

int yalm_attention_no_alloc(const void* q, const void* kv_step, const void* k_cache,
                            const void* v_cache, const int* token_seq, const int* q_start,
                            const int* seq_slot, const int* slot_pos, void* out, int dtype,
                            int n_tokens, int H, int G, int hd, int capacity, int window,
                            int nsplit, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
