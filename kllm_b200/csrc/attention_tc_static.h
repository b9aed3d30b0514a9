// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for
// programs that embed these kernels where cudaMalloc is off limits: a caller that
// runs inside a memory pool it does not own, a plugin that is handed a fixed
// arena by its host application, or a real-time loop that may not enter the
// allocator because an allocation can synchronise the whole device.  The regular
// entry point (kllm_attention_decode) wants two scratch buffers for the partial
// results of its key ranges, which somebody has to allocate; this one brings its
// own.
//
// The scratch lives in a file-scope `static __device__` array of
// KLLM_ATTN_STATIC_SCRATCH_FLOATS floats (4 MiB) inside the library, so every GPU
// that loads the library holds those 4 MiB until the process exits, used or not.
// A call needs n_tokens * n_heads * num_splits * (head_dim + 2) floats of it and
// is refused with a clear message when that is more than the array holds; with
// num_splits == 1 nothing of it is used.  The function itself calls neither
// cudaMalloc nor cudaFree nor any allocating library routine.
//
// First call on a device: the array's device address is looked up once per device
// (cudaGetSymbolAddress with that device current) and the kernels' shared-memory
// limit is raised.  Make that first call outside of any stream capture.  The look-up
// is guarded by a mutex, so threads may make their first calls at the same time.
//
// All calls share the one array and it keeps whatever the last call left there.
// Nothing in it has to start at zero: every slot that a call reads was written by
// that same call before.  Two calls whose kernels overlap on the GPU (different
// streams, no dependency between them) would write the same slots and race; issue
// them on one stream or order them with events.
//
// Arguments are those of kllm_attention_decode without the two scratch pointers.
// Returns 0, a positive cudaError_t, or a negative code for a refused argument;
// kllm_last_error_attention_tc() then holds the message.
#pragma once
#include <stdint.h>

#define KLLM_ATTN_STATIC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int kllm_attention_decode_static(void* out, const void* q, int64_t q_stride, const void* kcache,
                                 const void* vcache, const int* positions, const int* token_req,
                                 const int* block_table, int max_blocks, int n_tokens, int n_heads,
                                 int n_kv, int hd, int page_size, int window, float scale,
                                 int num_splits, void* stream);

#ifdef __cplusplus
}
#endif
