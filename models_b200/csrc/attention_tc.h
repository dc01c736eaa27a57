/* C interface of the tensor-core attention library (attention_tc.cu), one build per head size
 * (-DMB_HEAD_DIM).  Every function returns 0, or non-zero with a message in mb_last_error().
 * Pointers are device pointers unless stated; `stream` is the CUDA stream to launch on. */
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* mb_last_error(void);
int mb_attention_head_dim(void);

/* Page stages (2 or 3) a decode call with `splits` blocks per sequence runs with, and the shared memory in bytes of
 * one block with so many stages: for callers that plan how many blocks are resident at once. */
int mb_decode_stages(int splits);
size_t mb_decode_block_bytes(int stages);

/* Floats of scratch a decode call with `splits` > 1 needs (0 for one split). */
size_t mb_decode_scratch_floats(int sequences, int heads, int splits);

/* One query token per sequence against its cached keys and values.  With splits > 1 the partial
 * results of the split keys go through `scratch` (mb_decode_scratch_floats floats, from the caller)
 * and a second kernel; with scratch == NULL and splits <= 8 the blocks of a sequence form a
 * thread-block cluster and combine in shared memory instead. */
int mb_decode_attention(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_pool,
                        const void* v_pool, const int* block_table, int max_blocks, const int* cu_q, const int* kv_lens,
                        int sequences, int heads, int kv_heads, int page_size, int window, float scale, int splits,
                        float* scratch, cudaStream_t stream);

/* Any number of new tokens per sequence, their keys and values already cached. */
int mb_prefill_attention(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_pool,
                         const void* v_pool, const int* block_table, int max_blocks, const int* cu_q, const int* kv_lens,
                         int sequences, int max_q_len, int heads, int kv_heads, int page_size, int window, float scale,
                         cudaStream_t stream);

/* No counterpart in integrallis/models.  mb_decode_attention for callers that cannot allocate
 * device memory -- a host program without the framework's allocator that gave all device memory to
 * its own arena, or that may not call cudaMalloc where it calls this.  It allocates nothing: the
 * partial results of the split keys go to an array built into the library
 * (mb_decode_attention_static_capacity() floats, 4 MiB, held by every GPU that loads the library
 * until the process exits).  sequences * heads * splits * (head size + 2) must not exceed that
 * capacity when splits > 1; a larger request is refused with a message.  The first call on a
 * device looks the array's address up (make that call outside any stream capture).  All calls share
 * the array: calls that may overlap on the GPU race on it and must be ordered by the caller. */
size_t mb_decode_attention_static_capacity(void);
int mb_decode_attention_static(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_pool,
                               const void* v_pool, const int* block_table, int max_blocks, const int* cu_q,
                               const int* kv_lens, int sequences, int heads, int kv_heads, int page_size, int window,
                               float scale, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
