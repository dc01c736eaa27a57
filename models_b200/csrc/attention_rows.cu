// Causal grouped-query attention over a paged cache, one warp per (token, head) row.
//
// This is the plain-arithmetic kernel: every size of head (up to 256), float or bfloat16 storage,
// prompts and single decoded tokens alike.  It is the whole attention of the 32-bit path and the
// fallback of the bfloat16 path for head sizes its tensor-core kernels do not take.
//
// Formula (integrallis/models, backend-java/.../llama/LlamaForwardPass.java:1543-1670 and
// backend-java/.../ops/TensorOps.java:1247-1279): kvHead = head / (heads / kv_heads);
// score_p = dot(q, K[p]) * scale for the visible p; softmax with the maximum subtracted;
// out = sum_p prob_p * V[p].  The softmax here is the running ("online") form of the same sum:
// it keeps a running maximum m and rescales the partial sums when m grows.  All of it in float.
//
// Cache layout of one layer: pool[page][kv_head][page_size][head_dim]; block_table[seq][i] is the
// page that holds positions [i*page_size, (i+1)*page_size) of that sequence.
#include "common.cuh"

#include <math_constants.h>

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kMaxHeadDim = 256;
constexpr int kAccPerLane = kMaxHeadDim / 32;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q_shared, const T* __restrict__ k_row, int head_dim,
                                         bool vector_ok) {
    float sum = 0.0f;
    if (vector_ok) {
        for (int d = 0; d < head_dim; d += 8) {
            float kv[8];
            load8(k_row + d, kv);
#pragma unroll
            for (int i = 0; i < 8; ++i) sum = fmaf(q_shared[d + i], kv[i], sum);
        }
    } else {
        for (int d = 0; d < head_dim; ++d) sum = fmaf(q_shared[d], Num<T>::load(k_row + d), sum);
    }
    return sum;
}

// grid (ceil(max_q_len / warps), heads, sequences); block warps*32.
template <typename T, int kWarps>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_rows_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out, int out_row_stride,
                            const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                            const int* __restrict__ kv_lens, int heads, int kv_heads, int head_dim, int page_size,
                            int window, float scale) {
    extern __shared__ float q_shared_all[];  // kWarps * head_dim floats
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int q_begin = cu_q[seq];
    const int q_len = cu_q[seq + 1] - q_begin;
    const int j = blockIdx.x * kWarps + warp;
    if (j >= q_len) return;  // no block-wide barrier below, so a warp may leave alone
    const int kv_len = kv_lens[seq];
    const int pos = kv_len - q_len + j;
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int kv_head = head / (heads / kv_heads);
    const bool vector_ok = (head_dim % 8) == 0;

    float* q_shared = q_shared_all + warp * head_dim;
    const T* q_row = q + (size_t)(q_begin + j) * q_row_stride + (size_t)head * head_dim;
    for (int d = lane; d < head_dim; d += 32) q_shared[d] = Num<T>::load(q_row + d);
    __syncwarp();

    float acc[kAccPerLane];
#pragma unroll
    for (int i = 0; i < kAccPerLane; ++i) acc[i] = 0.0f;
    float running_max = -CUDART_INF_F, running_sum = 0.0f;
    const int* table = block_table + (size_t)seq * max_blocks;

    for (int chunk = first - (first % 32); chunk <= pos; chunk += 32) {
        // page_size is a multiple of 32, so a chunk of 32 positions lies in one page
        const size_t page = table[chunk / page_size];
        const size_t base = ((page * kv_heads + kv_head) * page_size + (chunk % page_size)) * head_dim;
        const int p = chunk + lane;
        const bool visible = p >= first && p <= pos;
        float score = -CUDART_INF_F;
        if (visible) score = dot_row<T>(q_shared, k_pool + base + (size_t)lane * head_dim, head_dim, vector_ok) * scale;
        const float chunk_max = warp_max(score);
        const float new_max = fmaxf(running_max, chunk_max);  // finite: position `pos` is visible in the last chunk,
                                                              // and earlier chunks hold at least one visible key
        const float e = visible ? expf(score - new_max) : 0.0f;
        const float correction = expf(running_max - new_max);  // exp(-inf) = 0 on the first chunk
        running_sum = running_sum * correction + warp_sum(e);
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < kAccPerLane; ++i) acc[i] *= correction;
        const int last = (pos - chunk < 31) ? pos - chunk : 31;
        const int begin = first > chunk ? first - chunk : 0;
        for (int jj = begin; jj <= last; ++jj) {
            const float prob = __shfl_sync(0xffffffffu, e, jj);
            const T* v_row = v_pool + base + (size_t)jj * head_dim;
#pragma unroll
            for (int i = 0; i < kAccPerLane; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(prob, Num<T>::load(v_row + d), acc[i]);
            }
        }
    }
    const float inv_sum = 1.0f / running_sum;
    T* out_row = out + (size_t)(q_begin + j) * out_row_stride + (size_t)head * head_dim;
#pragma unroll
    for (int i = 0; i < kAccPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) Num<T>::store(out_row + d, acc[i] * inv_sum);
    }
}

}  // namespace mb

using namespace mb;

// q: rows of `heads` heads (row stride in elements), out likewise.  cu_q[sequences + 1] are the
// first rows of each sequence's new tokens; kv_lens[sequences] the cache lengths including them.
MB_EXPORT int mb_paged_attention_rows(const void* q, int q_row_stride, void* out, int out_row_stride, int dtype,
                                      const void* k_pool, const void* v_pool, const int* block_table, int max_blocks,
                                      const int* cu_q, const int* kv_lens, int sequences, int max_q_len, int heads,
                                      int kv_heads, int head_dim, int page_size, int window, float scale,
                                      cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0) return 0;
    if (head_dim <= 0 || head_dim > kMaxHeadDim) return fail("paged_attention_rows: head_dim %d is outside 1..%d", head_dim, kMaxHeadDim);
    if (kv_heads <= 0 || heads % kv_heads) return fail("paged_attention_rows: %d heads are no multiple of %d kv heads", heads, kv_heads);
    if (page_size <= 0 || page_size % 32) return fail("paged_attention_rows: page_size %d must be a multiple of 32", page_size);
    if (sequences > 65535) return fail("paged_attention_rows: %d sequences exceed the grid limit 65535", sequences);
    if (heads > 65535) return fail("paged_attention_rows: %d heads exceed the grid limit 65535", heads);
    constexpr int kWarps = 4;
    const dim3 grid((max_q_len + kWarps - 1) / kWarps, heads, sequences);
    const size_t smem = (size_t)kWarps * head_dim * sizeof(float);
    if (dtype == MB_F32)
        paged_attention_rows_kernel<float, kWarps><<<grid, kWarps * 32, smem, stream>>>(
            (const float*)q, q_row_stride, (float*)out, out_row_stride, (const float*)k_pool, (const float*)v_pool,
            block_table, max_blocks, cu_q, kv_lens, heads, kv_heads, head_dim, page_size, window, scale);
    else if (dtype == MB_BF16)
        paged_attention_rows_kernel<__nv_bfloat16, kWarps><<<grid, kWarps * 32, smem, stream>>>(
            (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, out_row_stride, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, block_table, max_blocks, cu_q, kv_lens, heads, kv_heads, head_dim, page_size,
            window, scale);
    else
        return fail("paged_attention_rows: unknown dtype code %d", dtype);
    return check_launch("paged_attention_rows");
}
