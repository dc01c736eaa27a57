// The tile machinery of the tensor-core attention kernels, shared by csrc/attention_tc.cu and the fused
// decode step (csrc/decode_step.cu): a tile is the 64 positions of one cache page of one kv head,
// [64][head size] contiguous in the pool, brought to shared memory with cp.async into rows padded by 16
// bytes so that ldmatrix reads are conflict-free; scores and outputs are m16n8k16 products.
// Compiled for one head size: -DMB_HEAD_DIM=<multiple of 16>.
#pragma once

#include "common.cuh"

#include <math_constants.h>

#ifndef MB_HEAD_DIM
#error "compile with -DMB_HEAD_DIM=<head size>"
#endif

namespace mb {

constexpr int HD = MB_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 in 16..256");
constexpr int kTile = 64;                 // keys per tile, one cache page
constexpr int kRowBytes = HD * 2 + 16;    // padded shared-memory row
constexpr int kTileBytes = kTile * kRowBytes;
constexpr int kChunks = HD / 8;           // 16-byte pieces of a row
constexpr int kKSteps = HD / 16;
constexpr int kThreads = 128;
constexpr int kQRowsDecode = 16;
// Pages of keys and values in shared memory per decode block: two or three, chosen at launch (mb_decode_stages; six for
// a few blocks over long contexts, see decode_stages).
// A third stage helps where a block has only a few pages -- all of them are then in flight at once; with four blocks
// of three stages per sequence, batch 8 of the 1B model gains 2 % over eight blocks of two -- and at head sizes of 96
// and more (64 sequences of 1,280 positions at head size 128: 4.3 -> 5.2 TB/s).  With heads of 64 and long loops it
// costs a resident block per multiprocessor and loses (batch 64: 49.7 -> 46.6 k tokens/s), and eight blocks of three
// stages per sequence no longer fit one round at batch 8 (9.2 -> 8.3 k tokens/s).
constexpr int kQRowsPrefill = 64;

using bf16 = __nv_bfloat16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// One page of one kv head -> a padded tile in shared memory (all threads of the block).
__device__ __forceinline__ void load_tile(uint32_t dst, const bf16* __restrict__ pool, size_t page, int kv_head,
                                          int kv_heads) {
    const bf16* src = pool + (page * kv_heads + kv_head) * (size_t)(kTile * HD);
    static_assert((kTile * kChunks) % kThreads == 0, "every thread copies the same number of pieces");
#pragma unroll
    for (int j = 0; j < kTile * kChunks / kThreads; ++j) {  // (unrolled: the offsets are the same for every page)
        const int i = threadIdx.x + j * kThreads;
        const int row = i / kChunks, chunk = i % kChunks;
        cp_async16(dst + row * kRowBytes + chunk * 16, src + row * HD + chunk * 8);
    }
}

// The 16 rows of a page that one decode warp works on (rows 16 * warp ...), copied by that warp alone: what a warp
// reads it has fetched itself, so the warps of a block need no barrier between pages.
__device__ __forceinline__ void load_tile_rows(uint32_t dst, const bf16* __restrict__ pool, size_t page, int kv_head,
                                               int kv_heads, int warp, int lane) {
    const bf16* src = pool + (page * kv_heads + kv_head) * (size_t)(kTile * HD) + (size_t)warp * 16 * HD;
    dst += warp * 16 * kRowBytes;
#pragma unroll
    for (int j = 0; j < 16 * kChunks / 32; ++j) {
        const int i = lane + j * 32;
        const int row = i / kChunks, chunk = i % kChunks;
        cp_async16(dst + row * kRowBytes + chunk * 16, src + row * HD + chunk * 8);
    }
}

// Rows of queries -> padded rows in shared memory; rows >= valid are zero.
__device__ __forceinline__ void load_queries(unsigned char* dst, const bf16* __restrict__ q_first_row, size_t row_stride,
                                             int rows, int valid) {
    for (int i = threadIdx.x; i < rows * kChunks; i += kThreads) {
        const int row = i / kChunks, chunk = i % kChunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < valid) v = *reinterpret_cast<const uint4*>(q_first_row + (size_t)row * row_stride + chunk * 8);
        *reinterpret_cast<uint4*>(dst + row * kRowBytes + chunk * 16) = v;
    }
}

// Query fragments of one warp's 16 rows for every 16-wide step over the head.
__device__ __forceinline__ void load_q_fragments(uint32_t (&a)[kKSteps][4], uint32_t q_rows_base) {
    const int lane = threadIdx.x & 31;
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) ldmatrix_x4(a[ks], q_rows_base + row * kRowBytes + (ks * 2 + (lane >> 4)) * 16);
}

// S[16 x 16 keys] for keys key0..key0+15 of a tile: two 8-key accumulators.
__device__ __forceinline__ void scores_16_keys(float (&s)[2][4], const uint32_t (&a)[kKSteps][4], uint32_t k_tile, int key0) {
    const int lane = threadIdx.x & 31;
    const int key = key0 + (lane & 7) + ((lane >> 4) & 1) * 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) s[0][i] = s[1][i] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
        uint32_t b[4];
        ldmatrix_x4(b, k_tile + key * kRowBytes + (ks * 2 + ((lane >> 3) & 1)) * 16);
        mma_bf16(s[0], a[ks], b[0], b[1]);
        mma_bf16(s[1], a[ks], b[2], b[3]);
    }
}

// O[16 x HD] += P[16 x 16 keys] . V[16 keys x HD]
__device__ __forceinline__ void accumulate_16_keys(float (&o)[HD / 8][4], const uint32_t (&p)[4], uint32_t v_tile, int key0) {
    const int lane = threadIdx.x & 31;
    const int key = key0 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_tile + key * kRowBytes + (dp * 2 + (lane >> 4)) * 16);
        mma_bf16(o[2 * dp], p, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], p, b[2], b[3]);
    }
}

// 2^x by the special-function unit (about two units in the last place; the probabilities it feeds are
// rounded to bfloat16 afterwards).  2^-inf = 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

}  // namespace mb
