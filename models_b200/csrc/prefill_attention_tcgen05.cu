// Prefill attention on the fifth-generation tensor cores: causal grouped-query attention of many new
// tokens over the paged cache, bfloat16 storage, float accumulation and softmax.  Compiled for one
// head size: -DMB_HEAD_DIM=64 or 128.
//
// A block takes 128 consecutive query tokens of one head and walks the visible cache pages (64 keys
// each).  Its six warps have three roles:
//   * warp 0, one thread: TMA.  The query tile once, then per page the key tile and the value tile
//     ([64 keys][head size], contiguous in the pool) into two rings of shared-memory stages (keys,
//     values), 128-byte swizzle.
//   * warp 1, one thread: tcgen05.mma.  S = Q . K^T (M = 128, N = 64 keys, K = head size) into one of
//     two score buffers in tensor memory, then O += P . V (M = 128, N = head size, K = 64 keys,
//     V read as an MN-major operand) into the output accumulator, which stays in tensor memory over
//     all pages.  The scores of page t + 1 are issued before the softmax of page t has finished, so
//     the tensor cores and the softmax overlap.
//   * warps 2..5, one thread per query row: the running softmax.  A thread reads its row of scores
//     with tcgen05.ld, masks, takes the maximum, exponentiates (special-function exp2 with the scale
//     folded into the exponent, two floats per instruction around it) and writes the probabilities
//     as bfloat16 pairs over its scores in tensor memory (tcgen05.st), from where the next product
//     takes them as its A operand: they never pass through shared memory.  The base of
//     the exponents follows the running maximum lazily; only when it moves is the accumulator read
//     back, rescaled and stored again (tcgen05.ld / tcgen05.st).  At the end the thread divides its
//     row by the sum and stores it.  No shuffles: a row never leaves its thread.
//
// Formula: integrallis/models, backend-java/.../llama/LlamaForwardPass.java:1543-1670 (kvHead = head /
// group; dot first, then scale; only positions <= the query's are read; with a window of n only the n
// positions that end at the query) and backend-java/.../ops/TensorOps.java:1247-1279 (softmax), in its
// running form.  Probabilities enter the P . V product as bfloat16: scaled up by 1 + 2^-9 and truncated, which errs
// like rounding to nearest (the sum takes the same scaled values, and the factor is divided out at the end).
//
// Every mbarrier wait is bounded (about two seconds); a role that gives up records where, all roles
// meet at the final barrier, tensor memory is freed and the kernel returns.
// mb_prefill_attention_tc_status() reads the record.
#include "tcgen05.cuh"

#include <math_constants.h>

#ifndef MB_HEAD_DIM
#error "compile with -DMB_HEAD_DIM=64 or 128"
#endif

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int HD = MB_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "this kernel is built for head sizes 64 and 128");
constexpr int kQRows = 128;               // query tokens per block
constexpr int kKeys = 64;                 // keys per step: one cache page
constexpr int kBoxes = HD / 64;           // 64-column TMA boxes per row of a tile
constexpr int kQBoxBytes = kQRows * 128;  // [128 rows][64 columns]
constexpr int kQBytes = kBoxes * kQBoxBytes;
constexpr int kKVBoxBytes = kKeys * 128;  // [64 keys][64 columns]
constexpr int kKVTileBytes = kBoxes * kKVBoxBytes;
constexpr int kStages = HD == 64 ? 3 : 2;      // of the key ring and of the value ring, each
// Of every four pairs of probabilities, so many are exponentiated by arithmetic (soft_exp2_x2) instead of the
// special-function unit, which gives 16 results a clock and multiprocessor and is the busiest pipe of this kernel
// (66 % of its cycles at heads of 64).  Measured at 2,048 / 8,192 tokens, heads of 64: none 477 / 726 TFLOP/s, one
// 498 / 737, two 461 / 700, three 424 / 634: past one pair the added instructions cost more than the unit gains.
constexpr int kSoftPairs = HD == 64 ? 1 : 0;
constexpr int kCols = kKeys;                   // keys of a page per softmax thread: a thread takes its whole row
constexpr int kSoftmaxWarps = 4;
constexpr int kThreads = 64 + 32 * kSoftmaxWarps;
constexpr int kScoreColumns = 64;
constexpr int kTmemColumns = 256;  // two score buffers and the output: 2 * 64 + HD
static_assert(2 * kScoreColumns + HD <= kTmemColumns, "tensor memory budget");
constexpr float kSlack = 8.0f;     // how far (in the exponent) the maximum may run ahead of the base
constexpr size_t kSmemBytes = (size_t)kQBytes + 2 * (size_t)kStages * kKVTileBytes + 1024;

constexpr uint32_t kScoreInstruction = instruction_descriptor(kQRows, kKeys);
constexpr uint32_t kOutputInstruction = instruction_descriptor(kQRows, HD) | (1u << 16);  // B is MN-major

// MN-major operand with 128-byte swizzle: 64 elements of the MN extent are contiguous (one 128-byte
// row per step of K), 8-row groups along K are 1024 bytes apart, and further 64-element blocks of
// the MN extent are `block_bytes` apart.
__device__ __forceinline__ uint64_t umma_descriptor_mn(uint32_t smem_addr, uint32_t block_bytes) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    desc |= (uint64_t)(block_bytes >> 4) << 16;  // leading byte offset
    desc |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    return desc;
}

__device__ __forceinline__ void tmem_load_32_raw(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_loads() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_store_32_raw(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_stores() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// two floats in one 64-bit register, and arithmetic on both at once
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// 2^x for two floats at once without the special-function unit: x = n + f with n the nearest integer (the
// magic-number addition leaves n in the low mantissa bits) and f in [-0.5, 0.5]; 2^f by a cubic (relative error 1e-4,
// a twentieth of the rounding to bfloat16 that follows); n is added into the exponent bits.  x below -126 counts as -126.
__device__ __forceinline__ void soft_exp2_x2(uint64_t x2, float& e0, float& e1) {
    float x0, x1;
    unpack_f32x2(x2, x0, x1);
    const uint64_t x = pack_f32x2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
    const uint64_t magic = pack_f32x2(12582912.0f, 12582912.0f), minus_magic = pack_f32x2(-12582912.0f, -12582912.0f);
    const uint64_t minus_one = pack_f32x2(-1.0f, -1.0f), one = pack_f32x2(1.0f, 1.0f);
    const uint64_t c1 = pack_f32x2(0.69328290f, 0.69328290f), c2 = pack_f32x2(0.24221095f, 0.24221095f), c3 = pack_f32x2(0.05500893f, 0.05500893f);
    const uint64_t r = add_f32x2(x, magic);
    const uint64_t f = fma_f32x2(add_f32x2(r, minus_magic), minus_one, x);
    const uint64_t p = fma_f32x2(fma_f32x2(fma_f32x2(c3, f, c2), f, c1), f, one);
    float r0, r1, p0, p1;
    unpack_f32x2(r, r0, r1);
    unpack_f32x2(p, p0, p1);
    e0 = __uint_as_float(__float_as_uint(p0) + (__float_as_uint(r0) << 23));
    e1 = __uint_as_float(__float_as_uint(p1) + (__float_as_uint(r1) << 23));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// The upper halves of two floats as a pair of bfloat16 (one byte permutation; a conversion instruction would
// queue behind the exponentials on the special-function unit).  This truncates: the softmax below feeds it
// probabilities scaled up by 1 + 2^-9, which centres the truncation error on zero like rounding to nearest.
__device__ __forceinline__ uint32_t upper_halves(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}
constexpr float kTruncationLift = 0.0028150156f;  // log2(1 + 2^-9)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// tcgen05.mma with the 128 x 16 A operand in tensor memory (lane = row, two bfloat16 per 32-bit column)
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t instruction, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(instruction), "r"(accumulate)
        : "memory");
}

struct AttentionArgs {
    bf16* out;
    int out_row_stride;
    const int* block_table;
    int max_blocks;
    const int* cu_q;
    const int* kv_lens;
    int heads, kv_heads, window;
    float scale;
};

// roles in the status record: 1 TMA (stage free), 2 MMA (queries), 3 MMA (keys), 4 MMA (probabilities),
// 5 softmax (scores), 6 softmax (output of a page)
__global__ void __launch_bounds__(kThreads, 2)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const AttentionArgs args) {
    // blocks start in the order of their index: all heads of the query tile with the most keys first, then
    // the next tile, so that the long blocks are under way early and the short ones fill the end
    const int seq = blockIdx.z, head = blockIdx.x;
    const int q_begin = args.cu_q[seq], q_len = args.cu_q[seq + 1] - q_begin;  // written before the step, by a copy
    const int q_tile = gridDim.y - 1 - blockIdx.y;
    const int t0 = q_tile * kQRows;
    if (t0 >= q_len) return;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t barriers[4 * kStages + 7];
    __shared__ uint32_t tmem_base_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_smem = smem_u32(smem);
    // keys and values have rings of their own: a key tile is free as soon as its scores are computed,
    // a value tile only after the softmax of its page, and the next keys must not wait for that
    const uint32_t k_smem = q_smem + kQBytes, v_smem = k_smem + kStages * kKVTileBytes;
    const uint32_t k_full = smem_u32(&barriers[0]), k_empty = smem_u32(&barriers[kStages]);
    const uint32_t v_full = smem_u32(&barriers[2 * kStages]), v_empty = smem_u32(&barriers[3 * kStages]);
    const uint32_t q_full = smem_u32(&barriers[4 * kStages]);
    const uint32_t s_full = smem_u32(&barriers[4 * kStages + 1]);  // two
    const uint32_t p_full = smem_u32(&barriers[4 * kStages + 3]);  // two
    const uint32_t o_full = smem_u32(&barriers[4 * kStages + 5]);  // two

    const int valid = min(kQRows, q_len - t0);
    const int kv_len = args.kv_lens[seq];
    const int pos0 = kv_len - q_len + t0;  // position of the tile's first token
    const int last_pos = pos0 + valid - 1;
    const int window = args.window;
    const int first_needed = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int t_begin = first_needed / kKeys, t_end = last_pos / kKeys + 1;
    const int pages = t_end - t_begin;
    const int kv_head = head / (args.heads / args.kv_heads);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1);
            mbar_init(v_empty + 8 * s, 1);
        }
        mbar_init(q_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full + 8 * b, 1);
            mbar_init(p_full + 8 * b, kSoftmaxWarps);  // one arrival per softmax warp
            mbar_init(o_full + 8 * b, 1);
        }

        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemColumns));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t tmem_scores = tmem_base, tmem_output = tmem_base + 2 * kScoreColumns;  // output: one buffer, all pages
    grid_launch_dependents();
    grid_dependency_wait();  // queries, and the newest keys and values, come from the kernel before this one

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(q_full, kQBytes);
#pragma unroll
            for (int b = 0; b < kBoxes; ++b) tma_load_2d(q_smem + b * kQBoxBytes, &map_q, head * HD + b * 64, q_begin + t0, q_full);
            const int* table = args.block_table + (size_t)seq * args.max_blocks;
            for (int t = 0; t < pages; ++t) {
                const int stage = t % kStages;
                const uint32_t free_parity = ((t / kStages) & 1) ^ 1;
                const int row = (table[t_begin + t] * args.kv_heads + kv_head) * kKeys;
                if (!mbar_wait(k_empty + 8 * stage, free_parity, 1)) break;
                mbar_expect_tx(k_full + 8 * stage, kKVTileBytes);
#pragma unroll
                for (int b = 0; b < kBoxes; ++b)
                    tma_load_2d(k_smem + stage * kKVTileBytes + b * kKVBoxBytes, &map_k, b * 64, row, k_full + 8 * stage);
                if (!mbar_wait(v_empty + 8 * stage, free_parity, 1)) break;
                mbar_expect_tx(v_full + 8 * stage, kKVTileBytes);
#pragma unroll
                for (int b = 0; b < kBoxes; ++b)
                    tma_load_2d(v_smem + stage * kKVTileBytes + b * kKVBoxBytes, &map_v, b * 64, row, v_full + 8 * stage);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            auto issue_scores = [&](int t) {  // S[t % 2] = Q . K(t)^T
                const uint32_t k_tile = k_smem + (t % kStages) * kKVTileBytes;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint64_t a_desc = umma_descriptor(q_smem + (ks / 4) * kQBoxBytes) + 2 * (ks % 4);
                    const uint64_t b_desc = umma_descriptor(k_tile + (ks / 4) * kKVBoxBytes) + 2 * (ks % 4);
                    umma(tmem_scores + (t & 1) * kScoreColumns, a_desc, b_desc, kScoreInstruction, ks > 0 ? 1u : 0u);
                }
                umma_commit(s_full + 8 * (t & 1));
                umma_commit(k_empty + 8 * (t % kStages));  // the key tile is free once these products have read it
            };
            bool ok = mbar_wait(q_full, 0, 2) && mbar_wait(k_full, 0, 3);
            if (ok) {
                tcgen05_fence_after();
                issue_scores(0);
            }
            for (int t = 0; t < pages && ok; ++t) {
                if (t + 1 < pages) {
                    if (!(ok = mbar_wait(k_full + 8 * ((t + 1) % kStages), ((t + 1) / kStages) & 1, 3))) break;
                    tcgen05_fence_after();
                    issue_scores(t + 1);
                }
                if (!(ok = mbar_wait(p_full + 8 * (t & 1), (t >> 1) & 1, 4))) break;
                if (!(ok = mbar_wait(v_full + 8 * (t % kStages), (t / kStages) & 1, 3))) break;
                tcgen05_fence_after();
                const uint32_t v_tile = v_smem + (t % kStages) * kKVTileBytes;
                const uint32_t p_tile = tmem_scores + (t & 1) * kScoreColumns;  // the probabilities lie over the scores they came from
#pragma unroll
                for (int j = 0; j < kKeys / 16; ++j)  // 16 keys per instruction: 8 columns of P, 16 rows of V
                    umma_a_tmem(tmem_output, p_tile + 8 * j, umma_descriptor_mn(v_tile + j * 16 * 128, kKVBoxBytes),
                                kOutputInstruction, (t > 0 || j > 0) ? 1u : 0u);
                umma_commit(o_full + 8 * (t & 1));
                umma_commit(v_empty + 8 * (t % kStages));
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax: one thread per query row
        const int quarter = warp & 3;  // the quarter of the tensor-memory lanes this warp may read
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t my_output = tmem_output + lane_base;
        const int row_pos = row < valid ? pos0 + row : -1;  // a row beyond the sequence sees nothing
        const int row_first = (window > 0 && row_pos - window + 1 > 0) ? row_pos - window + 1 : 0;
        const float scale_log2 = args.scale * 1.4426950408889634f;
        const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
        // `base` is the score the exponents are taken against.  It follows the running maximum lazily:
        // it moves (and the output so far is rescaled) only when the maximum has grown by more than
        // kSlack in the exponent, so most pages cost no pass over the output.  Until then the
        // probabilities of later pages may exceed 1, by at most 2^kSlack; sum and output share the base,
        // so their quotient is the same.
        float base = -CUDART_INF_F, run_sum = 0.0f;
        bool ok = true;
        for (int t = 0; t < pages; ++t) {
            ok = mbar_wait(s_full + 8 * (t & 1), (t >> 1) & 1, 5);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            uint32_t s[kCols];
            const uint32_t my_scores = tmem_scores + (t & 1) * kScoreColumns + lane_base;
#pragma unroll
            for (int c = 0; c < kCols; c += 32) tmem_load_32_raw(my_scores + c, &s[c]);
            tmem_wait_loads();
            const int key_base = (t_begin + t) * kKeys;
            if (!(key_base + kCols - 1 <= row_pos && key_base >= row_first)) {  // not the whole page is visible to this row
#pragma unroll
                for (int i = 0; i < kCols; ++i) {
                    const int key = key_base + i;
                    if (!(key <= row_pos && key >= row_first)) s[i] = __float_as_uint(-CUDART_INF_F);
                }
            }
            float part[8];  // eight chains, two more scores a step
#pragma unroll
            for (int i = 0; i < 8; ++i) part[i] = fmaxf(__uint_as_float(s[i]), __uint_as_float(s[8 + i]));
#pragma unroll
            for (int i = 16; i < kCols; i += 16)
#pragma unroll
                for (int j = 0; j < 8; ++j) part[j] = max3(part[j], __uint_as_float(s[i + j]), __uint_as_float(s[i + 8 + j]));
            const float page_max = max3(max3(part[0], part[1], part[2]), max3(part[3], part[4], part[5]), fmaxf(part[6], part[7]));
            // scores stay raw; the scale (times log2 e) is folded into the exponent: 2^(s*c - base*c)
            float factor = 1.0f;
            if (base == -CUDART_INF_F) {
                base = page_max;  // nothing accumulated so far (or still nothing visible)
            } else if ((page_max - base) * scale_log2 > kSlack) {
                factor = fast_exp2((base - page_max) * scale_log2);
                base = page_max;
            }
            run_sum *= factor;
            // a row that has seen nothing yet keeps -inf; subtract 0 then so that the exponent is -inf, not NaN
            const float offset = base == -CUDART_INF_F ? 0.0f : fmaf(-base, scale_log2, kTruncationLift);
            const uint64_t offset2 = pack_f32x2(offset, offset);
            uint64_t sums[4] = {0ull, 0ull, 0ull, 0ull};  // eight partial sums, two per register pair
            uint32_t packed[kCols / 2];
#pragma unroll
            for (int c = 0; c < kCols / 8; ++c) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(s[c * 8 + 2 * i]), __uint_as_float(s[c * 8 + 2 * i + 1])), scale2, offset2);
                    float e0, e1;
                    if (i < kSoftPairs) {
                        soft_exp2_x2(x2, e0, e1);
                    } else {
                        float x0, x1;
                        unpack_f32x2(x2, x0, x1);
                        e0 = fast_exp2(x0);
                        e1 = fast_exp2(x1);
                    }
                    sums[i] = add_f32x2(sums[i], pack_f32x2(e0, e1));
                    packed[c * 4 + i] = upper_halves(e0, e1);
                }
            }
            // the row's probabilities go where its scores were: the next product takes them from tensor memory
            tmem_store_32_raw(my_scores, packed);
            {
                float lo, hi;
                unpack_f32x2(add_f32x2(add_f32x2(sums[0], sums[1]), add_f32x2(sums[2], sums[3])), lo, hi);
                run_sum += lo + hi;
            }
            if (__any_sync(0xffffffffu, factor != 1.0f)) {
                // the output so far moves to the new base (the product of the page before must have landed) before the
                // product of this page adds to it; the scores' registers are free by now
                ok = mbar_wait(o_full + 8 * ((t - 1) & 1), ((t - 1) >> 1) & 1, 6);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t r[32];
                    tmem_load_32_raw(my_output + c, r);
                    tmem_wait_loads();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                    tmem_store_32_raw(my_output + c, r);
                }
                tmem_wait_stores();
            }
            tmem_wait_stores();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * (t & 1));
        }
        if (ok) {
            ok = mbar_wait(o_full + 8 * ((pages - 1) & 1), ((pages - 1) >> 1) & 1, 6);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tcgen05_fence_after();
            const float inv = exp2f(kTruncationLift) / run_sum;  // the sum holds the lifted probabilities, the products their truncations
            bf16* dst = args.out + (size_t)(q_begin + t0 + row) * args.out_row_stride + (size_t)head * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                uint32_t r[32];
                tmem_load_32_raw(my_output + c, r);
                tmem_wait_loads();
                if (row < valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float piece[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) piece[j] = __uint_as_float(r[i + j]) * inv;
                        store8(dst + c + i, piece);
                    }
                }
            }
        }
    }

    // every role has left its loop (done, or after a bounded wait gave up): free tensor memory
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
    }
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_prefill_attention_tc_head_dim() { return HD; }

// q: bfloat16 rows (row stride q_row_stride) of total_rows tokens, head h at columns [h * HD, +HD); out likewise.
// k_pool, v_pool: bfloat16 [pages][kv_heads][64][HD].  block_table: int32 [sequences][max_blocks];
// cu_q: int32 [sequences + 1]; kv_lens: int32 [sequences] (the new tokens included).
MB_EXPORT int mb_prefill_attention_tcgen05(const void* q, int q_row_stride, int total_rows, void* out, int out_row_stride,
                                           const void* k_pool, const void* v_pool, int pool_pages, const int* block_table,
                                           int max_blocks, const int* cu_q, const int* kv_lens, int sequences, int max_q_len,
                                           int heads, int kv_heads, int page_size, int window, float scale,
                                           cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0) return 0;
    if (kv_heads <= 0 || heads % kv_heads) return fail("prefill_attention_tcgen05: %d heads are no multiple of %d kv heads", heads, kv_heads);
    if (page_size != kKeys) return fail("prefill_attention_tcgen05: the cache page must hold %d positions, got %d", kKeys, page_size);
    if (q_row_stride % 8 || out_row_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15))
        return fail("prefill_attention_tcgen05: query and output rows must start on 16-byte boundaries");
    if (((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15)) return fail("prefill_attention_tcgen05: the cache pools must start on 16-byte boundaries");
    if (sequences > 65535 || (max_q_len + kQRows - 1) / kQRows > 65535) return fail("prefill_attention_tcgen05: grid too large");
    if ((long long)pool_pages * kv_heads * kKeys > 0x7fffffffLL) return fail("prefill_attention_tcgen05: the cache pool has too many rows for one map");
    CUtensorMap map_q, map_k, map_v;
    if (int status = make_map(&map_q, q, total_rows, heads * HD, q_row_stride, kQRows)) return status;
    if (int status = make_map(&map_k, k_pool, pool_pages * kv_heads * kKeys, HD, HD, kKeys)) return status;
    if (int status = make_map(&map_v, v_pool, pool_pages * kv_heads * kKeys, HD, HD, kKeys)) return status;
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(prefill_attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (status != cudaSuccess)
            return fail("prefill_attention_tcgen05: cannot reserve %zu bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(status));
        configured = true;
    }
    AttentionArgs args{(bf16*)out, out_row_stride, block_table, max_blocks, cu_q, kv_lens, heads, kv_heads, window, scale};
    const dim3 grid(heads, (max_q_len + kQRows - 1) / kQRows, sequences);
    return launch_dependent("prefill_attention_tcgen05", prefill_attention_tcgen05_kernel, grid, dim3(kThreads), kSmemBytes, stream,
                            true, map_q, map_k, map_v, args);
}

// 0 when no wait ever gave up; else 1 + (role << 8).
MB_EXPORT int mb_prefill_attention_tc_status() {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    return status;
}
