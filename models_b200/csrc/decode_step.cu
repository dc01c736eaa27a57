// One decode step of a whole model -- every layer, final norm and output matrix -- as ONE kernel,
// for up to 8 sequences of one new token each (bfloat16 weights and cache, float accumulation).
//
// A decode step at small batch reads every weight once and computes next to nothing: it is as fast as
// the weights stream.  Run as a kernel per matrix (csrc/skinny_gemm.cu, five per layer) the stream
// stops at every kernel boundary: the next kernel waits for the one before it, stages its activations,
// and only then are its loads in flight again -- about as long as the streaming itself takes.  Here
// the blocks are persistent (one per multiprocessor, launched cooperatively so that all are resident)
// and walk a list of PHASES:
//     embed | per layer: q/k/v -> attention -> output -> gate/up -> down | head
// Every warp keeps a private ring of weight stages filled with cp.async that runs on ACROSS tiles and
// phases: weights never depend on the step's activations, so while the blocks meet at the barrier
// between two phases, and while they stage the next phase's activations, the next weights are already
// on their way.  Between phases the blocks meet at a barrier in global memory (an arrival counter;
// every wait is bounded and ends the kernel with a status instead of hanging).
//
// A matrix phase is the decode product of csrc/skinny_gemm.cu with eight warps: a block owns row tiles
// of 16 weight rows (8 pairs for the gated and the rotary epilogue), its warps split K, partial sums
// are added in warp order (no result depends on timing), and what surrounds the product rides in it:
//   q/k/v    RMSNorm of the float32 residual rows on the way in (sumSq/size + eps, sqrt, 1/rms:
//            integrallis/models, backend-java/.../ops/TensorOps.java:45-58); rotation of query and key
//            pairs (x0' = x0*c - x1*s, x1' = x0*s + x1*c, :1481-1486) and the paged cache write of keys
//            and values on the way out (backend-java/.../llama/LlamaForwardPass.java:1070-1086)
//   output   the attention's split partial results are combined while they are staged; x += W.a (:1131-1138)
//   gate/up  RMSNorm on the way in, act(gate) * up on the way out (:1150-1170)
//   down     x += W.h (:1172-1178); a K too long for a block's shared memory runs as several sub-phases
//            over column ranges, each adding into the rows the block owns (no barrier between them)
//   head     final RMSNorm on the way in, float32 logits out (:1184-1196)
// The attention phase is the split-key decode attention of csrc/attention_tc.cu on the same tile
// machinery (attention_tiles.cuh): work items are (sequence, kv head, split of the keys).
//
// Compiled per head size: -DMB_HEAD_DIM=<multiple of 16, at most 128>.
#include "attention_tiles.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kStepWarps = 8;
constexpr int kStepThreads = kStepWarps * 32;
constexpr int kCols = 8;              // activation rows of a step = columns of the MMA
constexpr int kStageCols = 64;        // columns of K per ring stage
constexpr int kStageBytes = 2 * 2 * 32 * 16;  // [2 row halves][2 pieces][32 lanes][16 bytes]
constexpr int kDepth = 8;             // ring stages per warp
constexpr int kSliceCols = kStepWarps * kStageCols;  // K is padded to a multiple of this
constexpr int kMaxStageCols = 4096;   // most columns of one (sub-)phase: its activations must fit shared memory
constexpr int kMaxGroups = 4;
constexpr int kAttnWarps = HD <= 64 ? 8 : 4;  // warps that work in the attention phase (their page rings must fit)
constexpr int kAttnStages = 2;
constexpr int kAttnStageBytes = 2 * 16 * kRowBytes;  // a warp's 16 rows of a key page and of a value page
constexpr long kSpinLimit = 4L * 1000 * 1000;  // polls of the barrier counter before a block gives up (a second or so)
static_assert(HD <= 128, "the fused decode step is built for head sizes up to 128");

enum { PH_EMBED = 0, PH_QKV = 1, PH_ATTN = 2, PH_OUT = 3, PH_GATE_UP = 4, PH_DOWN = 5, PH_HEAD = 6 };

// One phase of the step.  The array of phases is the model: it is built once, in device memory.
struct Phase {
    int kind;
    int barrier_before;   // the phase reads what another block wrote in the phase before it: all blocks meet first
    const bf16* w;        // first weight row, at the first column of this (sub-)phase
    int ldw;              // weight row stride in elements
    int rows;             // rows of output (gate/up: gate rows; q/k/v: all of them)
    int tiles;            // row tiles: 16 rows, or 8 pairs
    int k_len;            // columns of this (sub-)phase, a multiple of 8
    int k_pad;            // k_len rounded up to kSliceCols
    int k_begin;          // first column of the activation row that this sub-phase covers
    int pair_offset;      // gate/up: first up row
    int activation;       // gate/up: MB_ACT_*
    float eps;            // norm prologue
    const float* gain;    // norm prologue: [k_len]; null for none
    int group;            // cache group of the layer: which page tables and slot mapping of the step
    int heads, kv_heads, window;
    float scale;
    bf16* k_pool;         // [pages][kv_heads][64][HD]
    bf16* v_pool;
    const float* cos_table;  // [positions][HD / 2]
    const float* sin_table;
};

// What changes from step to step; passed by value.
struct Step {
    const Phase* phases;
    int num_phases;
    int batch;            // sequences = rows, 1..8
    int hidden;
    const int* tokens;    // [batch]
    const int* positions; // [batch]
    const int* kv_lens;   // [batch] cached positions after this step
    const bf16* embedding;
    float embedding_scale;
    int max_blocks;       // width of the page tables
    const int* block_tables[kMaxGroups];   // [batch][max_blocks]
    const int* slot_mappings[kMaxGroups];  // [batch] flat cache position of the new token, < 0: do not store
    int splits[kMaxGroups];                // blocks that share one sequence's keys, per group
    float* x;             // [batch][hidden] the residual stream
    bf16* q;              // [batch][ld_q] rotated queries
    int ld_q;
    bf16* h;              // [batch][ld_h] gated activations
    int ld_h;
    float* attn_o;        // [batch][heads][splits][HD] partial outputs of the split keys
    float* attn_ml;       // [batch][heads][splits][2] their (maximum as an exponent of two, sum)
    float* logits;        // [batch][ld_logits]
    int ld_logits;
    unsigned int* barrier;  // arrival counter, zero at launch
    int* status;            // set to 1 + (phase << 8) by a block whose bounded wait ran out
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128_zero(uint32_t addr) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(addr), "r"(0u) : "memory");
}
__device__ __forceinline__ void cp_async16_mem(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_mem() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_mem() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Shared memory of a block, in bytes from the start:
//   activations  [8 rows][k_pad * 2 + 64]   (row stride = 64 mod 128: the eight rows a quarter-warp reads fall on
//                different banks); the attention phase has its query tile and page rings here instead
//   rings        [8 warps][kDepth][kStageBytes]
//   partial      [2 buffers][8 warps][16 rows][8 columns] floats
//   sums         [8] sums of squares of the rows, then [8 warps][8] the warps' parts of them
constexpr int kAttnBytes = kQRowsDecode * kRowBytes + kAttnWarps * kAttnStages * kAttnStageBytes;
constexpr int kMergeBytes = kQRowsDecode * kRowBytes + kAttnWarps * 16 * (HD + 2) * (int)sizeof(float);
constexpr int kActivationBytes = kCols * (kMaxStageCols * 2 + 64);
constexpr int max3(int a, int b, int c) { return a > b ? (a > c ? a : c) : (b > c ? b : c); }
constexpr int kFrontBytes = (max3(kAttnBytes, kMergeBytes, kActivationBytes) + 127) / 128 * 128;
constexpr int kRingBytes = kStepWarps * kDepth * kStageBytes;
constexpr int kPartialFloats = kStepWarps * 16 * kCols;
constexpr int kSmemBytes = kFrontBytes + kRingBytes + (2 * kPartialFloats + kCols + kStepWarps * kCols) * (int)sizeof(float);

// Where a warp's weight stream stands: the phases, the block's tiles of a phase and the warp's steps over its slice
// of K, flattened into one sequence of stages.  The producer runs kDepth - 1 stages ahead of the consumer.
struct Stream {
    int phase;        // index of the phase the next stage belongs to; num_phases when the stream has ended
    int tile;         // row tile of that stage
    int step;         // 64-column step within the warp's slice
    int steps;        // steps of the slice in this phase
    int kind, rows, tiles, pair_offset, ldw;
    int k0, k1;       // the warp's columns [k0, k1) of the (sub-)phase
    const bf16* w;
};

__device__ __forceinline__ int slice_steps(const Phase& p, int warp, int* k0, int* k1) {
    const int per_warp = p.k_pad / kStepWarps;
    *k0 = min(p.k_len, warp * per_warp);
    *k1 = min(p.k_len, *k0 + per_warp);
    return (*k1 - *k0 + kStageCols - 1) / kStageCols;
}

// Moves the stream to the first stage at or after phase `from` (a matrix phase in which this block has a tile and
// this warp a slice of K).
__device__ __forceinline__ void stream_seek(Stream& s, const Step& step, int from, int warp) {
    for (int ph = from; ph < step.num_phases; ++ph) {
        const Phase& p = step.phases[ph];
        if (p.kind == PH_EMBED || p.kind == PH_ATTN || (int)blockIdx.x >= p.tiles) continue;
        int k0, k1;
        const int steps = slice_steps(p, warp, &k0, &k1);
        if (steps == 0) continue;
        s.phase = ph; s.tile = blockIdx.x; s.step = 0; s.steps = steps;
        s.kind = p.kind; s.rows = p.rows; s.tiles = p.tiles; s.pair_offset = p.pair_offset; s.ldw = p.ldw;
        s.k0 = k0; s.k1 = k1; s.w = p.w;
        return;
    }
    s.phase = step.num_phases;
}

// Issues the loads of the stream's next stage into ring slot `slot` and moves the stream on.  Always one commit
// group, also when the stream has ended: the consumer's waits count groups.
__device__ __forceinline__ void stream_produce(Stream& s, const Step& step, uint32_t ring, int slot, int warp, int lane) {
    if (s.phase < step.num_phases) {
        const int group_id = lane >> 2, tid4 = lane & 3;
        const uint32_t stage = ring + slot * kStageBytes;
        const int kc = s.k0 + s.step * kStageCols + 8 * tid4;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // MMA rows group_id and group_id + 8: 16 consecutive weight rows, or 8 rows and their partners
            int row;
            if (s.kind == PH_GATE_UP) {
                row = min(s.rows - 1, s.tile * 8 + group_id) + h * s.pair_offset;
            } else if (s.kind == PH_QKV) {  // tile = (head, eighth of its first half); the partner lies half a head further
                constexpr int tiles_per_head = HD / 16;
                row = (s.tile / tiles_per_head) * HD + (s.tile % tiles_per_head) * 8 + group_id + h * (HD / 2);
            } else {
                row = min(s.rows - 1, s.tile * 16 + group_id + 8 * h);
            }
            const bf16* w_row = s.w + (size_t)row * s.ldw;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int kk = kc + 32 * c;
                const uint32_t dst = stage + ((h * 2 + c) * 32 + lane) * 16;
                if (kk < s.k1) cp_async16_mem(dst, w_row + kk);
                else sts128_zero(dst);
            }
        }
        if (++s.step == s.steps) {
            s.step = 0;
            s.tile += gridDim.x;
            if (s.tile >= s.tiles) stream_seek(s, step, s.phase + 1, warp);
        }
    }
    cp_async_commit_mem();
}

// All blocks meet: arrive, then poll the counter until every block of the grid has arrived `epoch` times.  Returns
// false (in every thread of the block) when the wait ran out; the kernel then ends.
__device__ __forceinline__ bool grid_barrier(const Step& step, unsigned int epoch, int phase) {
    __shared__ int barrier_ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(step.barrier, 1u);
        const unsigned int target = epoch * gridDim.x;
        unsigned int seen = 0;
        long polls = 0;
        do {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(step.barrier) : "memory");
        } while (seen < target && ++polls < kSpinLimit);
        barrier_ok = seen >= target;
        if (seen < target) atomicExch(step.status, 1 + (phase << 8));
        __threadfence();
    }
    __syncthreads();
    return barrier_ok != 0;
}

// ------------------------------------------------------------------------------------ staging of activations

// Rows of the float32 residual stream, multiplied by the norm's gain and rounded to bfloat16; their sums of squares
// go to sq_total.  (1/rms scales the accumulators at the end.)
__device__ __forceinline__ void stage_normed(const Step& step, const Phase& p, unsigned char* smem, float* sq_total, float* sq_warp) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int x_stride = p.k_pad * 2 + 64;
    const int chunks = p.k_len / 8;
    const float* src[kCols];
    float ss[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
        src[j] = step.x + (size_t)(j < step.batch ? j : 0) * step.hidden + p.k_begin;
        ss[j] = 0.0f;
    }
    for (int c = threadIdx.x; c < chunks; c += kStepThreads) {
        const float4 ga = *reinterpret_cast<const float4*>(p.gain + c * 8);
        const float4 gd = *reinterpret_cast<const float4*>(p.gain + c * 8 + 4);
        float4 a[kCols], d[kCols];
#pragma unroll
        for (int j = 0; j < kCols; ++j)
            if (j < step.batch) {
                a[j] = __ldcg(reinterpret_cast<const float4*>(src[j] + c * 8));
                d[j] = __ldcg(reinterpret_cast<const float4*>(src[j] + c * 8 + 4));
            }
#pragma unroll
        for (int j = 0; j < kCols; ++j)
            if (j < step.batch) {
                ss[j] += a[j].x * a[j].x + a[j].y * a[j].y + a[j].z * a[j].z + a[j].w * a[j].w + d[j].x * d[j].x +
                         d[j].y * d[j].y + d[j].z * d[j].z + d[j].w * d[j].w;
                *reinterpret_cast<uint4*>(smem + j * x_stride + c * 16) =
                    make_uint4(pack_bf16(a[j].x * ga.x, a[j].y * ga.y), pack_bf16(a[j].z * ga.z, a[j].w * ga.w),
                               pack_bf16(d[j].x * gd.x, d[j].y * gd.y), pack_bf16(d[j].z * gd.z, d[j].w * gd.w));
            }
    }
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
        const float total = warp_sum(ss[j]);
        if (lane == 0) sq_warp[warp * kCols + j] = total;
    }
    __syncthreads();
    if (threadIdx.x < kCols) {
        float s = 0.0f;
        for (int w = 0; w < kStepWarps; ++w) s += sq_warp[w * kCols + threadIdx.x];
        sq_total[threadIdx.x] = s;
    }
}

// Rows of a bfloat16 buffer (the gated activations), columns [k_begin, k_begin + k_len).
__device__ __forceinline__ void stage_bf16(const Step& step, const Phase& p, uint32_t smem_base, const bf16* from, int ld) {
    const int x_stride = p.k_pad * 2 + 64;
    const int chunks = p.k_len / 8;
    for (int b = 0; b < step.batch; ++b) {
        const bf16* src = from + (size_t)b * ld + p.k_begin;
        for (int c = threadIdx.x; c < chunks; c += kStepThreads) cp_async16_mem(smem_base + b * x_stride + c * 16, src + c * 8);
    }
}

// The attention's output rows, combined from the partial results of the split keys while they are staged: with
// (m_s, l_s, o_s) of split s, m = max m_s, out = sum o_s 2^(m_s - m) / sum l_s 2^(m_s - m).
__device__ __forceinline__ void stage_attention(const Step& step, const Phase& p, unsigned char* smem) {
    const int x_stride = p.k_pad * 2 + 64;
    const int splits = step.splits[p.group];
    const int quads = HD / 4;
    const int total = step.batch * p.heads * quads;
    for (int i = threadIdx.x; i < total; i += kStepThreads) {
        const int quad = i % quads, head = (i / quads) % p.heads, b = i / (quads * p.heads);
        const size_t slot = (size_t)(b * p.heads + head) * splits;
        float m = -CUDART_INF_F;
        for (int s = 0; s < splits; ++s) m = fmaxf(m, __ldcg(step.attn_ml + (slot + s) * 2));
        float sum = 0.0f;
        float4 value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s = 0; s < splits; ++s) {
            const float weight = fast_exp2(__ldcg(step.attn_ml + (slot + s) * 2) - m);  // 0 for a split that saw nothing
            if (weight > 0.0f) {
                sum += __ldcg(step.attn_ml + (slot + s) * 2 + 1) * weight;
                const float4 o = __ldcg(reinterpret_cast<const float4*>(step.attn_o + (slot + s) * HD + quad * 4));
                value.x += o.x * weight; value.y += o.y * weight; value.z += o.z * weight; value.w += o.w * weight;
            }
        }
        const float inv = 1.0f / sum;
        const int col = head * HD + quad * 4 - p.k_begin;  // (the output product is never split: k_begin is 0)
        *reinterpret_cast<uint2*>(smem + b * x_stride + col * 2) =
            make_uint2(pack_bf16(value.x * inv, value.y * inv), pack_bf16(value.z * inv, value.w * inv));
    }
}

// ------------------------------------------------------------------------------------ the attention phase

// 16 rows of [HD] from a pool -> a warp's own padded rows in shared memory.
__device__ __forceinline__ void load_rows16(uint32_t dst, const bf16* __restrict__ src, int lane) {
#pragma unroll
    for (int j = 0; j < 16 * kChunks / 32; ++j) {
        const int i = lane + j * 32;
        const int row = i / kChunks, chunk = i % kChunks;
        cp_async16(dst + row * kRowBytes + chunk * 16, src + row * HD + chunk * 8);
    }
}

// One (sequence, kv head, split) item: this block's warps take 16 keys of a page each (and, eight of them, two pages
// at a time), keep running maxima and sums, and write the item's partial result.  As decode_attention_kernel of
// csrc/attention_tc.cu (kvHead = head / group; dot first, then scale; positions <= the query's, of a window only its
// last n: backend-java/.../llama/LlamaForwardPass.java:1543-1670).
__device__ __forceinline__ void attention_item(const Step& step, const Phase& p, unsigned char* smem, int seq, int kv_head,
                                               int chunk, int split, int splits) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const int group = p.heads / p.kv_heads;
    const int head0 = kv_head * group + chunk * 16;
    const int rows_here = min(16, group - chunk * 16);
    const int kv_len = step.kv_lens[seq];
    const int pos = kv_len - 1;
    const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int first_tile = first / kTile;
    const int tiles = (kv_len + kTile - 1) / kTile - first_tile;
    const int per_split = (tiles + splits - 1) / splits;
    const int t_begin = first_tile + split * per_split;
    const int t_end = min(t_begin + per_split, first_tile + tiles);
    unsigned char* q_smem = smem;
    const uint32_t rings = smem_u32(smem) + kQRowsDecode * kRowBytes;
    constexpr int kPagesAtOnce = kAttnWarps / 4;  // pages the block's warps work on at the same time
    const int sub = warp & 3, lane_page = warp >> 2;
    const bool works = warp < kAttnWarps;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float run_max[2] = {-CUDART_INF_F, -CUDART_INF_F}, run_sum[2] = {0.0f, 0.0f};
    const float scale_log2 = p.scale * 1.4426950408889634f;

    // the query rows of this kv head's group
    for (int i = threadIdx.x; i < kQRowsDecode * kChunks; i += kStepThreads) {
        const int row = i / kChunks, c = i % kChunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows_here) v = __ldcg(reinterpret_cast<const uint4*>(step.q + (size_t)seq * step.ld_q + (size_t)(head0 + row) * HD + c * 8));
        *reinterpret_cast<uint4*>(q_smem + row * kRowBytes + c * 16) = v;
    }
    __syncthreads();
    if (works && t_begin < t_end) {
        const int* table = step.block_tables[p.group] + (size_t)seq * step.max_blocks;
        const uint32_t ring = rings + warp * kAttnStages * kAttnStageBytes;
        auto fetch = [&](int t, int stage) {
            const size_t page = table[t];
            const size_t at = ((page * p.kv_heads + kv_head) * kTile + sub * 16) * (size_t)HD;
            load_rows16(ring + stage * kAttnStageBytes, p.k_pool + at, lane);
            load_rows16(ring + stage * kAttnStageBytes + 16 * kRowBytes, p.v_pool + at, lane);
        };
        const int t0 = t_begin + lane_page;
#pragma unroll
        for (int ahead = 0; ahead < kAttnStages - 1; ++ahead) {
            if (t0 + ahead * kPagesAtOnce < t_end) fetch(t0 + ahead * kPagesAtOnce, ahead);
            cp_async_commit();
        }
        uint32_t a[kKSteps][4];
        load_q_fragments(a, smem_u32(q_smem));
        int round = 0;
        for (int t = t0; t < t_end; t += kPagesAtOnce, ++round) {
            const int next = t + (kAttnStages - 1) * kPagesAtOnce;
            if (next < t_end) fetch(next, (round + kAttnStages - 1) % kAttnStages);
            cp_async_commit();
            cp_async_wait<kAttnStages - 1>();
            __syncwarp();
            const uint32_t k_rows = ring + (round % kAttnStages) * kAttnStageBytes, v_rows = k_rows + 16 * kRowBytes;
            const int abs0 = t * kTile + sub * 16;
            if (abs0 <= pos && abs0 + 15 >= first) {  // this warp's 16 keys hold something visible
                float s[2][4];
                scores_16_keys(s, a, k_rows, 0);
                if (abs0 < first || abs0 + 15 > pos) {  // an end of the visible range runs through these 16 keys
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int key = abs0 + nt * 8 + tid4 * 2 + (i & 1);
                            if (key < first || key > pos) s[nt][i] = -CUDART_INF_F;
                        }
                }
                const float row_max[2] = {fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1])),
                                          fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]))};
                float probs[2][4];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const float tile_max = quad_max(row_max[r]);
                    const float new_max = fmaxf(run_max[r], tile_max);  // finite: a visible key exists
                    const float correction = fast_exp2((run_max[r] - new_max) * scale_log2);
                    const float offset = -new_max * scale_log2;
                    run_max[r] = new_max;
                    float local = 0.0f;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const float e = fast_exp2(fmaf(s[nt][2 * r + c], scale_log2, offset));
                            probs[nt][2 * r + c] = e;
                            local += e;
                        }
                    run_sum[r] = run_sum[r] * correction + local;
#pragma unroll
                    for (int i = 0; i < HD / 8; ++i) {
                        o[i][2 * r] *= correction;
                        o[i][2 * r + 1] *= correction;
                    }
                }
                const uint32_t pk[4] = {pack_bf16(probs[0][0], probs[0][1]), pack_bf16(probs[0][2], probs[0][3]),
                                        pack_bf16(probs[1][0], probs[1][1]), pack_bf16(probs[1][2], probs[1][3])};
                accumulate_16_keys(o, pk, v_rows, 0);
            }
            __syncwarp();
        }
        cp_async_wait<0>();
    }
    run_sum[0] = quad_sum(run_sum[0]);
    run_sum[1] = quad_sum(run_sum[1]);

    // the warps' partial results meet in shared memory (the page rings are free once every warp has left its loop)
    __syncthreads();
    float* merge_o = reinterpret_cast<float*>(smem + kQRowsDecode * kRowBytes);  // [warps][16][HD]
    float* merge_ml = merge_o + kAttnWarps * 16 * HD;                             // [warps][16][2]
    if (works) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = group_id + 8 * r;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                float* dst = merge_o + (size_t)(warp * 16 + row) * HD + i * 8 + tid4 * 2;
                dst[0] = o[i][2 * r];
                dst[1] = o[i][2 * r + 1];
            }
            if (tid4 == 0) {
                merge_ml[(warp * 16 + row) * 2] = run_max[r] * scale_log2;  // from here on maxima are exponents of two
                merge_ml[(warp * 16 + row) * 2 + 1] = run_sum[r];
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows_here * HD; i += kStepThreads) {
        const int row = i / HD, d = i % HD;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) m = fmaxf(m, merge_ml[(w * 16 + row) * 2]);
        float total = 0.0f, value = 0.0f;
        if (m != -CUDART_INF_F) {
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) {
                const float weight = fast_exp2(merge_ml[(w * 16 + row) * 2] - m);  // 0 for a warp that saw nothing
                total += merge_ml[(w * 16 + row) * 2 + 1] * weight;
                value += merge_o[(size_t)(w * 16 + row) * HD + d] * weight;
            }
        }
        const size_t slot = (size_t)(seq * p.heads + head0 + row) * splits + split;
        step.attn_o[slot * HD + d] = value;
        if (d == 0) {
            step.attn_ml[slot * 2] = m;
            step.attn_ml[slot * 2 + 1] = total;
        }
    }
    __syncthreads();  // the next item reuses the shared memory
}

// ------------------------------------------------------------------------------------ the kernel

__global__ void __launch_bounds__(kStepThreads, 1)
decode_step_kernel(const Step step) {
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const uint32_t ring = smem_base + kFrontBytes + warp * kDepth * kStageBytes;
    float* partial = reinterpret_cast<float*>(smem + kFrontBytes + kRingBytes);  // two buffers
    float* sq_total = partial + 2 * kPartialFloats;                              // [kCols]
    float* sq_warp = sq_total + kCols;                                           // [warps][kCols]

    // the weight stream starts at once: weights depend on nothing
    Stream stream;
    stream_seek(stream, step, 0, warp);
    int produce_slot = 0, consume_slot = 0;
    for (int s = 0; s < kDepth - 1; ++s) {
        stream_produce(stream, step, ring, produce_slot, warp, lane);
        produce_slot = (produce_slot + 1) % kDepth;
    }

    unsigned int epoch = 0;
    int tile_parity = 0;
    for (int ph = 0; ph < step.num_phases; ++ph) {
        const Phase& p = step.phases[ph];
        if (p.barrier_before && !grid_barrier(step, ++epoch, ph)) break;

        if (p.kind == PH_EMBED) {
            // x = E[token] * scale, a row per block (backend-java/.../llama/LlamaForwardPass.java:1024-1025)
            for (int b = blockIdx.x; b < step.batch; b += gridDim.x) {
                const bf16* row = step.embedding + (size_t)step.tokens[b] * step.hidden;
                for (int i = threadIdx.x; i < step.hidden; i += kStepThreads)
                    step.x[(size_t)b * step.hidden + i] = __bfloat162float(row[i]) * step.embedding_scale;
            }
            continue;
        }
        if (p.kind == PH_ATTN) {
            const int splits = step.splits[p.group];
            const int group = p.heads / p.kv_heads;
            const int head_chunks = (group + 15) / 16;
            const int per_sequence = p.kv_heads * head_chunks * splits;
            for (int item = blockIdx.x; item < step.batch * per_sequence; item += gridDim.x) {
                const int split = item % splits, kvc = (item / splits) % (p.kv_heads * head_chunks), seq = item / per_sequence;
                attention_item(step, p, smem, seq, kvc / head_chunks, kvc % head_chunks, split, splits);
            }
            continue;
        }

        // ---- a matrix phase: activations of its columns -> shared memory, bfloat16
        const int x_stride = p.k_pad * 2 + 64;
        const int chunks_padded = p.k_pad / 8, chunks = p.k_len / 8;
        __syncthreads();  // whoever still reads the front of shared memory (the phase before) is done
        for (int b = 0; b < kCols; ++b) {
            const int live = b < step.batch ? chunks : 0;
            for (int c = live + threadIdx.x; c < chunks_padded; c += kStepThreads) sts128_zero(smem_base + b * x_stride + c * 16);
        }
        if (p.gain) stage_normed(step, p, smem, sq_total, sq_warp);
        else if (p.kind == PH_OUT) stage_attention(step, p, smem);
        else stage_bf16(step, p, smem_base, step.h, step.ld_h);
        if (!p.gain && p.kind != PH_OUT) {
            // the copies of this staging are the newest groups: wait for all (the ring's older groups have long landed)
            cp_async_commit_mem();
            cp_async_wait_mem<0>();
        }
        __syncthreads();

        // ---- this block's row tiles; the ring keeps running across them
        const bool paired = p.kind == PH_GATE_UP || p.kind == PH_QKV;
        const int tile_rows = paired ? 8 : 16;
        int k0, k1;
        const int steps = slice_steps(p, warp, &k0, &k1);
        const uint32_t x_lane = smem_base + group_id * x_stride + (k0 + 8 * tid4) * 2;
        for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x) {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int s = 0; s < steps; ++s) {
                stream_produce(stream, step, ring, produce_slot, warp, lane);
                produce_slot = (produce_slot + 1) % kDepth;
                cp_async_wait_mem<kDepth - 1>();  // this lane's pieces of the stage have landed; nobody else reads them
                const uint32_t stage = ring + consume_slot * kStageBytes;
                consume_slot = (consume_slot + 1) % kDepth;
                uint4 wv[2][2];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 2; ++c) wv[h][c] = lds128(stage + ((h * 2 + c) * 32 + lane) * 16);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint4 xv = lds128(x_lane + (s * kStageCols + 32 * c) * 2);
                    mma_16816(acc, wv[0][c].x, wv[1][c].x, wv[0][c].y, wv[1][c].y, xv.x, xv.y);
                    mma_16816(acc, wv[0][c].z, wv[1][c].z, wv[0][c].w, wv[1][c].w, xv.z, xv.w);
                }
            }
            // the warps' partial sums: c0, c1 = (MMA row group_id, activation rows 2 * tid4, + 1); c2, c3 = row + 8
            float* mine = partial + tile_parity * kPartialFloats;
            tile_parity ^= 1;
#pragma unroll
            for (int i = 0; i < 4; ++i) mine[(warp * 16 + group_id + 8 * (i >> 1)) * kCols + tid4 * 2 + (i & 1)] = acc[i];
            __syncthreads();
            if (threadIdx.x < tile_rows * kCols) {
                const int row_in_tile = threadIdx.x % tile_rows, col = threadIdx.x / tile_rows;
                const int row = tile * tile_rows + row_in_tile;
                const int rows_total = p.kind == PH_QKV ? p.rows / 2 : p.rows;  // rows, or pairs
                if (row < rows_total && col < step.batch) {
                    float value = 0.0f, second = 0.0f;  // second: the partner row of a pair
#pragma unroll
                    for (int w = 0; w < kStepWarps; ++w) {
                        value += mine[(w * 16 + row_in_tile) * kCols + col];
                        if (paired) second += mine[(w * 16 + row_in_tile + 8) * kCols + col];
                    }
                    if (p.gain) {
                        const float inv_rms = 1.0f / sqrtf(sq_total[col] / (float)p.k_len + p.eps);
                        value *= inv_rms;
                        second *= inv_rms;
                    }
                    if (p.kind == PH_HEAD) {
                        step.logits[(size_t)col * step.ld_logits + row] = value;
                    } else if (p.kind == PH_OUT || p.kind == PH_DOWN) {
                        step.x[(size_t)col * step.hidden + row] += value;  // this block alone owns the row in this phase
                    } else if (p.kind == PH_GATE_UP) {
                        step.h[(size_t)col * step.ld_h + row] = __float2bfloat16_rn(gate_activation(p.activation, value) * second);
                    } else {  // PH_QKV
                        constexpr int tiles_per_head = HD / 16, half = HD / 2;
                        const int head = tile / tiles_per_head, d0 = (tile % tiles_per_head) * 8 + row_in_tile;
                        // queries and keys pass through bfloat16 before the rotation, as they do when a product stores them
                        float x0 = __bfloat162float(__float2bfloat16_rn(value)), x1 = __bfloat162float(__float2bfloat16_rn(second));
                        if (head < p.heads + p.kv_heads) {
                            const size_t at_table = (size_t)step.positions[col] * half + d0;
                            const float c = p.cos_table[at_table], sn = p.sin_table[at_table];
                            const float r0 = x0 * c - x1 * sn, r1 = x0 * sn + x1 * c;
                            x0 = r0;
                            x1 = r1;
                        }
                        if (head < p.heads) {
                            bf16* q = step.q + (size_t)col * step.ld_q + (size_t)head * HD;
                            q[d0] = __float2bfloat16_rn(x0);
                            q[d0 + half] = __float2bfloat16_rn(x1);
                        } else {
                            const int slot = step.slot_mappings[p.group][col];
                            if (slot >= 0) {
                                const bool is_key = head < p.heads + p.kv_heads;
                                const int kv_head = head - p.heads - (is_key ? 0 : p.kv_heads);
                                const size_t page = slot / kTile, offset = slot % kTile;
                                bf16* dst = (is_key ? p.k_pool : p.v_pool) + ((page * p.kv_heads + kv_head) * kTile + offset) * HD;
                                dst[d0] = __float2bfloat16_rn(x0);
                                dst[d0 + half] = __float2bfloat16_rn(x1);
                            }
                        }
                    }
                }
            }
        }
    }
    cp_async_wait_mem<0>();  // nothing of this block is in flight when it leaves
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_decode_step_head_dim() { return HD; }
MB_EXPORT size_t mb_decode_step_phase_bytes() { return sizeof(Phase); }
MB_EXPORT size_t mb_decode_step_step_bytes() { return sizeof(Step); }
MB_EXPORT int mb_decode_step_max_columns() { return kMaxStageCols; }
MB_EXPORT int mb_decode_step_slice_columns() { return kSliceCols; }
MB_EXPORT int mb_decode_step_max_groups() { return kMaxGroups; }

// Runs one decode step.  `step` (host memory) is copied; its `phases` point to device memory.  The barrier counter is
// set to zero on the stream first.  Blocks: one per multiprocessor, launched cooperatively (all resident, or the
// launch fails).
MB_EXPORT int mb_decode_step(const Step* given, int multiprocessors, cudaStream_t stream) {
    const Step step = *given;
    if (step.batch < 1 || step.batch > kCols) return fail("decode_step: takes 1 to %d sequences, got %d", kCols, step.batch);
    if (step.num_phases < 1 || !step.phases) return fail("decode_step: no phases");
    if (step.hidden % 8 || ((uintptr_t)step.x & 15) || ((uintptr_t)step.q & 15) || ((uintptr_t)step.h & 15) || step.ld_q % 8 || step.ld_h % 8)
        return fail("decode_step: rows of the residual stream, queries and gated activations must start on 16-byte boundaries");
    if (!step.barrier || !step.status) return fail("decode_step: needs a barrier counter and a status word");
    static bool configured[64] = {false};
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return fail("decode_step: cannot tell the current device");
    if (!configured[device]) {
        cudaError_t status = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (status != cudaSuccess) return fail("decode_step: cannot reserve %d bytes of shared memory: %s", kSmemBytes, cudaGetErrorString(status));
        int resident = 0;
        status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, decode_step_kernel, kStepThreads, kSmemBytes);
        if (status != cudaSuccess || resident < 1) return fail("decode_step: a block does not fit a multiprocessor");
        configured[device] = true;
    }
    cudaError_t status = cudaMemsetAsync(step.barrier, 0, sizeof(unsigned int), stream);
    if (status != cudaSuccess) return fail("decode_step: cannot clear the barrier counter: %s", cudaGetErrorString(status));
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(multiprocessors);
    config.blockDim = dim3(kStepThreads);
    config.dynamicSmemBytes = kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    status = cudaLaunchKernelEx(&config, decode_step_kernel, step);
    if (status != cudaSuccess) return fail("decode_step: launch failed: %s", cudaGetErrorString(status));
    return check_launch("decode_step");
}
