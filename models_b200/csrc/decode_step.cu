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

#include <string.h>

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kStepWarps = 8;
constexpr int kStepThreads = kStepWarps * 32;
constexpr int kCols = 8;              // activation rows of a step = columns of the MMA
constexpr int kTeams = 2;             // a block's warps work as two teams, each on a row tile of its own
constexpr int kTeamWarps = kStepWarps / kTeams;  // the warps of a team split K
constexpr int kTeamThreads = kTeamWarps * 32;
constexpr int kStageCols = 128;       // columns of K per ring stage
constexpr int kPieces = kStageCols / 32;  // 32 columns per piece, a lane takes 8 of each piece
constexpr int kStageBytes = 2 * kPieces * 32 * 16;  // [2 row halves][pieces][32 lanes][16 bytes]
constexpr int kDepth = 4;             // ring stages per warp
constexpr int kSliceCols = kTeamWarps * kStageCols;  // K is padded to a multiple of this
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

constexpr int kMaxPhases = 250;  // what fits a launch's 32 KB of parameters beside the step's own record

// What changes from step to step.
struct Step {
    const Phase* phases;  // host memory, copied into the launch's parameters
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
    int* attn_tickets;    // [batch][kv heads x head chunks] arrivals of a sequence's splits; zero before and after a step
    bf16* a;              // [batch][ld_q] the attention's output rows
    float* logits;        // [batch][ld_logits]
    int ld_logits;
    unsigned int* barrier;  // arrival counter: zero at launch, and zero again when the step is done
    int* status;            // set to 1 + (phase << 8) by a block whose bounded wait ran out
    long long* timeline;    // null, or [num_phases][6] clock readings of block 0: phase entered, barrier passed, activations staged, done, first tile's products done, its sums met
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
//   partial      [2 teams][2 buffers][4 warps][16 rows][8 columns] floats
//   sums         [8] sums of squares of the rows, then [8 warps][8] the warps' parts of them
constexpr int kAttnBytes = kQRowsDecode * kRowBytes + kAttnWarps * kAttnStages * kAttnStageBytes;
constexpr int kMergeBytes = kQRowsDecode * kRowBytes + kAttnWarps * 16 * (HD + 2) * (int)sizeof(float);
constexpr int kActivationBytes = kCols * (kMaxStageCols * 2 + 64);
constexpr int max3(int a, int b, int c) { return a > b ? (a > c ? a : c) : (b > c ? b : c); }
constexpr int kFrontBytes = (max3(kAttnBytes, kMergeBytes, kActivationBytes) + 127) / 128 * 128;
constexpr int kRingBytes = kStepWarps * kDepth * kStageBytes;
constexpr int kPartialFloats = kTeamWarps * 16 * kCols;  // one buffer of one team
constexpr int kSmemBytes = kFrontBytes + kRingBytes + (kTeams * 2 * kPartialFloats + kCols + kStepWarps * kCols) * (int)sizeof(float);

// A launch's parameters: the step and the phases, by value.  They reach the kernel through the constant bank, so
// walking the phases costs no trip to memory (a phase's record read from global memory at every phase boundary cost
// about a microsecond of latency per phase, in the consumer and again in the producer of the weight stream).
struct StepParams {
    Step step;
    Phase phases[kMaxPhases];
};

// Where a warp's weight stream stands: the phases, the block's tiles of a phase and the warp's steps over its slice
// of K, flattened into one sequence of stages.  The producer runs kDepth - 1 stages ahead of the consumer.
struct Stream {
    int phase;        // index of the phase the next stage belongs to; num_phases when the stream has ended
    int tile;         // row tile of that stage
    int step;         // 128-column step within the warp's slice
    int steps;        // steps of the slice in this phase
    int kind, rows, tiles, pair_offset, ldw;
    int k0, k1;       // the warp's columns [k0, k1) of the (sub-)phase
    const bf16* w;
    const bf16* row[2];  // of the current tile: this lane's two weight rows (MMA rows group_id and group_id + 8)
};

// The first row tile of a team in a phase, and the distance to its next: the teams of all blocks take the tiles in turn.
__device__ __forceinline__ int first_tile(int team) { return team * gridDim.x + blockIdx.x; }
__device__ __forceinline__ int tile_stride() { return kTeams * gridDim.x; }

// This lane's two weight rows of a tile: 16 consecutive rows, or 8 rows and their partners.
__device__ __forceinline__ void stream_rows(Stream& s, int lane) {
    const int group_id = lane >> 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int row;
        if (s.kind == PH_GATE_UP) {
            row = min(s.rows - 1, s.tile * 8 + group_id) + h * s.pair_offset;
        } else if (s.kind == PH_QKV) {  // tile = (head, eighth of its first half); the partner lies half a head further
            constexpr int tiles_per_head = HD / 16;
            row = (s.tile / tiles_per_head) * HD + (s.tile % tiles_per_head) * 8 + group_id + h * (HD / 2);
        } else {
            row = min(s.rows - 1, s.tile * 16 + group_id + 8 * h);
        }
        s.row[h] = s.w + (size_t)row * s.ldw;
    }
}

__device__ __forceinline__ int slice_steps(const Phase& p, int warp, int* k0, int* k1) {
    const int per_warp = p.k_pad / kTeamWarps;
    *k0 = min(p.k_len, (warp % kTeamWarps) * per_warp);
    *k1 = min(p.k_len, *k0 + per_warp);
    return (*k1 - *k0 + kStageCols - 1) / kStageCols;
}

// Moves the stream to the first stage at or after phase `from` (a matrix phase in which this block has a tile and
// this warp a slice of K).
__device__ __forceinline__ void stream_seek(Stream& s, const Step& step, const Phase* phases, int from, int warp) {
    for (int ph = from; ph < step.num_phases; ++ph) {
        const Phase& p = phases[ph];
        if (p.kind == PH_EMBED || p.kind == PH_ATTN || first_tile(warp / kTeamWarps) >= p.tiles) continue;
        int k0, k1;
        const int steps = slice_steps(p, warp, &k0, &k1);
        if (steps == 0) continue;
        s.phase = ph; s.tile = first_tile(warp / kTeamWarps); s.step = 0; s.steps = steps;
        s.kind = p.kind; s.rows = p.rows; s.tiles = p.tiles; s.pair_offset = p.pair_offset; s.ldw = p.ldw;
        s.k0 = k0; s.k1 = k1; s.w = p.w;
        stream_rows(s, threadIdx.x & 31);
        return;
    }
    s.phase = step.num_phases;
}

// Issues the loads of the stream's next stage into ring slot `slot` and moves the stream on.  Always one commit
// group, also when the stream has ended: the consumer's waits count groups.
__device__ __forceinline__ void stream_produce(Stream& s, const Step& step, const Phase* phases, uint32_t ring, int slot, int warp, int lane) {
    if (s.phase < step.num_phases) {
        const int tid4 = lane & 3;
        const uint32_t stage = ring + slot * kStageBytes;
        const int kc = s.k0 + s.step * kStageCols + 8 * tid4;
        const uint32_t dst0 = stage + lane * 16;
        if (s.k0 + (s.step + 1) * kStageCols <= s.k1) {  // the whole stage lies inside the slice (all but the last stage at most)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < kPieces; ++c) cp_async16_mem(dst0 + (h * kPieces + c) * 512, s.row[h] + kc + 32 * c);
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int c = 0; c < kPieces; ++c) {
                    const int kk = kc + 32 * c;
                    if (kk < s.k1) cp_async16_mem(dst0 + (h * kPieces + c) * 512, s.row[h] + kk);
                    else sts128_zero(dst0 + (h * kPieces + c) * 512);
                }
            }
        }
        if (++s.step == s.steps) {
            s.step = 0;
            s.tile += tile_stride();
            if (s.tile >= s.tiles) stream_seek(s, step, phases, s.phase + 1, warp);
            else stream_rows(s, lane);
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
        for (;;) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(step.barrier) : "memory");
            if (seen >= target || ++polls >= kSpinLimit) break;
            __nanosleep(32);  // 148 pollers of one word: leave the arrivals some room
        }
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

// Rows of a bfloat16 buffer (the gated activations or the attention's output), columns [k_begin, k_begin + k_len).
// Plain loads, not cp.async: waiting for these copies must not wait for the weight ring's newest stages too.
__device__ __forceinline__ void stage_bf16(const Step& step, const Phase& p, unsigned char* smem, const bf16* from, int ld) {
    const int x_stride = p.k_pad * 2 + 64;
    const int chunks = p.k_len / 8;
    const int total = step.batch * chunks;
#pragma unroll 8
    for (int i = threadIdx.x; i < total; i += kStepThreads) {
        const int b = i / chunks, c = i % chunks;
        *reinterpret_cast<uint4*>(smem + b * x_stride + c * 16) =
            __ldcg(reinterpret_cast<const uint4*>(from + (size_t)b * ld + p.k_begin + c * 8));
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

    // the first pages are asked for before anything else; then the query rows of this kv head's group
    const int* table = step.block_tables[p.group] + (size_t)seq * step.max_blocks;
    const uint32_t ring = rings + warp * kAttnStages * kAttnStageBytes;
    auto fetch = [&](int t, int stage) {
        const size_t page = table[t];
        const size_t at = ((page * p.kv_heads + kv_head) * kTile + sub * 16) * (size_t)HD;
        load_rows16(ring + stage * kAttnStageBytes, p.k_pool + at, lane);
        load_rows16(ring + stage * kAttnStageBytes + 16 * kRowBytes, p.v_pool + at, lane);
    };
    const int t0 = t_begin + lane_page;
    if (works && t_begin < t_end) {
#pragma unroll
        for (int ahead = 0; ahead < kAttnStages - 1; ++ahead) {
            if (t0 + ahead * kPagesAtOnce < t_end) fetch(t0 + ahead * kPagesAtOnce, ahead);
            cp_async_commit();
        }
    }
    for (int i = threadIdx.x; i < kQRowsDecode * kChunks; i += kStepThreads) {
        const int row = i / kChunks, c = i % kChunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows_here) v = __ldcg(reinterpret_cast<const uint4*>(step.q + (size_t)seq * step.ld_q + (size_t)(head0 + row) * HD + c * 8));
        *reinterpret_cast<uint4*>(q_smem + row * kRowBytes + c * 16) = v;
    }
    __syncthreads();
    if (works && t_begin < t_end) {
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
        if (splits == 1) {
            step.a[(size_t)seq * step.ld_q + (size_t)(head0 + row) * HD + d] = __float2bfloat16_rn(value * (1.0f / total));
        } else {
            const size_t slot = (size_t)(seq * p.heads + head0 + row) * splits + split;
            step.attn_o[slot * HD + d] = value;
            if (d == 0) {
                step.attn_ml[slot * 2] = m;
                step.attn_ml[slot * 2 + 1] = total;
            }
        }
    }
    if (splits > 1) {
        // whichever split's block stores last combines them all, in the order of the splits (the same additions whoever
        // that is): with (m_s, l_s, o_s) of split s, m = max m_s, out = sum o_s 2^(m_s - m) / sum l_s 2^(m_s - m)
        __shared__ int last_split;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            int* ticket = step.attn_tickets + seq * (p.kv_heads * ((group + 15) / 16)) + kv_head * ((group + 15) / 16) + chunk;
            last_split = atomicAdd(ticket, 1) == splits - 1;
            if (last_split) *ticket = 0;  // as the next step expects it
            __threadfence();
        }
        __syncthreads();
        if (last_split) {
            for (int i = threadIdx.x; i < rows_here * (HD / 4); i += kStepThreads) {
                const int row = i / (HD / 4), quad = i % (HD / 4);
                const size_t slot = (size_t)(seq * p.heads + head0 + row) * splits;
                float m = -CUDART_INF_F;
                for (int sp = 0; sp < splits; ++sp) m = fmaxf(m, __ldcg(step.attn_ml + (slot + sp) * 2));
                float sum = 0.0f;
                float4 value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int sp = 0; sp < splits; ++sp) {
                    const float weight = fast_exp2(__ldcg(step.attn_ml + (slot + sp) * 2) - m);  // 0 for a split that saw nothing
                    if (weight > 0.0f) {
                        sum += __ldcg(step.attn_ml + (slot + sp) * 2 + 1) * weight;
                        const float4 o4 = __ldcg(reinterpret_cast<const float4*>(step.attn_o + (slot + sp) * HD + quad * 4));
                        value.x += o4.x * weight; value.y += o4.y * weight; value.z += o4.z * weight; value.w += o4.w * weight;
                    }
                }
                const float inv = 1.0f / sum;
                *reinterpret_cast<uint2*>(step.a + (size_t)seq * step.ld_q + (size_t)(head0 + row) * HD + quad * 4) =
                    make_uint2(pack_bf16(value.x * inv, value.y * inv), pack_bf16(value.z * inv, value.w * inv));
            }
        }
    }
    __syncthreads();  // the next item reuses the shared memory
}

// ------------------------------------------------------------------------------------ the kernel

__global__ void __launch_bounds__(kStepThreads, 1)
decode_step_kernel(const __grid_constant__ StepParams params) {
    const Step& step = params.step;
    const Phase* phases = params.phases;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const uint32_t ring = smem_base + kFrontBytes + warp * kDepth * kStageBytes;
    const int team = warp / kTeamWarps, team_warp = warp % kTeamWarps, team_thread = threadIdx.x % kTeamThreads;
    float* partial = reinterpret_cast<float*>(smem + kFrontBytes + kRingBytes) + team * 2 * kPartialFloats;  // this team's two buffers
    float* sq_total = reinterpret_cast<float*>(smem + kFrontBytes + kRingBytes) + kTeams * 2 * kPartialFloats;  // [kCols]
    float* sq_warp = sq_total + kCols;                                           // [warps][kCols]

    // the weight stream starts at once: weights depend on nothing
    Stream stream;
    stream_seek(stream, step, phases, 0, warp);
    int produce_slot = 0, consume_slot = 0;
    for (int s = 0; s < kDepth - 1; ++s) {
        stream_produce(stream, step, phases, ring, produce_slot, warp, lane);
        produce_slot = (produce_slot + 1) % kDepth;
    }

    unsigned int epoch = 0;
    int tile_parity = 0;
    const bool timed = step.timeline != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
    for (int ph = 0; ph < step.num_phases; ++ph) {
        const Phase& p = phases[ph];
        if (timed) {
            if (ph > 0) step.timeline[(ph - 1) * 6 + 3] = clock64();
            step.timeline[ph * 6] = clock64();
        }
        if (p.barrier_before && !grid_barrier(step, ++epoch, ph)) break;
        if (timed) step.timeline[ph * 6 + 1] = step.timeline[ph * 6 + 2] = clock64();

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

        // ---- a matrix phase.  First what the finishing threads need from memory besides the sums (a position's
        // rotation, a cache slot): asked for now, there when the first tile is done
        const bool paired = p.kind == PH_GATE_UP || p.kind == PH_QKV;
        const int tile_rows = paired ? 8 : 16;
        const bool finisher = team_thread < tile_rows * kCols;
        const int row_in_tile = team_thread % tile_rows, col = team_thread / tile_rows;
        const bool live_col = finisher && col < step.batch;
        int position = 0, cache_slot = -1;
        if (live_col && p.kind == PH_QKV) {
            position = step.positions[col];
            cache_slot = step.slot_mappings[p.group][col];
        }
        // ---- activations of its columns -> shared memory, bfloat16
        const int x_stride = p.k_pad * 2 + 64;
        const int chunks_padded = p.k_pad / 8, chunks = p.k_len / 8;
        __syncthreads();  // whoever still reads the front of shared memory (the phase before) is done
        for (int b = 0; b < kCols; ++b) {
            const int live = b < step.batch ? chunks : 0;
            for (int c = live + threadIdx.x; c < chunks_padded; c += kStepThreads) sts128_zero(smem_base + b * x_stride + c * 16);
        }
        if (p.gain) stage_normed(step, p, smem, sq_total, sq_warp);
        else if (p.kind == PH_OUT) stage_bf16(step, p, smem, step.a, step.ld_q);
        else stage_bf16(step, p, smem, step.h, step.ld_h);
        __syncthreads();
        if (timed) step.timeline[ph * 6 + 2] = clock64();

        // ---- the row tiles of this warp's team; the ring keeps running across them
        const int rows_total = p.kind == PH_QKV ? p.rows / 2 : p.rows;  // rows, or pairs
        int k0, k1;
        const int steps = slice_steps(p, warp, &k0, &k1);
        const uint32_t x_lane = smem_base + group_id * x_stride + (k0 + 8 * tid4) * 2;
        // the thread of the team that finishes output (row_in_tile, col) of every tile
        float inv_rms = 1.0f;
        if (live_col && p.gain) inv_rms = 1.0f / sqrtf(sq_total[col] / (float)p.k_len + p.eps);
        for (int tile = first_tile(team); tile < p.tiles; tile += tile_stride()) {
            const int row = tile * tile_rows + row_in_tile;
            const bool live = live_col && row < rows_total;
            float before = 0.0f, rope_cos = 1.0f, rope_sin = 0.0f;
            float* x_at = nullptr;
            constexpr int tiles_per_head = HD / 16, half_head = HD / 2;
            const int head = tile / tiles_per_head, d0 = (tile % tiles_per_head) * 8 + row_in_tile;  // of a q/k/v tile
            if (live) {
                if (p.kind == PH_OUT || p.kind == PH_DOWN) {
                    x_at = step.x + (size_t)col * step.hidden + row;  // this thread alone owns the element in this phase
                    before = __ldcg(x_at);
                } else if (p.kind == PH_QKV && head < p.heads + p.kv_heads) {
                    rope_cos = p.cos_table[(size_t)position * half_head + d0];
                    rope_sin = p.sin_table[(size_t)position * half_head + d0];
                }
            }
            float acc[2 * kPieces][4];  // independent chains of products, added at the end
#pragma unroll
            for (int i = 0; i < 2 * kPieces; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
            for (int s = 0; s < steps; ++s) {
                stream_produce(stream, step, phases, ring, produce_slot, warp, lane);
                produce_slot = produce_slot + 1 == kDepth ? 0 : produce_slot + 1;
                cp_async_wait_mem<kDepth - 1>();  // this lane's pieces of the stage have landed; nobody else reads them
                const uint32_t stage = ring + consume_slot * kStageBytes;
                consume_slot = consume_slot + 1 == kDepth ? 0 : consume_slot + 1;
                uint4 wv[2][kPieces];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < kPieces; ++c) wv[h][c] = lds128(stage + ((h * kPieces + c) * 32 + lane) * 16);
#pragma unroll
                for (int c = 0; c < kPieces; ++c) {
                    const uint4 xv = lds128(x_lane + (s * kStageCols + 32 * c) * 2);
                    mma_16816(acc[2 * c], wv[0][c].x, wv[1][c].x, wv[0][c].y, wv[1][c].y, xv.x, xv.y);
                    mma_16816(acc[2 * c + 1], wv[0][c].z, wv[1][c].z, wv[0][c].w, wv[1][c].w, xv.z, xv.w);
                }
            }
            // the warps' partial sums: c0, c1 = (MMA row group_id, activation rows 2 * tid4, + 1); c2, c3 = row + 8
            if (timed && tile == (int)blockIdx.x) step.timeline[ph * 6 + 4] = clock64();
            float* mine = partial + tile_parity * kPartialFloats;
            tile_parity ^= 1;
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                float sum = 0.0f;
#pragma unroll
                for (int chain = 0; chain < 2 * kPieces; ++chain) sum += acc[chain][i];
                mine[(team_warp * 16 + group_id + 8 * (i >> 1)) * kCols + tid4 * 2 + (i & 1)] = sum;
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(kTeamThreads) : "memory");  // the team's warps meet; the other team runs on
            if (live) {
                float value = 0.0f, second = 0.0f;  // second: the partner row of a pair
#pragma unroll
                for (int w = 0; w < kTeamWarps; ++w) {
                    value += mine[(w * 16 + row_in_tile) * kCols + col];
                    if (paired) second += mine[(w * 16 + row_in_tile + 8) * kCols + col];
                }
                value *= inv_rms;
                second *= inv_rms;
                if (p.kind == PH_HEAD) {
                    step.logits[(size_t)col * step.ld_logits + row] = value;
                } else if (p.kind == PH_OUT || p.kind == PH_DOWN) {
                    __stcg(x_at, before + value);
                } else if (p.kind == PH_GATE_UP) {
                    step.h[(size_t)col * step.ld_h + row] = __float2bfloat16_rn(gate_activation(p.activation, value) * second);
                } else {  // PH_QKV
                    // queries and keys pass through bfloat16 before the rotation, as they do when a product stores them
                    float x0 = __bfloat162float(__float2bfloat16_rn(value)), x1 = __bfloat162float(__float2bfloat16_rn(second));
                    if (head < p.heads + p.kv_heads) {
                        const float r0 = x0 * rope_cos - x1 * rope_sin, r1 = x0 * rope_sin + x1 * rope_cos;
                        x0 = r0;
                        x1 = r1;
                    }
                    if (head < p.heads) {
                        bf16* q = step.q + (size_t)col * step.ld_q + (size_t)head * HD;
                        q[d0] = __float2bfloat16_rn(x0);
                        q[d0 + half_head] = __float2bfloat16_rn(x1);
                    } else if (cache_slot >= 0) {
                        const bool is_key = head < p.heads + p.kv_heads;
                        const int kv_head = head - p.heads - (is_key ? 0 : p.kv_heads);
                        const size_t page = cache_slot / kTile, offset = cache_slot % kTile;
                        bf16* dst = (is_key ? p.k_pool : p.v_pool) + ((page * p.kv_heads + kv_head) * kTile + offset) * HD;
                        dst[d0] = __float2bfloat16_rn(x0);
                        dst[d0 + half_head] = __float2bfloat16_rn(x1);
                    }
                }
            }
            if (timed && tile == (int)blockIdx.x) step.timeline[ph * 6 + 5] = clock64();
        }
    }
    if (timed) step.timeline[(step.num_phases - 1) * 6 + 3] = clock64();
    cp_async_wait_mem<0>();  // nothing of this block is in flight when it leaves
    // one more arrival, without a wait: whoever arrives last puts the counter back to zero for the next step (when a
    // wait ran out the count is short and stays: the status word says so, and the host clears both)
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(step.barrier, 1u) == (epoch + 1) * gridDim.x - 1) *step.barrier = 0u;
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_decode_step_head_dim() { return HD; }
MB_EXPORT size_t mb_decode_step_phase_bytes() { return sizeof(Phase); }
MB_EXPORT size_t mb_decode_step_step_bytes() { return sizeof(Step); }
MB_EXPORT int mb_decode_step_max_columns() { return kMaxStageCols; }
MB_EXPORT int mb_decode_step_slice_columns() { return kSliceCols; }
MB_EXPORT int mb_decode_step_max_groups() { return kMaxGroups; }

MB_EXPORT int mb_decode_step_max_phases() { return kMaxPhases; }

// Runs one decode step.  `step` and its `phases` (both host memory) are copied into the launch's parameters.  The
// barrier counter must be zero; a step leaves it zero (unless a bounded wait ran out: then the status word is set).
// Blocks: one per multiprocessor, launched cooperatively (all resident, or the launch fails).
MB_EXPORT int mb_decode_step(const Step* given, int multiprocessors, cudaStream_t stream) {
    static thread_local StepParams params;  // (32 KB: not on the stack)
    params.step = *given;
    const Step& step = params.step;
    if (step.num_phases < 1 || step.num_phases > kMaxPhases || !step.phases)
        return fail("decode_step: takes 1 to %d phases, got %d", kMaxPhases, step.num_phases);
    memcpy(params.phases, step.phases, sizeof(Phase) * step.num_phases);
    if (step.batch < 1 || step.batch > kCols) return fail("decode_step: takes 1 to %d sequences, got %d", kCols, step.batch);
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
    cudaError_t status = cudaSuccess;
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
    status = cudaLaunchKernelEx(&config, decode_step_kernel, params);
    if (status != cudaSuccess) return fail("decode_step: launch failed: %s", cudaGetErrorString(status));
    return check_launch("decode_step");
}
