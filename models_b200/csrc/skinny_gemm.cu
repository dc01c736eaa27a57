// Matrix products for decode: few activation rows (one per live sequence, up to 32) against a large
// bfloat16 weight matrix W[N, K] that is read exactly once.  The work is bound by the weight stream,
// so everything around the product is folded into the same kernel:
//   prologue  NORM: the activations are the float32 residual rows; RMSNorm (gain, epsilon) is applied
//             on the fly -- the rows are multiplied by the gain while they are staged, their sums of
//             squares are gathered by the same loads, and 1/rms scales the accumulators at the end
//             (sumSq/size + eps, sqrt, 1/rms: integrallis/models, backend-java/.../ops/TensorOps.java:45-58).
//   epilogue  BF16 / F32: store.  RESIDUAL: add into the float32 residual stream
//             (x = x + W.h, backend-java/.../llama/LlamaForwardPass.java:1131-1138,1172-1178).
//             SWIGLU: the 16 rows of a tile are 8 gate rows and the 8 up rows that match them, and
//             act(gate) * up is stored (silu: backend-java/.../ops/TensorOps.java:1407-1425; the
//             activation is an argument).
//             ROPE: W is [q heads; k heads; v heads]; the 16 rows of a tile are 8 coordinates of a head
//             and their rotation partners half a head further; query and key pairs are rotated by the
//             token's position (x0' = x0*c - x1*s, x1' = x0*s + x1*c, backend-java/.../ops/TensorOps.java:1481-1486),
//             queries go to the query buffer, keys and values straight into the paged cache
//             (backend-java/.../llama/LlamaForwardPass.java:1070-1086).
//
// Layout of the work.  A block of four warps owns 16 weight rows at a time and walks a sequence of
// such row tiles; its warps split the
// block's part of K.  Each warp streams its rows with cp.async through a private four-stage ring in
// shared memory, 128 columns per stage, and the stages run on across row tiles, so loads stay in flight
// from the first tile to the last.  The activations of the block's part of K are staged once, as
// bfloat16, in shared memory.  At the end of a row tile the warps' partial sums are added in warp
// order.  When the activations of all of K do not fit a block's shared memory (many rows, or a long
// K), K is also split over the blocks of a thread-block cluster (up to 8); their partial sums meet in
// the shared memory of the cluster's first block (distributed shared memory) and are added there in
// block order, so no result depends on timing.
//
// The kernel is launched as a programmatic dependent of the kernel before it: its blocks may start
// while that kernel drains, and they fill their weight rings (weights are never written) before they
// wait for it (griddepcontrol.wait) and touch the activations.
//
// In an m16n8k16 MMA the weights are the 16-row operand and 8 activation rows the 8-column one.  The
// order of k inside an MMA is free as long as both operands agree, so every lane works on 16-byte
// pieces: of a 64-column step, lane (groupID, tid4) takes columns [8*tid4, +8) and [32 + 8*tid4, +8)
// of weight rows groupID and groupID+8 and of activation row groupID.
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

MB_DEFINE_LAST_ERROR()

namespace mb {

using bf16 = __nv_bfloat16;

enum { PRO_NONE = 0, PRO_NORM = 1, PRO_PRE = 2 };
enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3, EPI_ROPE = 4 };

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxResident = 4;  // most blocks per multiprocessor the planner counts on
constexpr int kDepth = 4;        // stages of the weight ring
constexpr int kStep = 128;       // columns per stage: 32 per piece, a lane takes 8 of each piece
constexpr int kPieces = kStep / 32;
static_assert(kStep % 32 == 0 && kPieces >= 1 && kDepth >= 2, "a stage is a whole number of 32-column pieces");

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128_zero(uint32_t addr) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(addr), "r"(0u) : "memory");
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct SkinnyArgs {
    const bf16* w;
    int ldw, n, k, batch;
    const bf16* x;        // PRO_NONE, PRO_PRE: [batch, k]
    int ldx;
    const float* xf;      // PRO_NORM: float rows
    int ldxf;
    const float* gain;    // PRO_NORM: [k]
    float eps;
    // PRO_PRE: x holds the rows times the norm's gain, not yet divided by their root mean square; the rows' sums of
    // squares come in parts ([ssq_count][128], a column per row) and the results are scaled by 1 / sqrt(sum / k + eps)
    // (integrallis/models, backend-java/.../ops/TensorOps.java:45-58)
    const float* ssq_parts;
    int ssq_count;
    // EPI_RESIDUAL, optional: beside the new x, write x times the NEXT norm's gain as bfloat16 and, per row tile, the
    // tile's part of every row's sum of squares ([row tiles][128])
    const float* emit_gain;   // [n]
    bf16* emit_rows;          // [batch][ld_emit]
    int ld_emit;
    float* emit_ssq;
    const int* rows;      // optional: activation row b is xf row rows[b]
    bf16* out_bf16;
    float* out_f32;       // EPI_F32 output, or the residual stream for EPI_RESIDUAL
    int ld_out;
    int pair_offset;      // EPI_SWIGLU: the up tile starts pair_offset rows after the gate tile
    int activation;       // EPI_SWIGLU: the gate's activation (MB_ACT_*)
    int k_split;          // blocks of a cluster that share K
    int k_unit;           // columns per block, a multiple of 4 * kStep
    int k_warp;           // columns per warp, a multiple of kStep
    int clusters;         // clusters (of k_split blocks) in the grid; each walks row tiles cluster, cluster + clusters, ...
    int dependent;        // launch as a programmatic dependent of the kernel before it
    // EPI_ROPE
    int heads, kv_heads, head_dim, page_size;
    const int* positions;     // [batch]
    const int* slot_mapping;  // [batch] flat cache position, < 0: do not store
    const float* cos_table;   // [positions][head_dim / 2]
    const float* sin_table;
    bf16* k_pool;             // [pages][kv_heads][page_size][head_dim]
    bf16* v_pool;
};

// Shared memory of a block, in bytes from the start:
//   activations  [NT*8 rows][k_unit*2 + 64]          (row stride = 64 mod 128 keeps 8-lane phases conflict-free)
//   ring         [4 warps][kDepth][2 halves][kPieces][32 lanes][16]
//   partial      [2 buffers][4 warps][16][NT*8] floats, then sums of squares [NT*8], [4][NT*8]
template <int NT, int EPI>
struct SmemPlan {
    static constexpr int COLS = NT * 8;
    static constexpr int kStageBytes = 2 * kPieces * 32 * 16;
    static constexpr int kPartialFloats = kWarps * 16 * COLS;
    static __host__ __device__ int x_stride(int k_unit) { return k_unit * 2 + 64; }
    static __host__ __device__ int ring_offset(int k_unit) { return COLS * x_stride(k_unit); }
    static __host__ __device__ int partial_offset(int k_unit) { return ring_offset(k_unit) + kWarps * kDepth * kStageBytes; }
    static __host__ __device__ int total(int k_unit) {
        return partial_offset(k_unit) + (2 * kPartialFloats + COLS + kWarps * COLS) * (int)sizeof(float);
    }
};

template <int NT, int PRO, int EPI>
__global__ void __launch_bounds__(kThreads)
skinny_gemm_kernel(const SkinnyArgs args) {
    using Plan = SmemPlan<NT, EPI>;
    constexpr int COLS = Plan::COLS;
    constexpr bool kPaired = EPI == EPI_SWIGLU || EPI == EPI_ROPE;  // MMA rows 8..15 are the partners of rows 0..7
    constexpr int kTileRows = kPaired ? 8 : 16;  // output rows (or pairs) per tile
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group_id = lane >> 2, tid4 = lane & 3;
    const int rank = args.k_split > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int cluster_id = blockIdx.x / args.k_split, clusters = gridDim.x / args.k_split;
    const int rows_total = EPI == EPI_SWIGLU ? args.pair_offset : (EPI == EPI_ROPE ? args.n / 2 : args.n);  // rows, or pairs
    const int tiles_total = (rows_total + kTileRows - 1) / kTileRows;
    const int tiles_mine = cluster_id < tiles_total ? (tiles_total - cluster_id + clusters - 1) / clusters : 0;
    // K: the block's part, then this warp's slice of it
    const int part_begin = rank * args.k_unit;
    const int part_end = min(args.k, part_begin + args.k_unit);
    const int k_begin = min(part_end, part_begin + warp * args.k_warp);
    const int k_end = min(part_end, k_begin + args.k_warp);
    const int steps = (k_end - k_begin + kStep - 1) / kStep;
    const int stages_total = tiles_mine * steps;

    // where this lane reads its activations: row group_id (and 8, 16, ... further), its warp's columns of K, the lane's 8 of every 32
    const int x_stride = Plan::x_stride(args.k_unit);
    const uint32_t x_lane = smem_base + group_id * x_stride + ((k_begin - part_begin) + 8 * tid4) * 2;
    // Activations that arrive as bfloat16 are not staged ahead of the products: every lane fetches exactly the pieces that
    // it will read itself (no barrier, not even within the warp), those of a step of K together with the step's weights.
    auto issue_activations = [&](int step) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < kPieces; ++c) {
                const int row = nt * 8 + group_id, col = k_begin + step * kStep + 32 * c + 8 * tid4;
                const uint32_t dst = x_lane + nt * 8 * x_stride + (step * kStep + 32 * c) * 2;
                if (row < args.batch && col < k_end) cp_async16(dst, args.x + (size_t)row * args.ldx + col);
                else sts128_zero(dst);
            }
    };
    // ---- weights: this lane's pieces of each stage go to ring[stage][half][piece][lane]
    const uint32_t ring = smem_base + Plan::ring_offset(args.k_unit) + warp * kDepth * Plan::kStageBytes;
    auto issue = [&](int stage_index, bool with_activations) {
        if (PRO != PRO_NORM && with_activations && stage_index < steps) issue_activations(stage_index);  // (the first row tile's steps)
        const int tile = cluster_id + (stage_index / steps) * clusters, step = stage_index % steps;
        const uint32_t stage = ring + (stage_index % kDepth) * Plan::kStageBytes;
        const int kc = k_begin + step * kStep + 8 * tid4;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // MMA rows groupID and groupID+8: 16 consecutive weight rows, or 8 gate rows and their 8 up rows
            int row;
            if (EPI == EPI_SWIGLU) {
                row = min(rows_total - 1, tile * 8 + group_id) + h * args.pair_offset;
            } else if (EPI == EPI_ROPE) {  // tile = (head, eighth of its first half); partner half a head further
                const int tiles_per_head = args.head_dim / 16;
                row = (tile / tiles_per_head) * args.head_dim + (tile % tiles_per_head) * 8 + group_id + h * (args.head_dim / 2);
            } else {
                row = min(rows_total - 1, tile * 16 + group_id + 8 * h);
            }
            const bf16* w_row = args.w + (size_t)row * args.ldw;
#pragma unroll
            for (int c = 0; c < kPieces; ++c) {
                const int kk = kc + 32 * c;
                const uint32_t dst = stage + ((h * kPieces + c) * 32 + lane) * 16;
                if (kk < k_end) cp_async16(dst, w_row + kk);
                else sts128_zero(dst);
            }
        }
    };
    grid_launch_dependents();  // the next kernel's blocks may be scheduled as this one's leave
    // Weights depend on nothing: every stage of the ring is asked for before the wait.  (All of them, not all but one:
    // a warp of the q/k/v or output product has four steps in all, and its last step's weights would otherwise be
    // asked for after the wait and arrive from memory on the critical path.)
    for (int s = 0; s < kDepth; ++s) {
        if (s < stages_total) issue(s, false);
        cp_async_commit();
    }
    // What depends on no kernel of this step is asked for before the wait as well: the step's indices (written before the
    // step began) and weights -- the position, cache slot, cosine and sine of this thread's first finishing item, the next
    // norm's gain for it, and this norm's gain on its way into L2.
    int my_position = 0, my_slot = -1;   // EPI_ROPE: of the batch column of this thread's first finishing item
    float first_a = 0.0f, first_b = 0.0f;  // EPI_ROPE: its cosine and sine in the first row tile; EPI_RESIDUAL: the next norm's gain
    {
        const int row_in_tile = threadIdx.x % kTileRows, col = threadIdx.x / kTileRows;
        if (EPI == EPI_ROPE && col < args.batch) {
            my_position = args.positions[col];
            my_slot = args.slot_mapping[col];
            const int tiles_per_head = args.head_dim / 16;
            if (tiles_mine > 0 && cluster_id / tiles_per_head < args.heads + args.kv_heads) {
                const size_t at_table = (size_t)my_position * (args.head_dim / 2) + (cluster_id % tiles_per_head) * 8 + row_in_tile;
                first_a = args.cos_table[at_table];
                first_b = args.sin_table[at_table];
            }
        }
        if (EPI == EPI_RESIDUAL && args.emit_gain != nullptr && tiles_mine > 0 && cluster_id * kTileRows + row_in_tile < rows_total)
            first_a = args.emit_gain[cluster_id * kTileRows + row_in_tile];
        if (PRO == PRO_NORM)
            for (int c = threadIdx.x * 32; c < part_end - part_begin; c += kThreads * 32)  // a line of 128 bytes each
                asm volatile("prefetch.global.L2 [%0];" ::"l"(args.gain + part_begin + c));
    }
    grid_dependency_wait();  // from here on the results of the kernel before this one are visible

    // ---- activations of this block's part of K -> shared memory, bfloat16
    float* partial = reinterpret_cast<float*>(smem + Plan::partial_offset(args.k_unit));  // two buffers
    float* sq_total = partial + 2 * Plan::kPartialFloats;  // [COLS]
    float* sq_warp = sq_total + COLS;                      // [kWarps][COLS]
    const int chunks = (part_end - part_begin + 7) / 8;
    const int chunks_padded = args.k_unit / 8;  // the last steps may read past the part: zeros there
    constexpr int kHeld = COLS <= 16 ? COLS / 4 : 1;
    float4 parts_held[kHeld];  // PRO_PRE: the thread's first part of every row's sum of squares, asked for early, used late
    if (PRO != PRO_NORM) {
        // the activations of the steps whose weights are under way already; the rest follow step by step
        for (int s = 0; s < kDepth && s < steps; ++s) issue_activations(s);
        cp_async_commit();
        if (PRO == PRO_PRE) {
            // asked for now, looked at only when the first row tile is finished: the products do not wait for them
#pragma unroll
            for (int c = 0; c < kHeld; ++c)
                parts_held[c] = (int)threadIdx.x < args.ssq_count
                                    ? __ldcg(reinterpret_cast<const float4*>(args.ssq_parts + (size_t)threadIdx.x * 128 + 4 * c))
                                    : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        cp_async_wait<0>();
    } else {
        for (int b = 0; b < COLS; ++b) {
            const int live_chunks = b < args.batch ? max(chunks, 0) : 0;
            for (int c = live_chunks + threadIdx.x; c < chunks_padded; c += kThreads) sts128_zero(smem_base + b * x_stride + c * 16);
        }
#pragma unroll
        for (int b0 = 0; b0 < COLS; b0 += 8) {  // eight rows at a time: all their loads are issued before any is used
            if (b0 >= args.batch) break;
            const float* src[8];
            float ss[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int b = b0 + j;
                src[j] = args.xf + (size_t)(b < args.batch ? (args.rows ? args.rows[b] : b) : 0) * args.ldxf + part_begin;
                ss[j] = 0.0f;
            }
            for (int c = threadIdx.x; c < chunks; c += kThreads) {
                const float4 ga = *reinterpret_cast<const float4*>(args.gain + part_begin + c * 8);
                const float4 gd = *reinterpret_cast<const float4*>(args.gain + part_begin + c * 8 + 4);
                float4 a[8], d[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (b0 + j < args.batch) {
                        a[j] = *reinterpret_cast<const float4*>(src[j] + c * 8);
                        d[j] = *reinterpret_cast<const float4*>(src[j] + c * 8 + 4);
                    }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (b0 + j < args.batch) {
                        ss[j] += a[j].x * a[j].x + a[j].y * a[j].y + a[j].z * a[j].z + a[j].w * a[j].w + d[j].x * d[j].x +
                                 d[j].y * d[j].y + d[j].z * d[j].z + d[j].w * d[j].w;
                        *reinterpret_cast<uint4*>(smem + (b0 + j) * x_stride + c * 16) =
                            make_uint4(pack2(a[j].x * ga.x, a[j].y * ga.y), pack2(a[j].z * ga.z, a[j].w * ga.w),
                                       pack2(d[j].x * gd.x, d[j].y * gd.y), pack2(d[j].z * gd.z, d[j].w * gd.w));
                    }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float total = warp_sum(ss[j]);
                if (lane == 0) sq_warp[warp * COLS + b0 + j] = total;
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
    }
    if (PRO == PRO_NORM && threadIdx.x < COLS) {
        float s = 0.0f;
        if (threadIdx.x < (args.batch + 7) / 8 * 8)
            for (int w = 0; w < kWarps; ++w) s += sq_warp[w * COLS + threadIdx.x];
        sq_total[threadIdx.x] = s;
    }
    bool sq_gathered = args.k_split == 1;


    // ---- row tile after row tile; the ring keeps running across them
    int stage_index = 0;
    for (int local = 0; local < tiles_mine; ++local) {
        const int tile = cluster_id + local * clusters;
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
        for (int step = 0; step < steps; ++step, ++stage_index) {
            cp_async_wait<kDepth - 1>();  // this lane's pieces of the stage have landed; nobody else reads them
            const uint32_t stage = ring + (stage_index % kDepth) * Plan::kStageBytes;
            uint4 wv[2][kPieces];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < kPieces; ++c) wv[h][c] = lds128(stage + ((h * kPieces + c) * 32 + lane) * 16);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int c = 0; c < kPieces; ++c) {
                    const uint4 xv = lds128(x_lane + nt * 8 * x_stride + (step * kStep + 32 * c) * 2);
                    mma_bf16(acc[nt], wv[0][c].x, wv[1][c].x, wv[0][c].y, wv[1][c].y, xv.x, xv.y);
                    mma_bf16(acc[nt], wv[0][c].z, wv[1][c].z, wv[0][c].w, wv[1][c].w, xv.z, xv.w);
                }
            }
            // the stage has been read (by this lane, in program order): its slot takes the stage a ring's length further on
            if (stage_index + kDepth < stages_total) issue(stage_index + kDepth, true);
            cp_async_commit();
        }

        // the warps' partial sums of this row tile: c0,c1 = (MMA row groupID, activation rows 2*tid4, +1); c2,c3 = row +8
        float* mine = partial + (local & 1) * Plan::kPartialFloats;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                mine[(warp * 16 + group_id + 8 * (i >> 1)) * COLS + nt * 8 + tid4 * 2 + (i & 1)] = acc[nt][i];
        if (PRO == PRO_PRE && local == 0) {
            // every row's sum of squares: the parts in their order within a thread, then a fixed tree over lanes and warps
#pragma unroll
            for (int c = 0; c < kHeld; ++c) {
                float4 sum = parts_held[c];
                for (int part = threadIdx.x + kThreads; part < args.ssq_count; part += kThreads) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(args.ssq_parts + (size_t)part * 128 + 4 * c));
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                const float4 total = make_float4(warp_sum(sum.x), warp_sum(sum.y), warp_sum(sum.z), warp_sum(sum.w));
                if (lane == 0) *reinterpret_cast<float4*>(&sq_warp[warp * COLS + 4 * c]) = total;
            }
        }
        // What this thread's first item of the finishing below reads from memory is asked for before the block meets:
        // the residual stream's old value, or the rotation's cosine and sine (the position was read before the loop).
        float early_a = 0.0f, early_b = 0.0f;
        {
            const int row_in_tile = threadIdx.x % kTileRows, col = threadIdx.x / kTileRows;
            const int row = tile * kTileRows + row_in_tile;
            if (rank == 0 && row < rows_total && col < args.batch) {
                if (EPI == EPI_RESIDUAL) early_a = args.out_f32[(size_t)col * args.ld_out + row];
                if (EPI == EPI_ROPE) {
                    const int tiles_per_head = args.head_dim / 16;
                    if (local == 0) {
                        early_a = first_a;
                        early_b = first_b;
                    } else if (tile / tiles_per_head < args.heads + args.kv_heads) {
                        const size_t at_table = (size_t)my_position * (args.head_dim / 2) + (tile % tiles_per_head) * 8 + row_in_tile;
                        early_a = args.cos_table[at_table];
                        early_b = args.sin_table[at_table];
                    }
                }
            }
        }
        if (args.k_split > 1) {
            cg::this_cluster().sync();
            if (rank != 0) continue;
            if (PRO == PRO_NORM && !sq_gathered) {
                if (threadIdx.x < COLS) {
                    float s = 0.0f;
                    for (int r = 0; r < args.k_split; ++r) s += cg::this_cluster().map_shared_rank(sq_total, r)[threadIdx.x];
                    sq_warp[threadIdx.x] = s;  // the whole row's sum of squares
                }
                __syncthreads();
                sq_total = sq_warp;
                sq_gathered = true;
            }
        } else {
            __syncthreads();
        }
        for (int i = threadIdx.x; i < kTileRows * COLS; i += kThreads) {
            const int row_in_tile = i % kTileRows, col = i / kTileRows;  // neighbouring threads store neighbouring output columns
            const int row = tile * kTileRows + row_in_tile;
            const bool emits = EPI == EPI_RESIDUAL && args.emit_gain != nullptr;
            float squares = 0.0f;  // of the new x, where the next norm's rows are prepared
            if (row >= rows_total || col >= args.batch) {
                if (!emits) continue;  // (with them, whole warps stay for the sums below)
            } else {
            float value = 0.0f, second = 0.0f;  // second: the up row that matches a gate row
            for (int r = 0; r < args.k_split; ++r) {
                const float* from = args.k_split > 1 ? cg::this_cluster().map_shared_rank(mine, r) : mine;
                for (int w = 0; w < kWarps; ++w) {
                    value += from[(w * 16 + row_in_tile) * COLS + col];
                    if (kPaired) second += from[(w * 16 + row_in_tile + 8) * COLS + col];
                }
            }
            if (PRO == PRO_NORM) {
                const float inv_rms = 1.0f / sqrtf(sq_total[col] / (float)args.k + args.eps);
                value *= inv_rms;
                second *= inv_rms;
            }
            if (PRO == PRO_PRE) {
                float sum = 0.0f;
                for (int w = 0; w < kWarps; ++w) sum += sq_warp[w * COLS + col];
                const float inv_rms = 1.0f / sqrtf(sum / (float)args.k + args.eps);
                value *= inv_rms;
                second *= inv_rms;
            }
            const size_t at = (size_t)col * args.ld_out + row;
            if (EPI == EPI_BF16) args.out_bf16[at] = __float2bfloat16_rn(value);
            if (EPI == EPI_F32) args.out_f32[at] = value;
            if (EPI == EPI_RESIDUAL) {
                const float x_new = (i == (int)threadIdx.x ? early_a : args.out_f32[at]) + value;
                args.out_f32[at] = x_new;
                if (emits) {
                    const float gain = (local == 0 && i == (int)threadIdx.x) ? first_a : args.emit_gain[row];
                    args.emit_rows[(size_t)col * args.ld_emit + row] = __float2bfloat16_rn(x_new * gain);
                    squares = x_new * x_new;
                }
            }
            if (EPI == EPI_SWIGLU) args.out_bf16[at] = __float2bfloat16_rn(gate_activation(args.activation, value) * second);
            if (EPI == EPI_ROPE) {
                const int tiles_per_head = args.head_dim / 16, half = args.head_dim / 2;
                const int head = tile / tiles_per_head, d0 = (tile % tiles_per_head) * 8 + row_in_tile;
                // queries and keys pass through bfloat16 before the rotation, as they do when the product stores them
                float x0 = __bfloat162float(__float2bfloat16_rn(value)), x1 = __bfloat162float(__float2bfloat16_rn(second));
                if (head < args.heads + args.kv_heads) {
                    const bool early = i == (int)threadIdx.x;
                    const size_t at_table = early ? 0 : (size_t)args.positions[col] * half + d0;
                    const float c = early ? early_a : args.cos_table[at_table], sn = early ? early_b : args.sin_table[at_table];
                    const float r0 = x0 * c - x1 * sn, r1 = x0 * sn + x1 * c;
                    x0 = r0;
                    x1 = r1;
                }
                if (head < args.heads) {
                    bf16* q = args.out_bf16 + (size_t)col * args.ld_out + (size_t)head * args.head_dim;
                    q[d0] = __float2bfloat16_rn(x0);
                    q[d0 + half] = __float2bfloat16_rn(x1);
                } else {
                    const int slot = i == (int)threadIdx.x ? my_slot : args.slot_mapping[col];
                    if (slot >= 0) {
                        const bool is_key = head < args.heads + args.kv_heads;
                        const int kv_head = head - args.heads - (is_key ? 0 : args.kv_heads);
                        const size_t page = slot / args.page_size, offset = slot % args.page_size;
                        bf16* dst = (is_key ? args.k_pool : args.v_pool) +
                                    ((page * args.kv_heads + kv_head) * args.page_size + offset) * args.head_dim;
                        dst[d0] = __float2bfloat16_rn(x0);
                        dst[d0 + half] = __float2bfloat16_rn(x1);
                    }
                }
            }
            }
            if (emits) {
                // the sixteen threads of a batch column (one per row of the tile) add their squares, a fixed tree; their
                // first writes the tile's part
                squares += __shfl_xor_sync(0xffffffffu, squares, 8);
                squares += __shfl_xor_sync(0xffffffffu, squares, 4);
                squares += __shfl_xor_sync(0xffffffffu, squares, 2);
                squares += __shfl_xor_sync(0xffffffffu, squares, 1);
                if ((lane & 15) == 0 && col < args.batch) args.emit_ssq[(size_t)tile * 128 + col] = squares;
            }
        }
    }
    // a cluster's blocks leave together: the first block reads the others' shared memory until the end
    if (args.k_split > 1) cluster_leave_together();
}

template <int NT, int PRO, int EPI>
static int launch(const SkinnyArgs& args, cudaStream_t stream) {
    using Plan = SmemPlan<NT, EPI>;
    const int smem = Plan::total(args.k_unit);
    auto kernel = skinny_gemm_kernel<NT, PRO, EPI>;
    static int reserved = 0;
    if (smem > reserved) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (status != cudaSuccess) return fail("skinny_gemm: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(status));
        reserved = smem;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(args.clusters * args.k_split);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = args.k_split;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = (args.dependent && dependent_launches_allowed()) ? 2 : 1;
    cudaError_t status = cudaLaunchKernelEx(&config, kernel, args);
    if (status != cudaSuccess) return fail("skinny_gemm: launch failed: %s", cudaGetErrorString(status));
    return check_launch("skinny_gemm");
}

template <int PRO, int EPI>
static int launch_nt(const SkinnyArgs& args, cudaStream_t stream) {
    if (args.batch <= 8) return launch<1, PRO, EPI>(args, stream);
    if (args.batch <= 16) return launch<2, PRO, EPI>(args, stream);
    if (PRO != PRO_NONE) return fail("skinny_gemm: the norm prologues take at most 16 rows, got %d", args.batch);
    if (args.batch <= 32) return launch<4, PRO_NONE, EPI>(args, stream);
    return fail("skinny_gemm: takes at most 32 activation rows, got %d", args.batch);
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_skinny_max_rows(int with_norm) { return with_norm ? 16 : 32; }

// w: bfloat16 [n, k] (row stride ldw).  Activations: x (bfloat16 [batch, k]) when gain is null,
// else xf (float32 rows, optionally picked by `rows`) normalised with `gain` and `eps`.
// epilogue 0: out bfloat16 [batch, n]; 1: out float32; 2: out float32 += ; 3: w holds gate rows
// [0, n/2) and up rows [n/2, n), out bfloat16 [batch, n/2] = act(gate) * up with the activation code
// (MB_ACT_*) in bits 8 and up of `epilogue`.
static int skinny_gemm(const void* w, int ldw, int n, int k, int batch, const void* x, int ldx, const float* xf,
                       int ldxf, const float* gain, float eps, const int* rows, void* out, int ld_out,
                       int epilogue, int multiprocessors, int dependent, SkinnyArgs args, cudaStream_t stream) {
    if (batch <= 0 || n <= 0) return 0;
    const int activation = epilogue >> 8;
    epilogue &= 0xff;
    if (activation < 0 || activation >= MB_ACT_COUNT) return fail("skinny_gemm: unknown gate activation code %d", activation);
    args.activation = activation;
    if (batch > 32) return fail("skinny_gemm: takes at most 32 activation rows, got %d", batch);
    if (k <= 0 || k % 8 || ldw % 8) return fail("skinny_gemm: k (%d) and the weight row stride (%d) must be multiples of 8", k, ldw);
    if ((uintptr_t)w & 15) return fail("skinny_gemm: the weight matrix must start on a 16-byte boundary");
    const bool norm = gain != nullptr;
    if (norm && (!xf || ldxf % 4 || ((uintptr_t)xf & 15) || ((uintptr_t)gain & 15)))
        return fail("skinny_gemm: the norm prologue needs 16-byte aligned float rows and gain");
    if (!norm && (!x || ldx % 8 || ((uintptr_t)x & 15))) return fail("skinny_gemm: activations need 16-byte aligned bfloat16 rows");
    if (epilogue == EPI_SWIGLU && n % 2) return fail("skinny_gemm: the gated epilogue needs an even number of weight rows, got %d", n);
    args.w = (const bf16*)w; args.ldw = ldw; args.n = n; args.k = k; args.batch = batch;
    args.x = (const bf16*)x; args.ldx = ldx; args.xf = xf; args.ldxf = ldxf; args.gain = gain; args.eps = eps; args.rows = rows;
    args.out_bf16 = (bf16*)out; args.out_f32 = (float*)out; args.ld_out = ld_out;
    args.pair_offset = epilogue == EPI_SWIGLU ? n / 2 : 0;
    args.dependent = dependent;
    if (epilogue == EPI_SWIGLU) args.n = n / 2;
    // Planning.  A block's shared memory holds its activations (rows x k_unit bfloat16), the warps' rings
    // and the partial sums; as many blocks as fit stay resident per multiprocessor (at most four).
    // K is split over a cluster only when a block's activations would not fit otherwise: splitting it
    // to fill idle multiprocessors was measured and lost to the cluster barrier it adds.  Blocks walk
    // several row tiles when there are more tiles than resident blocks.
    const int rows_total = (epilogue == EPI_SWIGLU || epilogue == EPI_ROPE) ? n / 2 : n;
    const int tiles = (epilogue == EPI_SWIGLU || epilogue == EPI_ROPE) ? (rows_total + 7) / 8 : (rows_total + 15) / 16;
    const int cols = batch <= 8 ? 8 : (batch <= 16 ? 16 : 32);
    auto smem_for = [&](int split) {
        const int k_unit = ((k + split - 1) / split + kWarps * kStep - 1) / (kWarps * kStep) * (kWarps * kStep);
        return (size_t)cols * (k_unit * 2 + 64) + (size_t)kWarps * kDepth * (2 * kPieces * 512) +
               (size_t)(2 * kWarps * 16 * cols + (1 + kWarps) * cols) * sizeof(float);
    };
    auto resident_for = [&](int split) {
        const size_t per_sm = 220 * 1024 / smem_for(split);
        return multiprocessors * (int)(per_sm > kMaxResident ? kMaxResident : per_sm);
    };
    int split = 1;
    while (split < 8 && smem_for(split) > 200 * 1024) split *= 2;
    if (smem_for(split) > 200 * 1024)
        return fail("skinny_gemm: %d activation rows of %d columns do not fit shared memory", batch, k);
    args.k_split = split;
    args.k_unit = ((k + split - 1) / split + kWarps * kStep - 1) / (kWarps * kStep) * (kWarps * kStep);
    args.k_warp = args.k_unit / kWarps;
    const int resident_clusters = resident_for(split) / split;
    args.clusters = tiles < resident_clusters ? tiles : resident_clusters;
    if (args.clusters < 1) args.clusters = 1;
    const int prologue = norm ? PRO_NORM : (args.ssq_parts ? PRO_PRE : PRO_NONE);
    if (prologue == PRO_PRE && (batch > 16 || args.ssq_count <= 0 || ((uintptr_t)args.ssq_parts & 15)))
        return fail("skinny_gemm: parts of sums of squares come with at most 16 rows, a count, and 16-byte alignment");
    if (args.emit_gain && (epilogue != EPI_RESIDUAL || !args.emit_rows || !args.emit_ssq))
        return fail("skinny_gemm: the next norm's rows are written by the residual epilogue, with buffers for them");
#define MB_CASE(PRO, EPI) \
    if (prologue == PRO && epilogue == EPI) return launch_nt<PRO, EPI>(args, stream);
    MB_CASE(PRO_NONE, EPI_BF16)
    MB_CASE(PRO_NONE, EPI_F32)
    MB_CASE(PRO_NONE, EPI_RESIDUAL)
    MB_CASE(PRO_NORM, EPI_BF16)
    MB_CASE(PRO_NORM, EPI_F32)
    MB_CASE(PRO_NORM, EPI_SWIGLU)
    MB_CASE(PRO_NONE, EPI_SWIGLU)
    MB_CASE(PRO_NORM, EPI_ROPE)
    MB_CASE(PRO_NONE, EPI_ROPE)
    MB_CASE(PRO_PRE, EPI_BF16)
    MB_CASE(PRO_PRE, EPI_F32)
    MB_CASE(PRO_PRE, EPI_SWIGLU)
    MB_CASE(PRO_PRE, EPI_ROPE)
#undef MB_CASE
    return fail("skinny_gemm: no kernel for prologue %d with epilogue %d", prologue, epilogue);
}

// `dependent` != 0 launches the kernel as a programmatic dependent of the kernel before it in the stream.
// ssq_parts (or null; then x is the rows times their norm's gain): [ssq_count][128] parts of the rows' sums of squares;
// the results are scaled by 1 / sqrt(sum / k + eps).  emit_gain (or null; residual epilogue only): the next norm's gain;
// the new rows times it go to emit_rows (bfloat16, row stride ld_emit), a part of their sums of squares per tile of 16
// weight rows to emit_ssq ([(n + 15) / 16][128]), and *parts_written says how many parts there are.
MB_EXPORT int mb_skinny_gemm(const void* w, int ldw, int n, int k, int batch, const void* x, int ldx, const float* xf,
                             int ldxf, const float* gain, float eps, const int* rows, void* out, int ld_out,
                             int epilogue, int multiprocessors, int dependent, const float* ssq_parts, int ssq_count,
                             const float* emit_gain, void* emit_rows, int ld_emit, float* emit_ssq, int* parts_written,
                             cudaStream_t stream) {
    if ((epilogue & 0xff) == EPI_ROPE) return fail("skinny_gemm: the rotary epilogue has an entry point of its own");
    SkinnyArgs args{};
    args.ssq_parts = ssq_parts; args.ssq_count = ssq_count;
    args.emit_gain = emit_gain; args.emit_rows = (bf16*)emit_rows; args.ld_emit = ld_emit; args.emit_ssq = emit_ssq;
    if (parts_written) *parts_written = (n + 15) / 16;
    return skinny_gemm(w, ldw, n, k, batch, x, ldx, xf, ldxf, gain, eps, rows, out, ld_out, epilogue, multiprocessors, dependent,
                       args, stream);
}

// The q/k/v product of an attention layer with rotation and cache write folded in.  w: [(heads + 2 *
// kv_heads) * head_dim, k]; rotation over the whole head with split-half pairs; q_out: bfloat16
// [batch, heads * head_dim] (row stride ld_q); keys and values go to the pools at slot_mapping.
MB_EXPORT int mb_skinny_qkv_rope(const void* w, int ldw, int k, int batch, const void* x, int ldx, const float* xf, int ldxf,
                                 const float* gain, float eps, void* q_out, int ld_q, int heads, int kv_heads, int head_dim,
                                 const int* positions, const float* cos_table, const float* sin_table, void* k_pool,
                                 void* v_pool, const int* slot_mapping, int page_size, int multiprocessors, int dependent,
                                 const float* ssq_parts, int ssq_count, cudaStream_t stream) {
    if (head_dim <= 0 || head_dim % 16) return fail("skinny_qkv_rope: head_dim %d must be a multiple of 16", head_dim);
    if (!positions || !cos_table || !sin_table || !k_pool || !v_pool || !slot_mapping || page_size <= 0)
        return fail("skinny_qkv_rope: needs positions, cos/sin tables, cache pools, a slot mapping and a page size");
    SkinnyArgs args{};
    args.heads = heads; args.kv_heads = kv_heads; args.head_dim = head_dim; args.page_size = page_size;
    args.positions = positions; args.slot_mapping = slot_mapping; args.cos_table = cos_table; args.sin_table = sin_table;
    args.k_pool = (bf16*)k_pool; args.v_pool = (bf16*)v_pool;
    args.ssq_parts = ssq_parts; args.ssq_count = ssq_count;
    return skinny_gemm(w, ldw, (heads + 2 * kv_heads) * head_dim, k, batch, x, ldx, xf, ldxf, gain, eps, nullptr, q_out, ld_q,
                       EPI_ROPE, multiprocessors, dependent, args, stream);
}
