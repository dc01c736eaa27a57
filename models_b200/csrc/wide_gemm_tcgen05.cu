// Decode matrix products for wide batches (9 to 128 activation rows) on the tcgen05 tensor cores.
//
// With this many rows the weights still have to stream exactly once, but the arithmetic no longer
// fits the register-fed MMAs of the narrow decode kernel.  So the operands swap sides: a tile of 128
// WEIGHT rows is the 128-row operand of tcgen05.mma and the activations are the N = 32, 64 or 128
// side; both travel by TMA (the activations, a few hundred KB, are re-read from L2 for every weight
// tile) and the accumulator [128 weight rows x batch] lives in tensor memory.
//
//   * A block works on ONE tile, or on one part of K of one tile: a layer's matrices have 16 to 128
//     row tiles, too few to keep every multiprocessor streaming, so K is split over the 2, 4 or 8
//     blocks of a thread-block CLUSTER.  Their partial accumulators meet in distributed shared
//     memory: every block copies its accumulator from tensor memory into its own shared memory, the
//     cluster meets at its hardware barrier, and each block then finishes a share of the tile's rows,
//     adding the parts in the order of the blocks' ranks -- the same order in every run, no scratch
//     memory, no atomics, nobody polls.
//   * What surrounds the product rides in it, as in the narrow decode kernel (csrc/skinny_gemm.cu):
//     store bf16 / f32; add into the float32 residual stream (x = x + W.h, integrallis/models,
//     backend-java/.../llama/LlamaForwardPass.java:1131-1138,1172-1178); act(gate) * up, a tile then
//     being 64 gate rows and the 64 up rows that match them (backend-java/.../ops/TensorOps.java:1407-1449);
//     and for the q/k/v product the rotation of query and key pairs (x0' = x0*c - x1*s, x1' = x0*s +
//     x1*c, :1481-1486) with the paged cache write of keys and values (backend-java/.../llama/LlamaForwardPass.java:1070-1086).
//   * The kernel is a programmatic dependent of the kernel before it: its first weight tiles are
//     asked for before it waits for that kernel (weights depend on nothing), the activations after.
//
// Every mbarrier wait is bounded as in gemm_tcgen05.cu; mb_wide_gemm_status() reads the record.
#include "tcgen05.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3, EPI_ROPE = 4 };

constexpr int kTileRows = 128;                    // weight rows per tile (UMMA M)
constexpr int kTileBytes = kTileRows * kBlockK * 2;
constexpr int kThreads = 192;                     // warp 0: TMA, warp 1: MMA, warps 2..5: epilogue
constexpr int kFinishThreads = 128;

struct WideArgs {
    int rows_total;       // output columns = weight rows (EPI_SWIGLU: gate rows)
    int up_row_offset;    // EPI_SWIGLU: first up row of W
    int activation;       // EPI_SWIGLU: the gate's activation (MB_ACT_*)
    int batch, k;
    int splits;           // blocks of a cluster that share a tile, each with its own part of K
    int k_blocks_per_split;
    void* out;            // [batch, rows_total] bfloat16 / float32 (row stride ld_out); EPI_ROPE: the queries
    int ld_out;
    // EPI_ROPE: W is [q heads; k heads; v heads], head_dim divides 128
    int heads, kv_heads, head_dim, page_size;
    const int* positions;     // [batch]
    const int* slot_mapping;  // [batch] flat cache position, < 0: do not store
    const float* cos_table;   // [positions][head_dim / 2]
    const float* sin_table;
    bf16* k_pool;             // [pages][kv_heads][page_size][head_dim]
    bf16* v_pool;
    // The RMSNorm around a product, without a kernel of its own.  A product whose activations are x * gain (not yet
    // divided by the root mean square) gets the rows' sums of squares in parts and scales its results by
    // 1 / sqrt(sum / width + eps) (integrallis/models, backend-java/.../ops/TensorOps.java:45-58).  A residual product
    // writes, beside the new x, x * gain of the NEXT norm as bfloat16 and its blocks' parts of the sums of squares.
    const float* ssq_parts;   // [ssq_count][128]: parts of the sums of squares of the activation rows, or null
    int ssq_count;
    int norm_width;
    float eps;
    const float* emit_gain;   // EPI_RESIDUAL: gain of the next norm [rows_total], or null
    bf16* emit_rows;          // [batch][ld_emit]: x * gain
    int ld_emit;
    float* emit_ssq;          // [tiles * splits][128]: this block's part of each row's sum of squares
};

// kStages: eight where every block has a multiprocessor to itself anyway (few tiles: the ring is then all that keeps
// loads in flight); four where there are more blocks than multiprocessors: two then share one, and one streams while the
// other starts or finishes.
template <int kBatchN, int kStageCount>
struct WidePlan {
    static constexpr int kStageBytes = kTileBytes + kBatchN * kBlockK * 2;
    // (two blocks share a multiprocessor in the four-stage form: at 128 activation rows that leaves room for three stages each)
    static constexpr int kWanted = kStageCount == 4 && 4 * kStageBytes > 110 * 1024 ? 3 : kStageCount;
    static constexpr int kStages = kWanted * kStageBytes <= 200 * 1024 ? kWanted : 200 * 1024 / kStageBytes;
    static constexpr int kTmemColumns = kBatchN < 32 ? 32 : kBatchN;
    static constexpr int kPartialBytes = kBatchN * kTileRows * (int)sizeof(float);  // [batch column][128 rows], over the ring
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&pair);
}
// Four floats at the same place of the shared memory of block `rank` of this cluster (distributed shared memory).
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_shared_f32x4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

template <int EPI, int kBatchN, int kStageCount>
__global__ void __launch_bounds__(kThreads, kStageCount > 4 ? 1 : 2)
wide_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const WideArgs args) {
    using Plan = WidePlan<kBatchN, kStageCount>;
    constexpr int kStages = Plan::kStages;
    constexpr uint32_t kInstruction = instruction_descriptor(kTileRows, kBatchN);
    constexpr bool kPaired = EPI == EPI_SWIGLU || EPI == EPI_ROPE;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t barriers[2 * kStages + 1];
    static_assert(Plan::kPartialBytes <= kStages * Plan::kStageBytes, "the accumulator's copy reuses the ring");
    __shared__ uint32_t tmem_base_slot;
    __shared__ float inv_rms[kFinishThreads];  // of the activation rows, when the product carries a norm
    __shared__ __align__(16) float ssq_warp[4][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_u32(&barriers[0]), empty_bar = smem_u32(&barriers[kStages]);
    const uint32_t acc_full_bar = smem_u32(&barriers[2 * kStages]);
    const int splits = args.splits;
    const int rank = splits > 1 ? (int)cluster_rank() : 0;
    const int tile = blockIdx.x / splits;
    const int k_blocks = (args.k + kBlockK - 1) / kBlockK;
    const int kb_begin = rank * args.k_blocks_per_split;
    const int kb_end = min(k_blocks, kb_begin + args.k_blocks_per_split);  // (the launcher leaves no part empty)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        mbar_init(acc_full_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(Plan::kTmemColumns));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    grid_launch_dependents();
    bool ok = true;

    // What a thread's first item of the finishing below reads from memory -- the residual stream's old values and the
    // next norm's gain, or the rotation's cosines and sines and the cache slot -- is asked for long before the parts
    // meet (the item depends only on the thread and the block): by the warps that will copy the accumulator while
    // they wait for it, by the others when their own work is done.  Callers have waited for the kernel before this one.
    // (With 32 batch columns only the first two warps have such an item, and the step measured slower with the rotation's
    // part: there the residual product's threads ask where they always did, and the rotation reads in its loop.)
    constexpr bool kEarlyForAll = kBatchN >= 64;
    float4 early_before = make_float4(0.0f, 0.0f, 0.0f, 0.0f), early_gain = early_before;  // EPI_ROPE: cosines, sines
    int early_slot = -1;
    auto load_early = [&]() {
        if (EPI == EPI_RESIDUAL) {
            const int quads = 128 / splits / 4, item = threadIdx.x;
            const int row = tile * kTileRows + rank * (128 / splits) + (item & (quads - 1)) * 4, col = item / quads;
            if (col < args.batch && row < args.rows_total) {
                early_before = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(args.out) + (size_t)col * args.ld_out + row);
                if (args.emit_gain) early_gain = *reinterpret_cast<const float4*>(args.emit_gain + row);
            }
        }
        if (EPI == EPI_ROPE && kEarlyForAll) {
            const int quads = 64 / splits / 4, item = threadIdx.x;
            const int unit = rank * (64 / splits) + (item & (quads - 1)) * 4, col = item / quads;
            const int hd = args.head_dim, half = hd / 2;
            const int head = tile * (kTileRows / hd) + unit / half, d0 = unit % half;
            if (col < args.batch && head < args.heads + 2 * args.kv_heads) {
                early_slot = args.slot_mapping[col];
                if (head < args.heads + args.kv_heads) {
                    const size_t at_table = (size_t)args.positions[col] * half + d0;
                    early_before = *reinterpret_cast<const float4*>(args.cos_table + at_table);
                    early_gain = *reinterpret_cast<const float4*>(args.sin_table + at_table);
                }
            }
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // the weight rows of MMA rows 0..127: 128 consecutive rows, or 64 gate rows and the 64 up rows that match them
            auto load_weights = [&](uint32_t dst, int kb, uint32_t bar) {
                if (EPI == EPI_SWIGLU) {
                    tma_load_2d(dst, &map_w, kb * kBlockK, tile * 64, bar);
                    tma_load_2d(dst + kTileBytes / 2, &map_w, kb * kBlockK, args.up_row_offset + tile * 64, bar);
                } else {
                    tma_load_2d(dst, &map_w, kb * kBlockK, tile * kTileRows, bar);
                }
            };
            // the first weight tiles go out before this kernel waits for the one before it; the activations after
            const int early = min(kStages, kb_end - kb_begin);
            for (int s = 0; s < early; ++s) {
                mbar_expect_tx(full_bar + 8 * s, Plan::kStageBytes);
                load_weights(smem_u32(smem) + s * Plan::kStageBytes, kb_begin + s, full_bar + 8 * s);
            }
            grid_dependency_wait();
            for (int s = 0; s < early; ++s)
                tma_load_2d(smem_u32(smem) + s * Plan::kStageBytes + kTileBytes, &map_x, (kb_begin + s) * kBlockK, 0, full_bar + 8 * s);
            int stage = 0;
            uint32_t phase = 0;  // the second pass over the ring waits for the first pass's products
            for (int kb = kb_begin + early; kb < kb_end; ++kb) {
                if (!(ok = mbar_wait(empty_bar + 8 * stage, phase, 1))) break;
                const uint32_t dst = smem_u32(smem) + stage * Plan::kStageBytes;
                mbar_expect_tx(full_bar + 8 * stage, Plan::kStageBytes);
                load_weights(dst, kb, full_bar + 8 * stage);
                tma_load_2d(dst + kTileBytes, &map_x, kb * kBlockK, 0, full_bar + 8 * stage);
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!(ok = mbar_wait(full_bar + 8 * stage, phase, 3))) break;
                tcgen05_fence_after();
                const uint32_t base = smem_u32(smem) + stage * Plan::kStageBytes;
                const uint64_t w_desc = umma_descriptor(base), x_desc = umma_descriptor(base + kTileBytes);
#pragma unroll
                for (int ks = 0; ks < kBlockK / 16; ++ks)
                    umma(tmem_base, w_desc + 2 * ks, x_desc + 2 * ks, kInstruction, (kb > kb_begin || ks > 0) ? 1u : 0u);
                umma_commit(empty_bar + 8 * stage);
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) umma_commit(acc_full_bar);
        }
    } else {
        // ------------------------------------------------------------------ the accumulator -> this block's shared memory
        grid_dependency_wait();  // (what the finishing below reads and adds into comes from the kernel before this one)
        if (kEarlyForAll) load_early();
        const int quarter = warp & 3;
        if (args.ssq_parts) {
            // while the products run: 1 / rms of every activation row from the parts of its sum of squares.  Every lane
            // takes four rows, every warp a quarter of the parts (in their order, eight loads in flight at a time); the
            // warps' sums are then added in the order of the warps.
            const int per_warp = (args.ssq_count + 3) / 4;
            const int p_begin = min(args.ssq_count, quarter * per_warp), p_end = min(args.ssq_count, p_begin + per_warp);
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float4* parts = reinterpret_cast<const float4*>(args.ssq_parts) + lane;
#pragma unroll 8
            for (int p = p_begin; p < p_end; ++p) {
                const float4 v = __ldcg(parts + (size_t)p * 32);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            *reinterpret_cast<float4*>(&ssq_warp[quarter][4 * lane]) = sum;
            asm volatile("bar.sync 1, %0;" ::"r"(kFinishThreads) : "memory");
            const int col = threadIdx.x - 64;
            const float total = ssq_warp[0][col] + ssq_warp[1][col] + ssq_warp[2][col] + ssq_warp[3][col];
            inv_rms[col] = col < args.batch ? 1.0f / sqrtf(total / (float)args.norm_width + args.eps) : 0.0f;
        }
        ok = mbar_wait(acc_full_bar, 0, 4);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tcgen05_fence_after();
            // every product has read the ring: it now holds the accumulator, [batch column][128 rows]
            float* partial = reinterpret_cast<float*>(smem);
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < kBatchN; c += 32) {
                float v[32];
                tmem_load_32(taddr + c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) partial[(c + i) * kTileRows + quarter * 32 + lane] = v[i];
            }
        }
    }

    if (kEarlyForAll) {
        if (warp < 2 && (EPI == EPI_RESIDUAL || EPI == EPI_ROPE)) {
            grid_dependency_wait();
            load_early();
        }
    } else if (EPI == EPI_RESIDUAL) {
        if (warp < 2) grid_dependency_wait();
        load_early();
    }

    // ---- the parts of K meet: every block of the cluster has its accumulator in its shared memory
    tcgen05_fence_before();
    if (splits > 1) cluster_sync_all();
    else __syncthreads();

    {
        // ------------------------------------------------------------------ finishing: a share of the tile's rows (or pairs of rows) per
        // block, four neighbouring rows per thread and step (they are neighbours in shared memory and in the output);
        // all six warps take part (the loading and the issuing warp have nothing left to do)
        if (warp < 2) grid_dependency_wait();  // (their lanes read what the kernel before this one wrote, too)
        const int t = threadIdx.x;
        const uint32_t partial_addr = smem_u32(smem);
        constexpr int kUnits = kPaired ? 64 : 128;     // rows, or pairs of rows, of a tile
        const int per_block = kUnits / splits;         // splits is 1, 2, 4 or 8: a multiple of 4, and a power of two
        const int quads = per_block / 4;
        const int quad_shift = 31 - __clz(quads);
        const int first = rank * per_block;
        auto sum_parts = [&](int mma_row, int col) {   // rows mma_row .. mma_row + 3 of batch column col, over all parts of K
            const uint32_t at = partial_addr + (uint32_t)(col * kTileRows + mma_row) * 4u;
            if (splits == 1) return ld_shared_f32x4(at);
            float4 parts[8];  // all loads first (they are independent), then the sums in the order of the ranks
#pragma unroll
            for (int r = 0; r < 8; ++r) parts[r] = r < splits ? ld_cluster_f32x4(at, (uint32_t)r) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                v.x += parts[r].x; v.y += parts[r].y; v.z += parts[r].z; v.w += parts[r].w;
            }
            return v;
        };
        const bool scaled = args.ssq_parts != nullptr;
        const int total = quads * args.batch;
        for (int base = 0; base < total; base += kThreads) {  // (whole warps stay in the loop: the sums below use shuffles)
            const int item = base + t;
            const bool active = item < total;
            const int unit = first + (item & (quads - 1)) * 4, col = active ? item >> quad_shift : 0;  // neighbouring threads: neighbouring rows of one batch row
            const float scale = scaled ? inv_rms[col] : 1.0f;
            if (!kPaired) {
                const int row = tile * kTileRows + unit;
                const bool live = active && row < args.rows_total;  // (the number of rows is a multiple of 8: four rows are all inside or all outside)
                float4 value = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (live) value = sum_parts(unit, col);
                value.x *= scale; value.y *= scale; value.z *= scale; value.w *= scale;
                const size_t at = (size_t)col * args.ld_out + row;
                if (live && EPI == EPI_BF16)
                    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(args.out) + at) = make_uint2(pack_bf16(value.x, value.y), pack_bf16(value.z, value.w));
                if (live && EPI == EPI_F32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(args.out) + at) = value;
                if (EPI == EPI_RESIDUAL) {  // this thread alone owns the elements
                    float squares = 0.0f;
                    if (live) {
                        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(args.out) + at);
                        const float4 before = base == 0 ? early_before : *dst;
                        const float4 x = make_float4(before.x + value.x, before.y + value.y, before.z + value.z, before.w + value.w);
                        *dst = x;
                        if (args.emit_gain) {
                            const float4 g = base == 0 ? early_gain : *reinterpret_cast<const float4*>(args.emit_gain + row);
                            *reinterpret_cast<uint2*>(args.emit_rows + (size_t)col * args.ld_emit + row) =
                                make_uint2(pack_bf16(x.x * g.x, x.y * g.y), pack_bf16(x.z * g.z, x.w * g.w));
                            squares = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
                        }
                    }
                    if (args.emit_gain) {
                        // the `quads` neighbouring threads of one batch row add their squares (a fixed tree); their first writes the part
                        for (int offset = quads >> 1; offset > 0; offset >>= 1) squares += __shfl_down_sync(0xffffffffu, squares, offset);
                        if (active && (item & (quads - 1)) == 0) args.emit_ssq[(size_t)(tile * splits + rank) * 128 + col] = squares;
                    }
                }
            } else if (EPI == EPI_SWIGLU) {
                const int row = tile * 64 + unit;
                if (!active || row >= args.rows_total) continue;
                float4 gate = sum_parts(unit, col), up = sum_parts(unit + 64, col);
                gate.x *= scale; gate.y *= scale; gate.z *= scale; gate.w *= scale;
                up.x *= scale; up.y *= scale; up.z *= scale; up.w *= scale;
                const int a = args.activation;
                *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(args.out) + (size_t)col * args.ld_out + row) =
                    make_uint2(pack_bf16(gate_activation(a, gate.x) * up.x, gate_activation(a, gate.y) * up.y),
                               pack_bf16(gate_activation(a, gate.z) * up.z, gate_activation(a, gate.w) * up.w));
            } else {  // EPI_ROPE: pairs `unit`.. of the tile are coordinates d and d + head/2 of one of its heads
                const int hd = args.head_dim, half = hd / 2;
                const int head_in_tile = unit / half, d0 = unit % half;
                const int head = tile * (kTileRows / hd) + head_in_tile;
                if (!active || head >= args.heads + 2 * args.kv_heads) continue;
                const int mma_row = head_in_tile * hd + d0;
                const float4 first_half = sum_parts(mma_row, col), second_half = sum_parts(mma_row + half, col);
                // queries and keys pass through bfloat16 before the rotation, as they do when a product stores them
                float x0[4] = {first_half.x * scale, first_half.y * scale, first_half.z * scale, first_half.w * scale};
                float x1[4] = {second_half.x * scale, second_half.y * scale, second_half.z * scale, second_half.w * scale};
                if (head < args.heads + args.kv_heads) {
                    const bool early = kEarlyForAll && base == 0;
                    const size_t at_table = early ? 0 : (size_t)args.positions[col] * half + d0;
                    const float4 c4 = early ? early_before : *reinterpret_cast<const float4*>(args.cos_table + at_table);
                    const float4 s4 = early ? early_gain : *reinterpret_cast<const float4*>(args.sin_table + at_table);
                    const float c[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float a0 = __bfloat162float(__float2bfloat16_rn(x0[i])), a1 = __bfloat162float(__float2bfloat16_rn(x1[i]));
                        x0[i] = a0 * c[i] - a1 * sn[i];
                        x1[i] = a0 * sn[i] + a1 * c[i];
                    }
                }
                bf16* dst = nullptr;
                if (head < args.heads) {
                    dst = reinterpret_cast<bf16*>(args.out) + (size_t)col * args.ld_out + (size_t)head * hd;
                } else {
                    const int slot = (kEarlyForAll && base == 0) ? early_slot : args.slot_mapping[col];
                    if (slot >= 0) {
                        const bool is_key = head < args.heads + args.kv_heads;
                        const int kv_head = head - args.heads - (is_key ? 0 : args.kv_heads);
                        const size_t page = slot / args.page_size, offset = slot % args.page_size;
                        dst = (is_key ? args.k_pool : args.v_pool) + ((page * args.kv_heads + kv_head) * args.page_size + offset) * hd;
                    }
                }
                if (dst) {
                    *reinterpret_cast<uint2*>(dst + d0) = make_uint2(pack_bf16(x0[0], x0[1]), pack_bf16(x0[2], x0[3]));
                    *reinterpret_cast<uint2*>(dst + d0 + half) = make_uint2(pack_bf16(x1[0], x1[1]), pack_bf16(x1[2], x1[3]));
                }
            }
        }
    }

    // a cluster's blocks leave together: each has read the others' shared memory until now
    if (splits > 1) cluster_leave_together();
    else __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Plan::kTmemColumns));
    }
}

template <int EPI, int kBatchN, int kStageCount>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const WideArgs& args, int tiles, cudaStream_t stream) {
    using Plan = WidePlan<kBatchN, kStageCount>;
    const size_t smem = (size_t)Plan::kStages * Plan::kStageBytes + 1024;
    auto kernel = wide_gemm_kernel<EPI, kBatchN, kStageCount>;
    static bool configured[64] = {false};  // the attribute is a device's
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return fail("wide_gemm: cannot tell the current device");
    if (!configured[device]) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("wide_gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
        configured[device] = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(tiles * args.splits);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = args.splits;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent_launches_allowed() ? 2 : 1;
    cudaError_t status = cudaLaunchKernelEx(&config, kernel, map_w, map_x, args);
    if (status != cudaSuccess) return fail("wide_gemm: launch failed: %s", cudaGetErrorString(status));
    return check_launch("wide_gemm");
}

// How many blocks share a tile's K: as many (1, 2, 4 or 8: a cluster) as it takes for every multiprocessor to have a
// block, while a block keeps at least four 64-column steps of K (eight were measured too: a little slower).
static void plan(int tiles, int k, int multiprocessors, int* splits, int* per_split) {
    const int k_blocks = (k + kBlockK - 1) / kBlockK;
    int s = 1;
    while (s < 8 && tiles * s * 2 <= multiprocessors + multiprocessors / 4 && k_blocks / (s * 2) >= 4) s *= 2;
    // Blocks of a cluster run with the four-stage ring, two to a multiprocessor: while there is at most one for each,
    // half of what could be in flight is not, so K is split once more where a block still keeps eight steps (the down
    // products of the 3B and 8B layer shapes: +5 % and +2 % tokens a second at batch 16 and 64).  A matrix with a tile
    // per multiprocessor is not split at all: its blocks run alone with the eight-stage ring.
    if (s > 1 && s < 8 && tiles * s <= multiprocessors && k_blocks / (s * 2) >= 8) s *= 2;
    *per_split = (k_blocks + s - 1) / s;
    while (s > 1 && (s - 1) * *per_split >= k_blocks) {  // no part may be empty: fewer, as a power of two
        s /= 2;
        *per_split = (k_blocks + s - 1) / s;
    }
    *splits = s;
}

template <int EPI>
static int launch_n(const CUtensorMap& map_w, const void* x, int ldx, const WideArgs& args, int tiles, int multiprocessors,
                    cudaStream_t stream) {
    const int batch_n = args.batch <= 32 ? 32 : (args.batch <= 64 ? 64 : 128);
    CUtensorMap map_x;
    if (int status = make_map(&map_x, x, args.batch, args.k, ldx, batch_n)) return status;
    // a block per multiprocessor at most, and no cluster (a cluster of eight blocks that each fill a multiprocessor
    // finds room for only some of the clusters at a time): the deeper ring
    const bool deep = args.splits == 1 && tiles <= multiprocessors;
    // (up to 32 rows a stage is 20 KB: five of them leave room for a block of the kernel before or after on the same
    // multiprocessor, which was measured to count for more than a deeper ring: +1.4 % tokens a second at batch 16)
    if (batch_n == 32) return deep ? launch<EPI, 32, 5>(map_w, map_x, args, tiles, stream) : launch<EPI, 32, 4>(map_w, map_x, args, tiles, stream);
    if (batch_n == 64) return deep ? launch<EPI, 64, 8>(map_w, map_x, args, tiles, stream) : launch<EPI, 64, 4>(map_w, map_x, args, tiles, stream);
    return deep ? launch<EPI, 128, 8>(map_w, map_x, args, tiles, stream) : launch<EPI, 128, 4>(map_w, map_x, args, tiles, stream);
}

static int check_operands(const char* what, const void* x, int ldx, const void* w, int ldw, int batch, int k) {
    if (batch > 128) return fail("%s: takes at most 128 activation rows, got %d", what, batch);
    if (k <= 0 || k % 8 || ldx % 8 || ldw % 8) return fail("%s: k (%d) and the row strides (%d, %d) must be multiples of 8", what, k, ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail("%s: operands must start on 16-byte boundaries", what);
    return 0;
}

}  // namespace mb

using namespace mb;

// x: bfloat16 [batch, k] (up to 128 rows); w: bfloat16 [n_w, k].
// epilogue 0: out bfloat16 [batch, n_w]; 1: float32; 2: float32 += ; 3: w = [gate rows; up rows], out
// bfloat16 [batch, n_w/2] = act(gate) * up, the activation code (MB_ACT_*) in bits 8 and up of `epilogue`.
// ssq_parts (or null): [ssq_count][128] parts of the sums of squares of the rows that x is the gained copy of; the
// results are then scaled by 1 / sqrt(sum / norm_width + eps).  emit_gain (or null, epilogue 2 only): the next norm's
// gain; the new x times it goes to emit_rows (bfloat16, row stride ld_emit), the blocks' parts of the new rows' sums of
// squares to emit_ssq [parts][128], and *parts_written says how many parts there are.
MB_EXPORT int mb_wide_gemm(const void* x, int ldx, const void* w, int ldw, void* out, int ld_out, int batch, int n_w, int k,
                           int epilogue, int multiprocessors, const float* ssq_parts, int ssq_count, int norm_width, float eps,
                           const float* emit_gain, void* emit_rows, int ld_emit, float* emit_ssq, int* parts_written,
                           cudaStream_t stream) {
    if (batch <= 0 || n_w <= 0) return 0;
    const int activation = epilogue >> 8;
    epilogue &= 0xff;
    if (activation < 0 || activation >= MB_ACT_COUNT) return fail("wide_gemm: unknown gate activation code %d", activation);
    if (int status = check_operands("wide_gemm", x, ldx, w, ldw, batch, k)) return status;
    if (epilogue == EPI_SWIGLU && n_w % 2) return fail("wide_gemm: the gated epilogue needs an even number of weight rows, got %d", n_w);
    WideArgs args{};
    args.rows_total = epilogue == EPI_SWIGLU ? n_w / 2 : n_w;
    args.up_row_offset = args.rows_total;
    args.activation = activation;
    args.batch = batch;
    args.k = k;
    args.out = out;
    args.ld_out = ld_out;
    const int tiles = epilogue == EPI_SWIGLU ? (args.rows_total + 63) / 64 : (args.rows_total + kTileRows - 1) / kTileRows;
    plan(tiles, k, multiprocessors, &args.splits, &args.k_blocks_per_split);
    args.ssq_parts = ssq_parts; args.ssq_count = ssq_count; args.norm_width = norm_width; args.eps = eps;
    if (emit_gain) {
        if (epilogue != EPI_RESIDUAL || !emit_rows || !emit_ssq || ld_emit % 4 || ((uintptr_t)emit_gain & 15) || ((uintptr_t)emit_rows & 7))
            return fail("wide_gemm: the next norm's rows are written by the residual epilogue, into aligned buffers");
        args.emit_gain = emit_gain; args.emit_rows = (bf16*)emit_rows; args.ld_emit = ld_emit; args.emit_ssq = emit_ssq;
    }
    if (parts_written) *parts_written = tiles * args.splits;
    CUtensorMap map_w;
    // (the gated tile is two boxes of 64 rows; rows past the matrix are zeros and their results are not stored)
    if (int status = make_map(&map_w, w, n_w, k, ldw, epilogue == EPI_SWIGLU ? 64 : kTileRows)) return status;
    switch (epilogue) {
        case EPI_BF16: return launch_n<EPI_BF16>(map_w, x, ldx, args, tiles, multiprocessors, stream);
        case EPI_F32: return launch_n<EPI_F32>(map_w, x, ldx, args, tiles, multiprocessors, stream);
        case EPI_RESIDUAL: return launch_n<EPI_RESIDUAL>(map_w, x, ldx, args, tiles, multiprocessors, stream);
        case EPI_SWIGLU: return launch_n<EPI_SWIGLU>(map_w, x, ldx, args, tiles, multiprocessors, stream);
    }
    return fail("wide_gemm: unknown epilogue %d", epilogue);
}

// The q/k/v product of an attention layer on up to 128 rows with what follows it folded in: rotation of queries and
// keys (split-half pairs over the whole head) and the paged cache write of keys and values.  w: bfloat16 [(heads + 2 *
// kv_heads) * head_dim, k]; head_dim divides 128; q_out: bfloat16 [batch, heads * head_dim] (row stride ld_q).
MB_EXPORT int mb_wide_qkv_rope(const void* x, int ldx, const void* w, int ldw, void* q_out, int ld_q, int batch, int k, int heads,
                               int kv_heads, int head_dim, const int* positions, const float* cos_table, const float* sin_table,
                               void* k_pool, void* v_pool, const int* slot_mapping, int page_size, int multiprocessors,
                               const float* ssq_parts, int ssq_count, int norm_width, float eps, cudaStream_t stream) {
    if (batch <= 0) return 0;
    if (head_dim < 16 || kTileRows % head_dim) return fail("wide_qkv_rope: the head size must divide 128, got %d", head_dim);
    if (!positions || !cos_table || !sin_table || !k_pool || !v_pool || !slot_mapping || page_size <= 0)
        return fail("wide_qkv_rope: needs positions, cos/sin tables, cache pools, a slot mapping and a page size");
    if (int status = check_operands("wide_qkv_rope", x, ldx, w, ldw, batch, k)) return status;
    WideArgs args{};
    args.rows_total = (heads + 2 * kv_heads) * head_dim;
    args.batch = batch;
    args.k = k;
    args.out = q_out;
    args.ld_out = ld_q;
    args.heads = heads; args.kv_heads = kv_heads; args.head_dim = head_dim; args.page_size = page_size;
    args.positions = positions; args.slot_mapping = slot_mapping; args.cos_table = cos_table; args.sin_table = sin_table;
    args.k_pool = (bf16*)k_pool; args.v_pool = (bf16*)v_pool;
    args.ssq_parts = ssq_parts; args.ssq_count = ssq_count; args.norm_width = norm_width; args.eps = eps;
    const int tiles = (args.rows_total + kTileRows - 1) / kTileRows;
    plan(tiles, k, multiprocessors, &args.splits, &args.k_blocks_per_split);
    CUtensorMap map_w;
    if (int status = make_map(&map_w, w, args.rows_total, k, ldw, kTileRows)) return status;
    return launch_n<EPI_ROPE>(map_w, x, ldx, args, tiles, multiprocessors, stream);
}

MB_EXPORT int mb_wide_gemm_status() {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    return status;
}
