// Decode matrix products for wide batches (33 to 128 activation rows) on the tcgen05 tensor cores.
//
// With this many rows the weights still have to stream exactly once, but the arithmetic no longer
// fits the register-fed MMAs of the narrow decode kernel.  So the operands swap sides: a tile of 128
// WEIGHT rows is the 128-row operand of tcgen05.mma and the activations are the N = 64 or 128 side;
// both travel by TMA (the activations, a few hundred KB, are re-read from L2 for every weight tile)
// and the accumulator [128 weight rows x batch] lives in tensor memory.
//
//   * Work units are (weight row tile, K split).  Matrices with few row tiles split K so that every
//     multiprocessor streams; blocks are persistent and walk the units round-robin, the TMA ring runs
//     on across units.
//   * Split K without waiting: every split stores its partial accumulator to scratch memory and takes
//     a ticket (atomic counter per row tile and warp quarter); the split that draws the last ticket
//     adds all partials in split order -- the same order whoever comes last -- and runs the epilogue.
//     Nobody waits for anybody, and the counter is back at zero when the tile is done.
//   * Epilogues as in the other product kernels: store bf16 / f32, add into the float32 residual
//     stream, or silu(gate) * up when the unit carries a gate tile and its up tile (two accumulators).
//     The accumulator is transposed with respect to the output ([weight row][batch row]); a warp's 32
//     lanes hold 32 neighbouring output columns of one batch row, so stores stay coalesced.
//
// Every mbarrier wait is bounded as in gemm_tcgen05.cu; mb_wide_gemm_status() reads the record.
#include "tcgen05.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3 };

constexpr int kTileRows = 128;                    // weight rows per tile (UMMA M)
constexpr int kTileBytes = kTileRows * kBlockK * 2;
constexpr int kThreads = 192;                     // warp 0: TMA, warp 1: MMA, warps 2..5: epilogue

struct WideArgs {
    int rows_total;       // output columns = weight rows (for EPI_SWIGLU: gate rows)
    int up_row_offset;    // EPI_SWIGLU: first up row of W
    int activation;       // EPI_SWIGLU: the gate's activation (MB_ACT_*)
    int batch, k;
    int tiles, splits, k_blocks_per_split;
    void* out;            // [batch, rows_total] bfloat16 / float32 (row stride ld_out)
    int ld_out;
    float* partial;       // splits > 1: [tile][split][accumulators][batch columns][128 rows] floats
    int* tickets;         // splits > 1: [tile][4 warp quarters], zero before the launch and after it
};

template <int EPI, int kBatchN>
struct WidePlan {
    static constexpr int kAccumulators = EPI == EPI_SWIGLU ? 2 : 1;   // gate and up
    static constexpr int kStageBytes = kAccumulators * kTileBytes + kBatchN * kBlockK * 2;
    static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
    static constexpr int kUnitColumns = kAccumulators * kBatchN;        // tensor-memory columns per unit
    static constexpr int kTmemColumns = 2 * kUnitColumns <= 128 ? 128 : (2 * kUnitColumns <= 256 ? 256 : 512);
    static_assert(2 * kUnitColumns <= 512, "two units of accumulators must fit tensor memory");
};

template <int EPI, int kBatchN>
__global__ void __launch_bounds__(kThreads, 1)
wide_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const WideArgs args) {
    using Plan = WidePlan<EPI, kBatchN>;
    constexpr int kStages = Plan::kStages, kAccumulators = Plan::kAccumulators;
    constexpr uint32_t kInstruction = instruction_descriptor(kTileRows, kBatchN);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t barriers[2 * kStages + 4];
    __shared__ uint32_t tmem_base_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_u32(&barriers[0]), empty_bar = smem_u32(&barriers[kStages]);
    const uint32_t acc_full_bar = smem_u32(&barriers[2 * kStages]), acc_empty_bar = smem_u32(&barriers[2 * kStages + 2]);
    const int units = args.tiles * args.splits;
    const int k_blocks = (args.k + kBlockK - 1) / kBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar + 8 * a, 1);
            mbar_init(acc_empty_bar + 8 * a, 4);
        }
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
    grid_dependency_wait();  // the activations come from the kernel before this one

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 1;
            bool ok = true;
            for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
                const int tile = unit / args.splits, split = unit % args.splits;
                const int kb_begin = split * args.k_blocks_per_split;
                const int kb_end = min(k_blocks, kb_begin + args.k_blocks_per_split);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!(ok = mbar_wait(empty_bar + 8 * stage, phase, 1))) break;
                    const uint32_t dst = smem_u32(smem) + stage * Plan::kStageBytes;
                    mbar_expect_tx(full_bar + 8 * stage, Plan::kStageBytes);
                    tma_load_2d(dst, &map_w, kb * kBlockK, tile * kTileRows, full_bar + 8 * stage);
                    if (kAccumulators == 2)
                        tma_load_2d(dst + kTileBytes, &map_w, kb * kBlockK, args.up_row_offset + tile * kTileRows, full_bar + 8 * stage);
                    tma_load_2d(dst + kAccumulators * kTileBytes, &map_x, kb * kBlockK, 0, full_bar + 8 * stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 1;
            bool ok = true;
            for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
                const int split = unit % args.splits;
                const int kb_begin = split * args.k_blocks_per_split;
                const int kb_end = min(k_blocks, kb_begin + args.k_blocks_per_split);
                if (!(ok = mbar_wait(acc_empty_bar + 8 * acc, acc_phase, 2))) break;
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * Plan::kUnitColumns;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!(ok = mbar_wait(full_bar + 8 * stage, phase, 3))) break;
                    tcgen05_fence_after();
                    const uint32_t base = smem_u32(smem) + stage * Plan::kStageBytes;
                    const uint64_t x_desc = umma_descriptor(base + kAccumulators * kTileBytes);
#pragma unroll
                    for (int a = 0; a < kAccumulators; ++a) {
                        const uint64_t w_desc = umma_descriptor(base + a * kTileBytes);
#pragma unroll
                        for (int ks = 0; ks < kBlockK / 16; ++ks)
                            umma(tmem_d + a * kBatchN, w_desc + 2 * ks, x_desc + 2 * ks, kInstruction, (kb > kb_begin || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar + 8 * stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(acc_full_bar + 8 * acc);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: 4 warps, 32 weight rows each
        const int quarter = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
            const int tile = unit / args.splits, split = unit % args.splits;
            ok = mbar_wait(acc_full_bar + 8 * acc, acc_phase, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const int row = tile * kTileRows + quarter * 32 + lane;   // output column = weight row
            const uint32_t taddr = tmem_base + acc * Plan::kUnitColumns + ((uint32_t)(quarter * 32) << 16);
            bool finish = true;  // this warp runs the epilogue of its 32 rows
            // this warp's slice of a partial: [accumulator][batch column][32 rows of this quarter]
            const size_t slice = (size_t)kAccumulators * kBatchN * 32;
            float* partial = args.partial + ((size_t)(tile * args.splits) * 4 + quarter) * slice;  // split 0; split s: + s * 4 * slice
            if (args.splits > 1) {
                float* mine = partial + (size_t)split * 4 * slice;
#pragma unroll 1
                for (int c = 0; c < kAccumulators * kBatchN; c += 32) {
                    float v[32];
                    tmem_load_32(taddr + c, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) mine[(size_t)(c + i) * 32 + lane] = v[i];
                }
                __threadfence();
                __syncwarp();
                int ticket = 0;
                if (lane == 0) ticket = atomicAdd(args.tickets + tile * 4 + quarter, 1);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                finish = ticket == args.splits - 1;
                if (finish) {
                    __threadfence();
                    if (lane == 0) args.tickets[tile * 4 + quarter] = 0;  // ready for the next launch
                }
            }
            // the accumulator has been read (or will not be needed): hand it back early
            if (args.splits > 1) {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar + 8 * acc);
            }
            if (finish) {
#pragma unroll 1
                for (int c = 0; c < kBatchN; c += 32) {
                    float v[32], u[32];
                    if (args.splits > 1) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = u[i] = 0.0f;
                        for (int s = 0; s < args.splits; ++s) {  // split order, whoever finishes
                            const float* from = partial + (size_t)s * 4 * slice;
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                v[i] += __ldcg(from + (size_t)(c + i) * 32 + lane);
                                if (kAccumulators == 2) u[i] += __ldcg(from + (size_t)(kBatchN + c + i) * 32 + lane);
                            }
                        }
                    } else {
                        tmem_load_32(taddr + c, v);
                        if (kAccumulators == 2) tmem_load_32(taddr + kBatchN + c, u);
                    }
                    if (row < args.rows_total) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int b = c + i;
                            if (b >= args.batch) break;
                            float value = v[i];
                            if (EPI == EPI_SWIGLU) value = gate_activation(args.activation, value) * u[i];
                            const size_t at = (size_t)b * args.ld_out + row;
                            if (EPI == EPI_BF16 || EPI == EPI_SWIGLU) reinterpret_cast<bf16*>(args.out)[at] = __float2bfloat16_rn(value);
                            if (EPI == EPI_F32) reinterpret_cast<float*>(args.out)[at] = value;
                            if (EPI == EPI_RESIDUAL) reinterpret_cast<float*>(args.out)[at] += value;
                        }
                    }
                }
            }
            if (args.splits == 1) {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar + 8 * acc);
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Plan::kTmemColumns));
    }
}

template <int EPI, int kBatchN>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const WideArgs& args, int grid, cudaStream_t stream) {
    using Plan = WidePlan<EPI, kBatchN>;
    const size_t smem = (size_t)Plan::kStages * Plan::kStageBytes + 1024;
    auto kernel = wide_gemm_kernel<EPI, kBatchN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("wide_gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
        configured = true;
    }
    return launch_dependent("wide_gemm", kernel, dim3(grid), dim3(kThreads), smem, stream, true, map_w, map_x, args);
}

static void plan(int rows_total, int k, int multiprocessors, int* tiles, int* splits, int* per_split) {
    const int k_blocks = (k + kBlockK - 1) / kBlockK;
    *tiles = (rows_total + kTileRows - 1) / kTileRows;
    int s = 1;
    // split K until every multiprocessor has a unit, keeping at least four stages of K per unit
    while (s < 16 && *tiles * s < multiprocessors && k_blocks / (s * 2) >= 4) s *= 2;
    *per_split = (k_blocks + s - 1) / s;
    *splits = (k_blocks + *per_split - 1) / *per_split;
}

}  // namespace mb

using namespace mb;

// Scratch a call needs: floats of partial accumulators and ints of tickets (both 0 when K is not split).
// The tickets must be zero before the first launch that uses them; every launch leaves them zero.
MB_EXPORT void mb_wide_gemm_scratch(int n_w, int k, int batch, int epilogue, int multiprocessors, size_t* partial_floats,
                                    size_t* ticket_ints) {
    epilogue &= 0xff;
    const int rows_total = epilogue == EPI_SWIGLU ? n_w / 2 : n_w;
    int tiles, splits, per_split;
    plan(rows_total, k, multiprocessors, &tiles, &splits, &per_split);
    const int batch_n = batch <= 64 ? 64 : 128;
    const int accumulators = epilogue == EPI_SWIGLU ? 2 : 1;
    *partial_floats = splits > 1 ? (size_t)tiles * splits * accumulators * batch_n * kTileRows : 0;
    *ticket_ints = splits > 1 ? (size_t)tiles * 4 : 0;
}

// x: bfloat16 [batch, k] (33..128 rows pay off; 1..128 are taken); w: bfloat16 [n_w, k].
// epilogue 0: out bfloat16 [batch, n_w]; 1: float32; 2: float32 += ; 3: w = [gate rows; up rows], out
// bfloat16 [batch, n_w/2] = act(gate) * up, the activation code (MB_ACT_*) in bits 8 and up of `epilogue`.
MB_EXPORT int mb_wide_gemm(const void* x, int ldx, const void* w, int ldw, void* out, int ld_out, int batch, int n_w, int k,
                           int epilogue, float* partial, int* tickets, int multiprocessors, cudaStream_t stream) {
    if (batch <= 0 || n_w <= 0) return 0;
    const int activation = epilogue >> 8;
    epilogue &= 0xff;
    if (activation < 0 || activation >= MB_ACT_COUNT) return fail("wide_gemm: unknown gate activation code %d", activation);
    if (batch > 128) return fail("wide_gemm: takes at most 128 activation rows, got %d", batch);
    if (k <= 0 || k % 8 || ldx % 8 || ldw % 8) return fail("wide_gemm: k (%d) and the row strides (%d, %d) must be multiples of 8", k, ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail("wide_gemm: operands must start on 16-byte boundaries");
    if (epilogue == EPI_SWIGLU && (n_w % 2 || (n_w / 2) % 8)) return fail("wide_gemm: the gated epilogue needs gate and up halves that are multiples of 8 rows, got %d rows", n_w);
    WideArgs args{};
    args.rows_total = epilogue == EPI_SWIGLU ? n_w / 2 : n_w;
    args.up_row_offset = args.rows_total;
    args.activation = activation;
    args.batch = batch;
    args.k = k;
    plan(args.rows_total, k, multiprocessors, &args.tiles, &args.splits, &args.k_blocks_per_split);
    if (args.splits > 1 && (!partial || !tickets)) return fail("wide_gemm: %d splits of K need scratch memory", args.splits);
    args.out = out;
    args.ld_out = ld_out;
    args.partial = partial;
    args.tickets = tickets;
    const int batch_n = batch <= 64 ? 64 : 128;
    CUtensorMap map_w, map_x;
    if (int status = make_map(&map_w, w, n_w, k, ldw, kTileRows)) return status;
    if (int status = make_map(&map_x, x, batch, k, ldx, batch_n)) return status;
    const int units = args.tiles * args.splits;
    const int grid = units < multiprocessors ? units : multiprocessors;
#define MB_WIDE(EPI) \
    if (epilogue == EPI) return batch_n == 64 ? launch<EPI, 64>(map_w, map_x, args, grid, stream) : launch<EPI, 128>(map_w, map_x, args, grid, stream);
    MB_WIDE(EPI_BF16)
    MB_WIDE(EPI_F32)
    MB_WIDE(EPI_RESIDUAL)
    MB_WIDE(EPI_SWIGLU)
#undef MB_WIDE
    return fail("wide_gemm: unknown epilogue %d", epilogue);
}

MB_EXPORT int mb_wide_gemm_status() {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    return status;
}
