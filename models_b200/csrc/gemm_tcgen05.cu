// Prefill matrix products on the fifth-generation tensor cores: C[M, N] = A[M, K] . W[N, K]^T with
// bfloat16 operands and float accumulation, for many activation rows (a whole prompt).
//
//   * Operand tiles travel by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a ring of shared
//     memory: 128 rows of A and 256 (or 128) rows of W, 64 columns of K per stage, four (six) stages.
//   * One thread issues tcgen05.mma (M = 128, N = 256 or 128, K = 16, operands from shared-memory
//     descriptors); the accumulator lives in tensor memory, double-buffered, so the epilogue of one
//     tile overlaps the products of the next.
//   * Eight epilogue warps (two per quarter of the tensor-memory lanes, half the columns each) read
//     the accumulator back with tcgen05.ld and finish the layer's arithmetic in registers: store as
//     bfloat16 / float, add into the float32 residual stream (a vector reduction at the memory side:
//     the stream is not read back), or -- when W
//     holds gate rows and up rows -- silu(gate) * up, so the gated activation never passes through
//     memory.  (x = x + W.h: integrallis/models, backend-java/.../llama/LlamaForwardPass.java:1131-1138,
//     1172-1178; SwiGLU: backend-java/.../ops/TensorOps.java:1407-1425.)
//   * Blocks are persistent (one per multiprocessor) and walk the output tiles with the row tile
//     index running fastest inside groups of 2,048 rows, so neighbouring blocks share a weight tile
//     through L2 and a group of activation rows stays there while the weights stream past.
//   * Where there are tiles enough, two blocks of a cluster share a tile of 256 rows by 256 columns
//     (tcgen05 cta_group::2): each loads its own 128 rows of A and its half of W (plain TMA loads, no
//     multicast; both blocks' bytes are counted on the leader's barrier), the leader issues products
//     that read both blocks' shared memory, tcgen05.commit tells both blocks' barriers, and each block
//     runs the epilogue of its rows from its own tensor memory.
//
// Every wait on an mbarrier is bounded: after about two seconds a role gives up, records where in
// g_gemm_status and leaves its loop; all roles then meet at the final barrier, tensor memory is
// freed and the kernel returns.  mb_gemm_tc_status() reads the record.
#include <algorithm>

#include "tcgen05.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3, EPI_ROPE = 4 };

constexpr int kBlockM = 128;
constexpr int kTileABytes = kBlockM * kBlockK * 2;      // 16 KB
constexpr int kBoxBBytes = 128 * kBlockK * 2;           // 16 KB: 128 rows of W; one or two boxes per stage
constexpr int kRingBytes = 192 * 1024;
// A tile is 128 rows by BN columns, BN = 256 (two boxes of W per stage, four stages) or 128 (one box,
// six stages).  The narrow tile moves more bytes per product, but twice as many tiles spread a small
// or oddly sized matrix more evenly over the multiprocessors.
template <int BN>
struct Tile {
    static_assert(BN == 128 || BN == 256, "tile widths built: 128 and 256");
    static constexpr int kBoxes = BN / 128;
    static constexpr int kStageBytes = kTileABytes + kBoxes * kBoxBBytes;
    static constexpr int kStages = kRingBytes / kStageBytes;
    static constexpr uint32_t kInstruction = instruction_descriptor(kBlockM, BN);
};
constexpr int kMaxStages = 6;
constexpr int kEpilogueWarps = 8;                       // two per quarter of the tensor-memory lanes: each takes half the columns
constexpr int kThreads = 64 + 32 * kEpilogueWarps;      // warp 0: TMA, warp 1: MMA, warps 2..9: epilogue
constexpr int kTmemColumns = 512;  // two accumulators of BN columns; all of it is taken either way

// An epilogue warp's staging tile: 32 rows of 128 bytes.  A thread holds one row of the accumulator (a tensor-memory
// lane), and storing from there would touch 32 lines per instruction; through the staging tile the rows are turned so
// that neighbouring threads hold neighbouring bytes of a row and every store covers whole lines.  The 16-byte units
// of a row are permuted by the row (unit ^ row % 8): the eight threads of a quarter-warp, which write the same unit of
// eight rows or read eight units of one row, then fall on different banks.
constexpr int kStagingBytes = 32 * 128;
__device__ __forceinline__ uint32_t staged_address(uint32_t staging, int row, int unit) {
    return staging + row * 128 + ((unit ^ (row & 7)) << 4);
}
__device__ __forceinline__ void stage_row(uint32_t staging, int row, const uint32_t (&packed)[32]) {
    __syncwarp();  // the pass before has been read
#pragma unroll
    for (int unit = 0; unit < 8; ++unit)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(staged_address(staging, row, unit)), "r"(packed[4 * unit]),
                     "r"(packed[4 * unit + 1]), "r"(packed[4 * unit + 2]), "r"(packed[4 * unit + 3])
                     : "memory");
    __syncwarp();
}
__device__ __forceinline__ uint4 staged_unit(uint32_t staging, int row, int unit) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(staged_address(staging, row, unit)) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&pair);
}
__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// The order in which tiles are walked: row tiles run fastest inside a group of kGroupRows rows of A, then the column
// tiles of W, then the next group.  Blocks that work at the same time then share a few tiles of W and one group of A,
// which stays in L2 while all of W streams past it once; with row tiles simply running fastest, a prompt of 16,384
// tokens re-read all of A (more than L2 holds) for every column tile.
constexpr int kGroupRows = 2048;
__device__ __forceinline__ void tile_coordinates(int tile, int m_tiles, int n_tiles, int group, int* m_tile, int* n_tile) {
    const int per_group = group * n_tiles;
    const int full_groups = m_tiles / group;
    const int g = tile / per_group;
    if (g < full_groups) {
        const int within = tile - g * per_group;
        *m_tile = g * group + within % group;
        *n_tile = within / group;
    } else {  // the last, smaller group
        const int rest = m_tiles - full_groups * group;
        const int within = tile - full_groups * per_group;
        *m_tile = full_groups * group + within % rest;
        *n_tile = within / rest;
    }
}

struct GemmArgs {
    int m, n, k;          // n: output columns (for EPI_SWIGLU the gate count, half the weight rows)
    int up_row_offset;    // EPI_SWIGLU: first up row of W
    int activation;       // EPI_SWIGLU: the gate's activation (MB_ACT_*)
    int k_splits;         // EPI_RESIDUAL: blocks that share an output tile, each with its own part of K (else 1)
    int cluster_sum;      // k_splits > 1 on single blocks: the parts' blocks are one thread-block cluster and their sums meet
                          // in distributed shared memory (no scratch, no tickets)
    float* partial;       // k_splits > 1: [tile][block of a pair][part of K][128 rows][tile columns] floats, or null
    int* tickets;         // k_splits > 1 with `partial`: [tile][block of a pair][8 epilogue warps][arrived, finished], zero before and after a launch
    void* out;            // bfloat16 [m, n], float [m, n], or the float residual stream; EPI_ROPE: the queries [m, heads * head_dim]
    int ld_out;
    // EPI_ROPE: W is [q heads; k heads; v heads]
    int heads, kv_heads, head_dim, page_size;
    const int* positions;     // [m]
    const int* slot_mapping;  // [m] flat cache position, < 0: do not store
    const float* cos_table;   // [positions][head_dim / 2]
    const float* sin_table;
    bf16* k_pool;             // [pages][kv_heads][page_size][head_dim]
    bf16* v_pool;
};

// kPair 1: a block works on a tile alone.  kPair 2: the two blocks of a cluster share a tile of 256 rows by BN columns
// (tcgen05 cta_group::2): each loads its 128 rows of A and its half of the BN rows of W, the leader issues the products
// for both, each block's tensor memory holds the accumulator of its own 128 rows, and each block runs the epilogue of
// its rows.  A block then moves 32 KB per 64 columns of K instead of 48 KB for the same work.
// Four floats at the same place of the shared memory of block `rank` of this cluster (distributed shared memory).
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
// Where 16-byte piece `piece` of row `row` of a block's partial tile [128 rows][BN floats] lies: the pieces of a row are
// permuted by the row's low bits, so that threads that hold a row each (and write the same piece of neighbouring rows at
// once) do not meet in a bank.
__device__ __forceinline__ uint32_t partial_piece(int row, int piece, int bn) { return (uint32_t)(row * bn * 4 + ((piece ^ (row & 7)) << 4)); }

template <int EPI, int BN, int kPair>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const GemmArgs args) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment of the tiles is what the swizzle and the descriptors assume
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int kBoxes = Tile<BN>::kBoxes / kPair;  // boxes of W this block loads per stage
    constexpr int kStageBytes = kTileABytes + kBoxes * kBoxBBytes, kStages = kRingBytes / kStageBytes, kAccumulatorColumns = BN;
    constexpr uint32_t kInstruction = instruction_descriptor(kBlockM * kPair, BN);
    static_assert(EPI != EPI_SWIGLU || BN == 256, "the gated epilogue pairs 128 gate columns with 128 up columns");
    static_assert(kPair == 1 || (kPair == 2 && BN == 256), "a pair of blocks shares a tile of 256 columns");
    static_assert(kStages <= kMaxStages, "ring deeper than its barriers");
    const int rank = kPair == 2 ? (int)cluster_rank() : 0;
    const bool leader = rank == 0;
    __shared__ __align__(8) uint64_t barriers[2 * kMaxStages + 4];
    __shared__ uint32_t tmem_base_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_u32(&barriers[0]), empty_bar = smem_u32(&barriers[kMaxStages]);
    const uint32_t acc_full_bar = smem_u32(&barriers[2 * kMaxStages]), acc_empty_bar = smem_u32(&barriers[2 * kMaxStages + 2]);

    // columns of output per tile: BN, or 128 gate/up pairs
    constexpr int kOutCols = EPI == EPI_SWIGLU ? 128 : BN;
    const int m_tiles = (args.m + kBlockM * kPair - 1) / (kBlockM * kPair);
    const int n_tiles = (args.n + kOutCols - 1) / kOutCols;
    // A work item is an output tile, or with k_splits > 1 one of the parts of K of an output tile: the parts' sums meet
    // in the residual stream, each added there by its own block.
    const int k_splits = EPI == EPI_RESIDUAL ? args.k_splits : 1;
    const int tiles = m_tiles * n_tiles * k_splits;
    const int k_blocks_all = (args.k + kBlockK - 1) / kBlockK;
    const int k_blocks_per_split = (k_blocks_all + k_splits - 1) / k_splits;  // the launcher leaves no part empty
    const int first_tile = blockIdx.x / kPair, tile_step = gridDim.x / kPair;  // a pair walks the tiles together

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar + 8 * a, 1);
            mbar_init(acc_empty_bar + 8 * a, kEpilogueWarps * kPair);  // the leader's copy hears from both blocks' epilogues
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // one warp allocates all 512 columns of tensor memory (of a pair: the same warp of both blocks)
        if (kPair == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemColumns));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemColumns));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (kPair == 2) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    grid_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 1;  // the first pass over the ring finds every stage free
            bool ok = true;
            auto announce = [&](int at) {  // both blocks' bytes of a pair are counted on the leader's barrier; the leader announces them
                if (kPair == 2) {
                    if (leader) mbar_expect_tx(full_bar + 8 * at, 2 * kStageBytes);
                } else {
                    mbar_expect_tx(full_bar + 8 * at, kStageBytes);
                }
            };
            auto load_weights = [&](int at, int kb, int w_row0, int w_row1) {
                const uint32_t dst = smem_u32(smem) + at * kStageBytes + kTileABytes;
                if (kPair == 2) {
                    tma_load_2d_pair(dst, &map_w, kb * kBlockK, leader ? w_row0 : w_row1, full_bar + 8 * at);
                } else {
                    tma_load_2d(dst, &map_w, kb * kBlockK, w_row0, full_bar + 8 * at);
                    if (kBoxes == 2) tma_load_2d(dst + kBoxBBytes, &map_w, kb * kBlockK, w_row1, full_bar + 8 * at);
                }
            };
            auto load_activations = [&](int at, int kb, int m0) {
                const uint32_t dst = smem_u32(smem) + at * kStageBytes;
                if (kPair == 2) tma_load_2d_pair(dst, &map_a, kb * kBlockK, m0, full_bar + 8 * at);
                else tma_load_2d(dst, &map_a, kb * kBlockK, m0, full_bar + 8 * at);
            };
            // The weights depend on nothing: the first tile's first stages of them are asked for before this kernel waits
            // for the one before it; the activations, which that kernel wrote, after.
            int early = 0;
            if (first_tile < tiles) {
                int m_tile, n_tile;
                tile_coordinates(first_tile / k_splits, m_tiles, n_tiles, kGroupRows / (kBlockM * kPair), &m_tile, &n_tile);
                const int kb_begin = (first_tile % k_splits) * k_blocks_per_split, kb_end = min(kb_begin + k_blocks_per_split, k_blocks_all);
                const int w_row0 = EPI == EPI_SWIGLU ? n_tile * 128 : n_tile * BN;
                const int w_row1 = EPI == EPI_SWIGLU ? args.up_row_offset + n_tile * 128 : n_tile * BN + 128;
                early = min(kStages, kb_end - kb_begin);
                for (int s = 0; s < early; ++s) {
                    announce(s);
                    load_weights(s, kb_begin + s, w_row0, w_row1);
                }
                grid_dependency_wait();
                const int m0 = m_tile * kBlockM * kPair + rank * kBlockM;
                for (int s = 0; s < early; ++s) load_activations(s, kb_begin + s, m0);
                stage = early;
                if (stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
                int m_tile, n_tile;
                tile_coordinates(tile / k_splits, m_tiles, n_tiles, kGroupRows / (kBlockM * kPair), &m_tile, &n_tile);
                const int kb_begin = (tile % k_splits) * k_blocks_per_split, kb_end = min(kb_begin + k_blocks_per_split, k_blocks_all);
                const int m0 = m_tile * kBlockM * kPair + rank * kBlockM;
                const int w_row0 = EPI == EPI_SWIGLU ? n_tile * 128 : n_tile * BN;
                const int w_row1 = EPI == EPI_SWIGLU ? args.up_row_offset + n_tile * 128 : n_tile * BN + 128;
                for (int kb = kb_begin + (tile == first_tile ? early : 0); kb < kb_end; ++kb) {
                    if (!(ok = mbar_wait(empty_bar + 8 * stage, phase, 1))) break;
                    announce(stage);
                    load_activations(stage, kb, m0);
                    load_weights(stage, kb, w_row0, w_row1);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 1;  // both accumulators start free
            bool ok = true;
            for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
                if (!(ok = mbar_wait(acc_empty_bar + 8 * acc, acc_phase, 2))) break;
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * kAccumulatorColumns;
                const int kb_begin = (tile % k_splits) * k_blocks_per_split, kb_end = min(kb_begin + k_blocks_per_split, k_blocks_all);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!(ok = mbar_wait(full_bar + 8 * stage, phase, 3))) break;
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(smem) + stage * kStageBytes;
                    const uint64_t a_desc = umma_descriptor(a_addr), b_desc = umma_descriptor(a_addr + kTileABytes);
#pragma unroll
                    for (int ks = 0; ks < kBlockK / 16; ++ks) {  // 32 bytes further along K per step: +2 in the address field
                        if (kPair == 2) umma_pair(tmem_d, a_desc + 2 * ks, b_desc + 2 * ks, kInstruction, (kb > kb_begin || ks > 0) ? 1u : 0u);
                        else umma(tmem_d, a_desc + 2 * ks, b_desc + 2 * ks, kInstruction, (kb > kb_begin || ks > 0) ? 1u : 0u);
                    }
                    // the stage is free (in both blocks of a pair) once these products have read it
                    if (kPair == 2) umma_commit_pair(empty_bar + 8 * stage);
                    else umma_commit(empty_bar + 8 * stage);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                // the accumulator (each block's half of it) is complete once all products are
                if (kPair == 2) umma_commit_pair(acc_full_bar + 8 * acc);
                else umma_commit(acc_full_bar + 8 * acc);
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: 8 warps; a warp reads one quarter of
        // the tensor-memory lanes (its index modulo 4) and half of the tile's columns
        grid_dependency_wait();  // what the epilogues read and add into comes from the kernels before this one
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const uint32_t staging = smem_u32(smem) + kRingBytes + (warp - 2) * kStagingBytes;
        constexpr int kHalfCols = kOutCols / 2;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
            int m_tile, n_tile;
            tile_coordinates(tile / k_splits, m_tiles, n_tiles, kGroupRows / (kBlockM * kPair), &m_tile, &n_tile);
            const int m0 = m_tile * kBlockM * kPair + rank * kBlockM;
            ok = mbar_wait(acc_full_bar + 8 * acc, acc_phase, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * kAccumulatorColumns + ((uint32_t)(quarter * 32) << 16);
            const int n0 = n_tile * kOutCols;
            // with K in parts and scratch given, the parts are summed in their order (see below)
            const int mn_tile = tile / k_splits;
            const bool ordered = EPI == EPI_RESIDUAL && k_splits > 1 && args.partial != nullptr && !args.cluster_sum;
            float* my_partial = ordered ? args.partial + ((size_t)(mn_tile * kPair + rank) * k_splits + tile % k_splits) * (kBlockM * kOutCols)
                                        : nullptr;
            if (EPI == EPI_ROPE) {
                // Whole heads lie inside this warp's half of the tile (head size 64 or 128).  Per head: the
                // coordinates d and d + head/2 are a rotation pair (x0' = x0*c - x1*s, x1' = x0*s + x1*c,
                // integrallis/models, backend-java/.../ops/TensorOps.java:1481-1486); queries go to the query
                // buffer, keys (rotated) and values (as they are) straight into the paged cache
                // (backend-java/.../llama/LlamaForwardPass.java:1070-1086).  Queries and keys pass through
                // bfloat16 before the rotation, as they do when the product stores them.
                const int hd = args.head_dim, half_head = hd / 2;
                const bool live = row < args.m;
                const int position = live ? args.positions[row] : 0;
                const int slot = live ? args.slot_mapping[row] : -1;
                for (int h0 = half * kHalfCols; h0 < (half + 1) * kHalfCols; h0 += hd) {
                    const int head = (n0 + h0) / hd;
                    if (head >= args.heads + 2 * args.kv_heads) break;
                    const bool is_query = head < args.heads, is_key = !is_query && head < args.heads + args.kv_heads;
                    bf16* dst = nullptr;
                    if (is_query) {
                        if (live) dst = reinterpret_cast<bf16*>(args.out) + (size_t)row * args.ld_out + (size_t)head * hd;
                    } else if (slot >= 0) {
                        const int kv_head = head - args.heads - (is_key ? 0 : args.kv_heads);
                        const size_t page = slot / args.page_size, offset = slot % args.page_size;
                        dst = (is_key ? args.k_pool : args.v_pool) + ((page * args.kv_heads + kv_head) * args.page_size + offset) * hd;
                    }
                    const unsigned long long dst_bits = reinterpret_cast<unsigned long long>(dst);
#pragma unroll 1
                    for (int c = 0; c < half_head; c += 32) {
                        // 32 coordinates of the lower half of the head and their partners of the upper half: a row's
                        // 128 staged bytes are [lower 32 | upper 32] in bfloat16
                        uint32_t packed[32];
                        {
                            float x0[32], x1[32];
                            tmem_load_32_issue(taddr + h0 + c, x0);
                            tmem_load_32_issue(taddr + h0 + half_head + c, x1);
                            tmem_load_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                packed[i] = pack_bf16(x0[2 * i], x0[2 * i + 1]);
                                packed[16 + i] = pack_bf16(x1[2 * i], x1[2 * i + 1]);
                            }
                        }
                        stage_row(staging, lane, packed);
                        // a quarter of a row per thread: 8 coordinates of the lower half with their 8 partners; four
                        // threads cover a row, so the tables and the destinations are read and written in whole lines
#pragma unroll
                        for (int pass = 0; pass < 4; ++pass) {
                            const int r = 8 * pass + (lane >> 2), unit = lane & 3;
                            const int r_position = __shfl_sync(0xffffffffu, position, r);
                            bf16* r_dst = reinterpret_cast<bf16*>(__shfl_sync(0xffffffffu, dst_bits, r));
                            const uint4 lo_raw = staged_unit(staging, r, unit), hi_raw = staged_unit(staging, r, 4 + unit);
                            if (r_dst == nullptr) continue;
                            float lo[8], hi[8];
                            unpack_bf16x8(lo_raw, lo);
                            unpack_bf16x8(hi_raw, hi);
                            if (is_query || is_key) {
                                float cs[8], sn[8];
                                load8(args.cos_table + (size_t)r_position * half_head + c + 8 * unit, cs);
                                load8(args.sin_table + (size_t)r_position * half_head + c + 8 * unit, sn);
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const float r0 = lo[j] * cs[j] - hi[j] * sn[j], r1 = lo[j] * sn[j] + hi[j] * cs[j];
                                    lo[j] = r0;
                                    hi[j] = r1;
                                }
                            }
                            store8(r_dst + c + 8 * unit, lo);
                            store8(r_dst + half_head + c + 8 * unit, hi);
                        }
                    }
                }
            } else {
                // 128 bytes of a row per pass: 32 columns of float, 64 of bfloat16
                constexpr bool kWide = EPI == EPI_F32 || EPI == EPI_RESIDUAL;
                constexpr int kPassCols = kWide ? 32 : 64, kUnitCols = kPassCols / 8;
#pragma unroll 1
                for (int c = half * kHalfCols; c < (half + 1) * kHalfCols; c += kPassCols) {
                    uint32_t packed[32];
                    if (kWide) {
                        float v[32];
                        tmem_load_32_issue(taddr + c, v);
                        tmem_load_wait();
                        if (EPI == EPI_RESIDUAL && kPair == 1 && args.cluster_sum) {
                            // this block's part of the sum goes to its own shared memory (the ring: every product has read
                            // it); the cluster's blocks add the parts below
                            const int tile_row = quarter * 32 + lane;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<float4*>(smem + partial_piece(tile_row, c / 4 + j, BN)) =
                                    make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                            continue;
                        }
#pragma unroll
                        for (int i = 0; i < 32; ++i) packed[i] = __float_as_uint(v[i]);
                    } else {
#pragma unroll
                        for (int part = 0; part < 2; ++part) {
                            float v[32];
                            if (EPI == EPI_SWIGLU) {
                                float u[32];
                                tmem_load_32_issue(taddr + c + 32 * part, v);
                                tmem_load_32_issue(taddr + 128 + c + 32 * part, u);
                                tmem_load_wait();
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[i] = gate_activation(args.activation, v[i]) * u[i];
                            } else {
                                tmem_load_32_issue(taddr + c + 32 * part, v);
                                tmem_load_wait();
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i) packed[16 * part + i] = pack_bf16(v[2 * i], v[2 * i + 1]);
                        }
                    }
                    stage_row(staging, lane, packed);
                    // eight threads per row and four rows per pass: every store covers whole lines of the output
                    const int col = n0 + c + (lane & 7) * kUnitCols;
#pragma unroll
                    for (int pass = 0; pass < 8; ++pass) {
                        const int r = 4 * pass + (lane >> 3);
                        const int out_row = m0 + quarter * 32 + r;
                        const uint4 value = staged_unit(staging, r, lane & 7);
                        if (out_row >= args.m || col >= args.n) continue;
                        if (kWide) {
                            float* dst = reinterpret_cast<float*>(args.out) + (size_t)out_row * args.ld_out + col;
                            const float v[4] = {__uint_as_float(value.x), __uint_as_float(value.y), __uint_as_float(value.z), __uint_as_float(value.w)};
                            if (ordered) {
                                // this part of K goes to scratch; the sum of the parts is taken below, in the order of the parts
                                *reinterpret_cast<float4*>(my_partial + (size_t)(quarter * 32 + r) * kOutCols + c + (lane & 7) * 4) =
                                    make_float4(v[0], v[1], v[2], v[3]);
                            } else if (col + 4 <= args.n) {
                                if (EPI == EPI_RESIDUAL) {
                                    // x += value without reading x here: the addition happens at the memory side.  Every
                                    // element of x gets one such addition per product (and, unordered, per part of K).
                                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3])
                                                 : "memory");
                                } else {
                                    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 4; ++i)  // (fixed indices: the values stay in registers)
                                    if (col + i < args.n) {
                                        if (EPI == EPI_RESIDUAL) atomicAdd(dst + i, v[i]);  // other parts of K add to the same element
                                        else dst[i] = v[i];
                                    }
                            }
                        } else {
                            bf16* dst = reinterpret_cast<bf16*>(args.out) + (size_t)out_row * args.ld_out + col;
                            if (col + 8 <= args.n) {
                                *reinterpret_cast<uint4*>(dst) = value;
                            } else {
                                const uint32_t w[4] = {value.x, value.y, value.z, value.w};
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    if (col + i < args.n) dst[i] = __ushort_as_bfloat16((unsigned short)(i & 1 ? w[i >> 1] >> 16 : w[i >> 1] & 0xffffu));
                            }
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (kPair == 2) mbar_arrive_leader(acc_empty_bar + 8 * acc);
                else mbar_arrive(acc_empty_bar + 8 * acc);
            }
            if (ordered) {
                // The parts of K of this warp's rows and columns lie in scratch memory once the same warp of every
                // block that shares the tile has stored its own.  Each of them then sums a share of the rows over all
                // parts, in the order of the parts -- the same additions in the same order whenever it runs -- and adds
                // the sum into the stream.  The blocks of a tile run at the same time (K is split only while all work
                // items fit one round of blocks), so the wait is short; it is bounded all the same.
                __threadfence();
                __syncwarp();
                int* arrived = args.tickets + ((size_t)(mn_tile * kPair + rank) * kEpilogueWarps + (warp - 2)) * 2;
                int* finished = arrived + 1;
                bool all_stored = true;
                if (lane == 0) {
                    atomicAdd(arrived, 1);
                    int seen = 0;
                    const long long start = clock64();
                    do {
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(arrived) : "memory");
                    } while (seen < k_splits && clock64() - start < kWaitCycles);
                    all_stored = seen >= k_splits;
                    if (!all_stored) atomicCAS(&g_gemm_status, 0, 1 + (5 << 8));  // role 5: the parts of K
                }
                all_stored = __shfl_sync(0xffffffffu, all_stored, 0);
                if (all_stored) {
                    const int split = tile % k_splits;
                    const float* parts = args.partial + (size_t)(mn_tile * kPair + rank) * k_splits * (kBlockM * kOutCols);
                    constexpr int kChunks = kHalfCols / 32;
#pragma unroll 1
                    for (int pass = split; pass < 8; pass += k_splits) {  // four rows per pass, dealt out over the parts' blocks
                        const int r = 4 * pass + (lane >> 3);
                        const int out_row = m0 + quarter * 32 + r;
                        if (out_row >= args.m) continue;
                        float4 sum[kChunks];
#pragma unroll
                        for (int ch = 0; ch < kChunks; ++ch) sum[ch] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        const float* at = parts + (size_t)(quarter * 32 + r) * kOutCols + half * kHalfCols + (lane & 7) * 4;
#pragma unroll 4
                        for (int part = 0; part < k_splits; ++part) {
#pragma unroll
                            for (int ch = 0; ch < kChunks; ++ch) {
                                if (n0 + half * kHalfCols + ch * 32 + (lane & 7) * 4 < args.n) {
                                    const float4 p = __ldcg(reinterpret_cast<const float4*>(at + (size_t)part * (kBlockM * kOutCols) + ch * 32));
                                    sum[ch].x += p.x; sum[ch].y += p.y; sum[ch].z += p.z; sum[ch].w += p.w;
                                }
                            }
                        }
#pragma unroll
                        for (int ch = 0; ch < kChunks; ++ch) {
                            const int col = n0 + half * kHalfCols + ch * 32 + (lane & 7) * 4;
                            if (col >= args.n) continue;
                            float* dst = reinterpret_cast<float*>(args.out) + (size_t)out_row * args.ld_out + col;
                            if (col + 4 <= args.n) {
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(sum[ch].x), "f"(sum[ch].y),
                                             "f"(sum[ch].z), "f"(sum[ch].w)
                                             : "memory");
                            } else {
                                const float v[4] = {sum[ch].x, sum[ch].y, sum[ch].z, sum[ch].w};
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    if (col + i < args.n) dst[i] += v[i];  // the only addition into this element
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0 && atomicAdd(finished, 1) == k_splits - 1) {  // everyone has read: as the next launch expects them
                    *arrived = 0;
                    *finished = 0;
                }
            }
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
    }

    if (EPI == EPI_RESIDUAL && kPair == 1 && args.cluster_sum) {
        // ---- the parts of K meet.  Every block of the cluster has its part of the tile in its shared memory; block r adds
        // rows r, r + k_splits, ... over all parts, in the order of the parts (the same bits in every run), and adds the
        // sums into the stream.  A block works on exactly one item here: the grid has a block per item.
        cluster_sync_all();
        if (warp >= 2) {
            const int parts = args.k_splits, mine = (int)cluster_rank();
            int m_tile, n_tile;
            tile_coordinates((int)blockIdx.x / parts, m_tiles, n_tiles, kGroupRows / kBlockM, &m_tile, &n_tile);
            constexpr int kPieces = BN / 4;  // 16-byte pieces of a row
            const uint32_t base = smem_u32(smem);
            for (int item = (threadIdx.x - 64); item < ((kBlockM - mine + parts - 1) / parts) * kPieces; item += kThreads - 64) {
                const int tile_row = mine + (item / kPieces) * parts, piece = item % kPieces;  // neighbouring threads: neighbouring pieces of a row
                const int out_row = m_tile * kBlockM + tile_row, col = n_tile * BN + piece * 4;
                if (out_row >= args.m || col >= args.n) continue;
                const uint32_t at = base + partial_piece(tile_row, piece, BN);
                float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int part = 0; part < parts; ++part) {
                    const float4 v = ld_cluster_f32x4(at, (uint32_t)part);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                float* dst = reinterpret_cast<float*>(args.out) + (size_t)out_row * args.ld_out + col;
                if (col + 4 <= args.n) {
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(sum.x), "f"(sum.y), "f"(sum.z), "f"(sum.w)
                                 : "memory");
                } else {
                    const float v[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (col + i < args.n) dst[i] += v[i];  // the only addition into this element
                }
            }
        }
        cluster_leave_together();  // nobody leaves while its shared memory may still be read
    }
    // every role has left its loop (done, or after a bounded wait gave up): free tensor memory
    tcgen05_fence_before();
    __syncthreads();
    if (kPair == 2) cluster_sync_all();  // neither block leaves while the other may still signal its barriers
    if (warp == 1) {
        tcgen05_fence_after();
        if (kPair == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
    }
}

// Few tiles and a long K (a prompt of a few hundred tokens; the down product above all): with the residual epilogue,
// parts of K go to blocks of their own, at least 8 steps of 64 each and at most 8 parts, and every part adds its sum
// to the residual stream.  Given scratch memory, every part stores its sum there, and once all parts of a tile are
// stored each of its blocks adds a share of the rows over the parts, in their order, so a result is the same bits in
// every run; without scratch each part adds into the stream as it finishes, in no fixed order, and an element's last bit may
// differ from run to run.  Measured at 256 rows, K = 8192, N = 2048: 40 us as 16 tiles, 15 us as 8 parts each, 14 us for
// the library's kernel.  `units`: blocks (or pairs) that run at once.
static int residual_k_splits(long tiles, int k, int units) {
    const int k_blocks = (k + kBlockK - 1) / kBlockK;
    const int want = (int)std::min<long>(std::min<long>(8, units / (tiles > 0 ? tiles : 1)), k_blocks / 8);
    if (want <= 1) return 1;
    const int per_split = (k_blocks + want - 1) / want;
    return (k_blocks + per_split - 1) / per_split;  // no part is empty
}

template <int EPI, int BN, int kPair>
static int launch_tile(const CUtensorMap& map_a, const CUtensorMap& map_w, const GemmArgs& given, int multiprocessors, cudaStream_t stream) {
    constexpr int kOutCols = EPI == EPI_SWIGLU ? 128 : BN;
    const size_t smem = (size_t)kRingBytes + kEpilogueWarps * kStagingBytes + 1024;
    auto kernel = gemm_tcgen05_kernel<EPI, BN, kPair>;
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
        configured = true;
    }
    GemmArgs args = given;
    int tiles = ((args.m + kBlockM * kPair - 1) / (kBlockM * kPair)) * ((args.n + kOutCols - 1) / kOutCols);
    if (EPI == EPI_RESIDUAL) {
        args.k_splits = residual_k_splits(tiles, args.k, kPair == 2 ? multiprocessors / 2 : multiprocessors);
        tiles *= args.k_splits;
    }
    if (kPair == 1 && EPI == EPI_RESIDUAL && args.k_splits > 1) {
        // The parts' blocks of a tile form a cluster, each block with a multiprocessor to itself: clusters of more than
        // four, and clusters of three that would need nearly every multiprocessor, do not find their places at once
        // (measured: 256 rows of the down product 29 us with clusters of eight, 20 with four; 768 rows 47 us with
        // clusters of three on 144 blocks, 33 with two).
        const int whole_tiles = tiles / args.k_splits;
        int parts = args.k_splits < 4 ? args.k_splits : 4;
        if (parts == 3 && whole_tiles * 3 > multiprocessors * 85 / 100) parts = 2;
        args.k_splits = parts;
        tiles = whole_tiles * parts;
    }
    if (kPair == 1 && EPI == EPI_RESIDUAL && args.k_splits > 1 && tiles <= multiprocessors) {
        // the blocks that share a tile's K are one cluster (K is split only while there is a multiprocessor for every
        // item): their sums meet in distributed shared memory, in the order of the parts
        args.cluster_sum = 1;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(tiles);
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = smem;
        config.stream = stream;
        cudaLaunchAttribute attribute[2];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = args.k_splits;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attribute;
        config.numAttrs = dependent_launches_allowed() ? 2 : 1;
        cudaError_t status = cudaLaunchKernelEx(&config, kernel, map_a, map_w, args);
        if (status != cudaSuccess) return fail("gemm_tcgen05: launch of a cluster per tile failed: %s", cudaGetErrorString(status));
        return check_launch("gemm_tcgen05");
    }
    if (kPair == 1) {
        const int grid = tiles < multiprocessors ? tiles : multiprocessors;
        return launch_dependent("gemm_tcgen05", kernel, dim3(grid), dim3(kThreads), smem, stream, true, map_a, map_w, args);
    }
    // pairs of blocks: a cluster of two per tile in flight
    const int pairs = tiles < multiprocessors / 2 ? tiles : multiprocessors / 2;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * (pairs < 1 ? 1 : pairs));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent_launches_allowed() ? 2 : 1;
    cudaError_t status = cudaLaunchKernelEx(&config, kernel, map_a, map_w, args);
    if (status != cudaSuccess) return fail("gemm_tcgen05: launch of block pairs failed: %s", cudaGetErrorString(status));
    return check_launch("gemm_tcgen05");
}

// Which tile width finishes first: rounds of tiles over the multiprocessors times the steps of a tile's loop over K,
// a narrow tile's step counted at 0.75 of a wide one's (it moves more bytes per product; measured 0.7 to 0.8), plus
// what a block costs before and after its loop (about 15 steps).  With the residual epilogue each width is taken
// with the split of K it would run with.
static bool narrow_tiles_are_faster(int m, int n, int k, int multiprocessors, bool residual) {
    const long m_tiles = (m + kBlockM - 1) / kBlockM;
    const long k_blocks = (k + kBlockK - 1) / kBlockK;
    long cost[2];
    for (int narrow = 0; narrow < 2; ++narrow) {
        const long tiles = m_tiles * ((n + (narrow ? 127 : 255)) / (narrow ? 128 : 256));
        const long splits = residual ? std::min(4, residual_k_splits(tiles, k, multiprocessors)) : 1;  // (single blocks: clusters of four at most)
        const long rounds = (tiles * splits + multiprocessors - 1) / multiprocessors;
        const long steps = (k_blocks + splits - 1) / splits;
        cost[narrow] = rounds * (steps * (narrow ? 75 : 100) + 1500);
    }
    return cost[1] < cost[0];
}

// Pairs of blocks (tiles of 256 x 256) move a third less through L2 and shared memory per product and win wherever
// there are tiles enough to keep most pairs busy and work enough per pair to repay the two cluster barriers: measured
// at 2,048 rows, 93.7 against 108 us for the gate/up product (1.47 PFLOP/s) and 49.9 against 54.8 us for the down
// product (K = 8192), but 17.5 against 16.6 us for the output product (one round of tiles over K = 2048); with few
// tiles (512 rows of a 2048-wide matrix) the smaller tiles of single blocks spread better.
static bool pairs_are_faster(int m, int n, int k, int multiprocessors) {
    const long tiles = (long)((m + 255) / 256) * ((n + 255) / 256);
    const long pairs = multiprocessors / 2 > 0 ? multiprocessors / 2 : 1;
    const long rounds = (tiles + pairs - 1) / pairs;
    return tiles >= 48 && rounds * k > 2048;
}

template <int EPI>
static int launch(const CUtensorMap& map_a, const CUtensorMap& map_w, const GemmArgs& args, int multiprocessors, int tile_width,
                  int pair, cudaStream_t stream) {
    if (pair == 2 || (pair == 0 && tile_width == 0 && pairs_are_faster(args.m, args.n, args.k, multiprocessors))) return launch_tile<EPI, 256, 2>(map_a, map_w, args, multiprocessors, stream);
    const bool narrow = tile_width == 128 || (tile_width == 0 && narrow_tiles_are_faster(args.m, args.n, args.k, multiprocessors, EPI == EPI_RESIDUAL));
    if (narrow) return launch_tile<EPI, 128, 1>(map_a, map_w, args, multiprocessors, stream);
    return launch_tile<EPI, 256, 1>(map_a, map_w, args, multiprocessors, stream);
}

}  // namespace mb

using namespace mb;

// a: bfloat16 [m, k] (row stride lda); w: bfloat16 [n_w, k] (row stride ldw).
// epilogue 0: out bfloat16 [m, n_w]; 1: out float32 [m, n_w]; 2: out float32 [m, n_w] += ; 3: w holds gate
// rows [0, n_w/2) and up rows [n_w/2, n_w): out bfloat16 [m, n_w/2] = act(gate) * up, the activation code (MB_ACT_*)
// in bits 8 and up of `epilogue`.
// tile_width: 0 lets the launcher choose between 128 and 256 output columns per tile; the gated epilogue takes 256.
// pair: 2 runs tiles of 256 rows x 256 columns on pairs of blocks (tcgen05 cta_group::2); 1: one block per tile; 0: the launcher chooses.
// Scratch that always suffices for the ordered sum of the parts of K (residual epilogue): K is split only while
// tiles x parts stay within the blocks that run at once, so there are at most `multiprocessors` partial tiles of at
// most 128 x 256 floats, and eight tickets for each.
MB_EXPORT void mb_gemm_tcgen05_scratch(int multiprocessors, size_t* partial_floats, size_t* ticket_ints) {
    *partial_floats = (size_t)multiprocessors * kBlockM * 256;
    *ticket_ints = (size_t)multiprocessors * kEpilogueWarps * 2;
}

// partial, tickets: scratch for the residual epilogue when K is split over blocks (mb_gemm_tcgen05_scratch says how much;
// the tickets zero before the first launch that uses them -- every launch leaves them zero); with both null the parts of K
// add into the stream as they finish, in no fixed order.
MB_EXPORT int mb_gemm_tcgen05(const void* a, int lda, const void* w, int ldw, void* out, int ld_out, int m, int n_w, int k,
                              int epilogue, int multiprocessors, int tile_width, int pair, float* partial, int* tickets,
                              cudaStream_t stream) {
    if (tile_width != 0 && tile_width != 128 && tile_width != 256) return fail("gemm_tcgen05: tile width %d is not built (128, 256)", tile_width);
    if (pair < 0 || pair > 2) return fail("gemm_tcgen05: pair must be 0, 1 or 2, got %d", pair);
    if (pair == 2 && tile_width == 128) return fail("gemm_tcgen05: pairs of blocks take tiles of 256 columns");
    const int activation = epilogue >> 8;
    epilogue &= 0xff;
    if (activation < 0 || activation >= MB_ACT_COUNT) return fail("gemm_tcgen05: unknown gate activation code %d", activation);
    if (m <= 0 || n_w <= 0) return 0;
    if (k <= 0 || k % 8 || lda % 8 || ldw % 8) return fail("gemm_tcgen05: k (%d) and the row strides (%d, %d) must be multiples of 8", k, lda, ldw);
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return fail("gemm_tcgen05: operands must start on 16-byte boundaries");
    if (epilogue == EPI_SWIGLU && n_w % 2) return fail("gemm_tcgen05: the gated epilogue needs an even number of weight rows, got %d", n_w);
    const int n = epilogue == EPI_SWIGLU ? n_w / 2 : n_w;
    const bool wide_out = epilogue == EPI_F32 || epilogue == EPI_RESIDUAL;
    if (((uintptr_t)out & 15) || ld_out % (wide_out ? 4 : 8)) return fail("gemm_tcgen05: output rows must start on 16-byte boundaries");
    CUtensorMap map_a, map_w;
    if (int status = make_map(&map_a, a, m, k, lda)) return status;
    if (int status = make_map(&map_w, w, n_w, k, ldw)) return status;
    GemmArgs args{};
    args.m = m; args.n = n; args.k = k; args.up_row_offset = n; args.activation = activation; args.k_splits = 1;
    args.partial = partial; args.tickets = tickets; args.out = out; args.ld_out = ld_out;
    switch (epilogue) {
        case EPI_BF16: return launch<EPI_BF16>(map_a, map_w, args, multiprocessors, tile_width, pair, stream);
        case EPI_F32: return launch<EPI_F32>(map_a, map_w, args, multiprocessors, tile_width, pair, stream);
        case EPI_RESIDUAL: return launch<EPI_RESIDUAL>(map_a, map_w, args, multiprocessors, tile_width, pair, stream);
        case EPI_SWIGLU:
            if (tile_width == 128) return fail("gemm_tcgen05: the gated epilogue takes tiles of 256 weight rows");
            if (pair == 2 || (pair == 0 && pairs_are_faster(m, 2 * n, k, multiprocessors))) return launch_tile<EPI_SWIGLU, 256, 2>(map_a, map_w, args, multiprocessors, stream);
            return launch_tile<EPI_SWIGLU, 256, 1>(map_a, map_w, args, multiprocessors, stream);
    }
    return fail("gemm_tcgen05: unknown epilogue %d", epilogue);
}

// The q/k/v product of an attention layer for a whole prompt, with the rotation of queries and keys and the paged
// cache write folded into its epilogue.  w: bfloat16 [(heads + 2 kv_heads) * head_dim, k], rows ordered q heads, k
// heads, v heads; q_out: bfloat16 [m, heads * head_dim].  Head sizes 64 and 128 (a tile half holds whole heads).
MB_EXPORT int mb_gemm_tcgen05_qkv_rope(const void* a, int lda, const void* w, int ldw, void* q_out, int ld_q, int m, int k,
                                       int heads, int kv_heads, int head_dim, const int* positions, const float* cos_table,
                                       const float* sin_table, void* k_pool, void* v_pool, const int* slot_mapping,
                                       int page_size, int multiprocessors, cudaStream_t stream) {
    if (m <= 0) return 0;
    if (head_dim != 64 && head_dim != 128) return fail("gemm_tcgen05_qkv_rope: head size %d is not built (64, 128)", head_dim);
    if (heads <= 0 || kv_heads <= 0 || page_size <= 0) return fail("gemm_tcgen05_qkv_rope: heads, kv heads and page size must be positive");
    if (k <= 0 || k % 8 || lda % 8 || ldw % 8) return fail("gemm_tcgen05_qkv_rope: k (%d) and the row strides (%d, %d) must be multiples of 8", k, lda, ldw);
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)q_out & 15) || ld_q % 8 || ((uintptr_t)k_pool & 15) ||
        ((uintptr_t)v_pool & 15) || ((uintptr_t)cos_table & 15) || ((uintptr_t)sin_table & 15))
        return fail("gemm_tcgen05_qkv_rope: operands, tables and pools must start on 16-byte boundaries");
    const int n_w = (heads + 2 * kv_heads) * head_dim;
    CUtensorMap map_a, map_w;
    if (int status = make_map(&map_a, a, m, k, lda)) return status;
    if (int status = make_map(&map_w, w, n_w, k, ldw)) return status;
    GemmArgs args{};
    args.m = m; args.n = n_w; args.k = k; args.up_row_offset = n_w; args.activation = MB_ACT_SILU; args.k_splits = 1;
    args.out = q_out; args.ld_out = ld_q; args.heads = heads; args.kv_heads = kv_heads; args.head_dim = head_dim;
    args.page_size = page_size; args.positions = positions; args.slot_mapping = slot_mapping; args.cos_table = cos_table;
    args.sin_table = sin_table; args.k_pool = (bf16*)k_pool; args.v_pool = (bf16*)v_pool;
    if (pairs_are_faster(m, n_w, k, multiprocessors)) return launch_tile<EPI_ROPE, 256, 2>(map_a, map_w, args, multiprocessors, stream);
    // a prompt of a few hundred tokens has few tiles of 256 columns: tiles of 128 (a half of which still holds a whole
    // head of 64) put twice the blocks to work, and what a block can load a second is what bounds it
    if (head_dim == 64 && narrow_tiles_are_faster(m, n_w, k, multiprocessors, false)) return launch_tile<EPI_ROPE, 128, 1>(map_a, map_w, args, multiprocessors, stream);
    return launch_tile<EPI_ROPE, 256, 1>(map_a, map_w, args, multiprocessors, stream);
}

// 0 when no wait ever gave up; else 1 + (role << 8): 1 producer, 2 MMA (accumulator), 3 MMA (operands), 4 epilogue.
MB_EXPORT int mb_gemm_tc_status() {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    return status;
}
