// Causal grouped-query attention over the paged cache on the tensor cores (bfloat16 storage,
// float accumulation and softmax), compiled for one head size: -DMB_HEAD_DIM=<multiple of 16>.
//
// Two kernels share the tile machinery:
//   * decode: one new token per sequence.  The query heads that share a kv head form the rows of
//     one 16-row MMA tile, so keys and values are read once for the whole group.  A sequence's keys
//     are split over several blocks; partial results (running maximum, sum, unnormalised output)
//     go to scratch memory and a small kernel combines them.
//   * prefill: any number of new tokens per sequence.  A block takes 64 consecutive query tokens of
//     one head (16 per warp) and walks the visible key tiles.
// A tile is the 64 positions of one cache page of one kv head: [64][head_dim], contiguous in the
// pool.  Tiles are brought to shared memory with cp.async, two stages deep, into rows padded by
// 16 bytes so that ldmatrix reads are conflict-free.
//
// Formula: integrallis/models, backend-java/.../llama/LlamaForwardPass.java:1543-1670 (kvHead =
// head / group; dot first, then scale; only positions <= the query's are read; with a window of n
// only the n positions that end at the query) and backend-java/.../ops/TensorOps.java:1247-1279
// (softmax), here in its running form.  Probabilities are rounded to bfloat16 for the P.V product.
#include "attention_tiles.cuh"

#include <cooperative_groups.h>

MB_DEFINE_LAST_ERROR()

namespace mb {

// ------------------------------------------------------------------------------------------ decode

// grid (splits, kv_heads * head_chunks, sequences).  Rows of the MMA tile are the (up to 16) query
// heads of one kv head; each of the 4 warps takes 16 of a tile's 64 keys.
// kCluster: the `splits` blocks of one (sequence, kv head) form a thread-block cluster and combine
// their partial results in the first block's shared memory (distributed shared memory) instead of
// going through scratch memory and a second kernel; splits <= 8 then.
template <bool kCluster, int kDecodeStages>
__global__ void __launch_bounds__(kThreads)
decode_attention_kernel(const bf16* __restrict__ q, int q_row_stride, bf16* __restrict__ out, int out_row_stride,
                        const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                        const int* __restrict__ kv_lens, int heads, int kv_heads, int head_chunks, int window,
                        float scale, int splits, float* __restrict__ partial_o, float* __restrict__ partial_ml) {
    grid_launch_dependents();
    // The query, and the keys and values of the newest position, come from the kernel before this one.
    // Lengths and page tables were written before the step began, and every older position of the
    // cache in an earlier step: a block may fetch its first pages before it waits for that kernel,
    // up to the one that holds the newest position.
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* stage_smem = smem;  // kDecodeStages x (K tile, V tile)
    // The 16 query rows pass through the last stage, which no page is fetched into before they are in registers: a
    // block's shared memory is its stages alone, and a fourth block with three stages fits a multiprocessor (heads of 64).
    // Every warp has a copy of them in the 16 key rows of that stage which only itself will ever write, so no warp waits
    // for another before the walk over the pages begins.
    unsigned char* q_smem = smem + (kDecodeStages - 1) * 2 * kTileBytes + (threadIdx.x >> 5) * 16 * kRowBytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const int split = blockIdx.x, seq = blockIdx.z;
    const int kv_head = blockIdx.y / head_chunks, chunk = blockIdx.y % head_chunks;
    const int group = heads / kv_heads;
    const int head0 = kv_head * group + chunk * 16;
    const int rows_here = min(16, group - chunk * 16);
    const int q_row = cu_q[seq];
    const int kv_len = kv_lens[seq];
    const int pos = kv_len - 1;
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first_tile = first / kTile;
    const int tiles = (kv_len + kTile - 1) / kTile - first_tile;
    const int per_split = (tiles + splits - 1) / splits;
    const int t_begin = first_tile + split * per_split;
    const int t_end = min(t_begin + per_split, first_tile + tiles);

    const bool empty = t_begin >= t_end;  // nothing for this split
    if (empty && !kCluster) {  // an empty partial
        grid_dependency_wait();  // (the scratch memory may still be read by a kernel before this one)
        if (threadIdx.x < rows_here) {
            float* ml = partial_ml + ((size_t)(seq * heads + head0 + threadIdx.x) * splits + split) * 2;
            ml[0] = -CUDART_INF_F;
            ml[1] = 0.0f;
        }
        return;
    }

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float run_max[2] = {-CUDART_INF_F, -CUDART_INF_F}, run_sum[2] = {0.0f, 0.0f};  // maxima of raw scores
    const float scale_log2 = scale * 1.4426950408889634f;  // positive
    if (empty) grid_dependency_wait();
    if (!empty) {
    const int* table = block_table + (size_t)seq * max_blocks;
    const uint32_t stage_base = smem_u32(stage_smem);
    // kDecodeStages - 1 pages are in flight while one is worked on; every stage is one commit group, empty
    // groups past the last page keep the count the waits rely on.  Of these first pages, those that hold no
    // position of this step (all but the sequence's last page) are asked for before the wait for the kernel
    // before this one, the others after it.
    const int newest = pos / kTile;
    bool waited = false;
#pragma unroll
    for (int ahead = 0; ahead < kDecodeStages - 1; ++ahead) {
        if (!waited && (t_begin + ahead >= t_end || t_begin + ahead == newest)) {
            grid_dependency_wait();
            waited = true;
        }
        if (t_begin + ahead < t_end) {
            const uint32_t dst = stage_base + ahead * 2 * kTileBytes;
            load_tile_rows(dst, k_pool, table[t_begin + ahead], kv_head, kv_heads, warp, lane);
            load_tile_rows(dst + kTileBytes, v_pool, table[t_begin + ahead], kv_head, kv_heads, warp, lane);
        }
        cp_async_commit();
    }
    if (!waited) grid_dependency_wait();
    {
        const bf16* q_first_row = q + (size_t)q_row * q_row_stride + (size_t)head0 * HD;  // (heads lie HD apart in a row of q)
        for (int i = lane; i < kQRowsDecode * kChunks; i += 32) {
            const int row = i / kChunks, chunk = i % kChunks;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (row < rows_here) v = *reinterpret_cast<const uint4*>(q_first_row + (size_t)row * HD + chunk * 8);
            *reinterpret_cast<uint4*>(q_smem + row * kRowBytes + chunk * 16) = v;
        }
    }
    __syncwarp();
    uint32_t a[kKSteps][4];
    load_q_fragments(a, smem_u32(q_smem));
    __syncwarp();  // the warp has its queries in registers: its rows of the last stage are free for pages

    // the page table is read one page ahead of the fetch that needs it, so that no fetch waits for its entry
    int page_ahead = t_begin + kDecodeStages - 1 < t_end ? table[t_begin + kDecodeStages - 1] : 0;
    for (int t = t_begin; t < t_end; ++t) {
        const int stage = (t - t_begin) % kDecodeStages;
        {
            const int fetch = t + kDecodeStages - 1;  // its stage was freed by the barrier that ended page t - 1
            const int page = page_ahead;
            if (fetch + 1 < t_end) page_ahead = table[fetch + 1];
            if (fetch < t_end) {
                const uint32_t next = stage_base + ((fetch - t_begin) % kDecodeStages) * 2 * kTileBytes;
                load_tile_rows(next, k_pool, page, kv_head, kv_heads, warp, lane);
                load_tile_rows(next + kTileBytes, v_pool, page, kv_head, kv_heads, warp, lane);
            }
            cp_async_commit();
            cp_async_wait<kDecodeStages - 1>();  // everything but the newest kDecodeStages - 1 groups: page t is in
        }
        __syncwarp();  // the warp's own rows: every lane's pieces have landed
        const uint32_t k_tile = stage_base + stage * 2 * kTileBytes, v_tile = k_tile + kTileBytes;
        const int key0 = warp * 16;
        const int abs0 = t * kTile + key0;
        if (abs0 <= pos && abs0 + 15 >= first) {  // this warp's 16 keys hold something visible
            float s[2][4];
            scores_16_keys(s, a, k_tile, key0);
            float tile_max = -CUDART_INF_F;
            if (abs0 < first || abs0 + 15 > pos) {  // an end of the visible range runs through these 16 keys
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int key = abs0 + nt * 8 + tid4 * 2 + (i & 1);
                        if (key < first || key > pos) s[nt][i] = -CUDART_INF_F;
                    }
            }
            // one token: both rows of a lane see the same keys, so one maximum test serves the mask
            float row_max[2] = {fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1])),
                                fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]))};
            uint32_t p[4];
            float probs[2][4];
            // scores stay raw; the scale (times log2 e) is folded into the exponent: 2^(s*c - m*c)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tile_max = quad_max(row_max[r]);
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
            p[0] = pack_bf16(probs[0][0], probs[0][1]);
            p[1] = pack_bf16(probs[0][2], probs[0][3]);
            p[2] = pack_bf16(probs[1][0], probs[1][1]);
            p[3] = pack_bf16(probs[1][2], probs[1][3]);
            accumulate_16_keys(o, p, v_tile, key0);
        }
        __syncwarp();  // the warp's rows of the stage are free for the load after next
    }
    }  // !empty
    run_sum[0] = quad_sum(run_sum[0]);
    run_sum[1] = quad_sum(run_sum[1]);

    // merge the four warps' partial results through shared memory: the stages are free once every warp has left its loop
    __syncthreads();
    float* merge_o = reinterpret_cast<float*>(stage_smem);         // [4 warps][16 rows][HD]
    float* merge_ml = merge_o + 4 * 16 * HD;                        // [4 warps][16 rows][2]
    float* block_o = merge_ml + 4 * 16 * 2;                         // [16 rows][HD]   (cluster: this block's result)
    float* block_ml = block_o + 16 * HD;                            // [16 rows][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = group_id + 8 * r;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            float* dst = merge_o + ((size_t)(warp * 16 + row)) * HD + i * 8 + tid4 * 2;
            dst[0] = o[i][2 * r];
            dst[1] = o[i][2 * r + 1];
        }
        if (tid4 == 0) {
            merge_ml[(warp * 16 + row) * 2] = run_max[r] * scale_log2;  // from here on maxima are exponents of two
            merge_ml[(warp * 16 + row) * 2 + 1] = run_sum[r];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows_here * HD; i += kThreads) {
        const int row = i / HD, d = i % HD;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, merge_ml[(w * 16 + row) * 2]);
        float total = 0.0f, value = 0.0f;
        if (m != -CUDART_INF_F) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float weight = fast_exp2(merge_ml[(w * 16 + row) * 2] - m);  // 2^-inf = 0 for a warp that saw nothing
                total += merge_ml[(w * 16 + row) * 2 + 1] * weight;
                value += merge_o[(size_t)(w * 16 + row) * HD + d] * weight;
            }
        }
        const int head = head0 + row;
        if (kCluster) {
            block_o[row * HD + d] = value;
            if (d == 0) {
                block_ml[row * 2] = m;
                block_ml[row * 2 + 1] = total;
            }
        } else if (splits == 1) {
            out[(size_t)q_row * out_row_stride + (size_t)head * HD + d] = __float2bfloat16_rn(value * (1.0f / total));
        } else {
            const size_t slot = (size_t)(seq * heads + head) * splits + split;
            partial_o[slot * HD + d] = value;
            if (d == 0) {
                partial_ml[slot * 2] = m;
                partial_ml[slot * 2 + 1] = total;
            }
        }
    }
    if (kCluster) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        // every block of the cluster combines a share of the (head, coordinate) results: all reads of the other blocks'
        // shared memory are asked for at once, then the parts are weighed in the order of the blocks
        const int rank = (int)cluster.block_rank();
        const int items = rows_here * HD, share = (items + splits - 1) / splits;
        for (int i = rank * share + threadIdx.x; i < min(items, (rank + 1) * share); i += kThreads) {
            const int row = i / HD, d = i % HD;
            float part_m[8], part_l[8], part_o[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < splits) {
                    const float* ml = cluster.map_shared_rank(block_ml, r);
                    part_m[r] = ml[row * 2];
                    part_l[r] = ml[row * 2 + 1];
                    part_o[r] = cluster.map_shared_rank(block_o, r)[row * HD + d];
                } else {
                    part_m[r] = -CUDART_INF_F;
                    part_l[r] = 0.0f;
                    part_o[r] = 0.0f;
                }
            }
            float m = part_m[0];
#pragma unroll
            for (int r = 1; r < 8; ++r) m = fmaxf(m, part_m[r]);
            float total = 0.0f, value = 0.0f;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float weight = fast_exp2(part_m[r] - m);  // 0 for a block that saw nothing
                if (weight > 0.0f) {
                    total += part_l[r] * weight;
                    value += part_o[r] * weight;
                }
            }
            out[(size_t)q_row * out_row_stride + (size_t)(head0 + row) * HD + d] = __float2bfloat16_rn(value * (1.0f / total));
        }
        cluster_leave_together();  // the other blocks' shared memory has been read; they may leave
    }
}

// grid (heads, sequences), HD threads... one thread per output coordinate (strided).
__global__ void combine_splits_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                      bf16* __restrict__ out, int out_row_stride, const int* __restrict__ cu_q,
                                      int heads, int splits) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int head = blockIdx.x, seq = blockIdx.y;
    const size_t base = (size_t)(seq * heads + head) * splits;
    float m = -CUDART_INF_F;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, partial_ml[(base + s) * 2]);
    float total = 0.0f;
    for (int s = 0; s < splits; ++s) total += partial_ml[(base + s) * 2 + 1] * fast_exp2(partial_ml[(base + s) * 2] - m);
    const float inv = 1.0f / total;
    const int row = cu_q[seq];
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float value = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float weight = fast_exp2(partial_ml[(base + s) * 2] - m);
            if (weight > 0.0f) value += partial_o[(base + s) * HD + d] * weight;  // an empty split wrote no output
        }
        out[(size_t)row * out_row_stride + (size_t)head * HD + d] = __float2bfloat16_rn(value * inv);
    }
}

// ------------------------------------------------------------------------------------------ prefill

// grid (query tiles of 64 tokens, heads, sequences); warp w owns tokens 16w..16w+15 of the tile.
__global__ void __launch_bounds__(kThreads)
prefill_attention_kernel(const bf16* __restrict__ q, int q_row_stride, bf16* __restrict__ out, int out_row_stride,
                         const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
                         const int* __restrict__ kv_lens, int heads, int kv_heads, int window, float scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* q_smem = smem;                                  // 64 rows
    unsigned char* stage_smem = smem + kQRowsPrefill * kRowBytes;  // 2 stages x (K tile, V tile)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int kv_head = head / (heads / kv_heads);
    const int q_begin = cu_q[seq];
    const int q_len = cu_q[seq + 1] - q_begin;
    const int q_tile = gridDim.x - 1 - blockIdx.x;  // the tiles with the most keys start first
    const int t0 = q_tile * kQRowsPrefill;
    if (t0 >= q_len) return;
    const int valid = min(kQRowsPrefill, q_len - t0);
    const int kv_len = kv_lens[seq];
    const int pos0 = kv_len - q_len + t0;  // position of the tile's first token
    const int last_pos = pos0 + valid - 1;
    const int first_needed = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int t_begin = first_needed / kTile, t_end = last_pos / kTile + 1;

    const int* table = block_table + (size_t)seq * max_blocks;
    const uint32_t stage_base = smem_u32(stage_smem);
    load_tile(stage_base, k_pool, table[t_begin], kv_head, kv_heads);
    load_tile(stage_base + kTileBytes, v_pool, table[t_begin], kv_head, kv_heads);
    cp_async_commit();
    load_queries(q_smem, q + (size_t)(q_begin + t0) * q_row_stride + (size_t)head * HD, q_row_stride, kQRowsPrefill, valid);
    __syncthreads();
    uint32_t a[kKSteps][4];
    load_q_fragments(a, smem_u32(q_smem) + warp * 16 * kRowBytes);

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float run_max[2] = {-CUDART_INF_F, -CUDART_INF_F}, run_sum[2] = {0.0f, 0.0f};
    // this lane's two rows: positions, and the first position each sees
    int row_pos[2], row_first[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + group_id + 8 * r;
        row_pos[r] = row < valid ? pos0 + row : -1;  // a row beyond the sequence sees nothing
        row_first[r] = (window > 0 && row_pos[r] - window + 1 > 0) ? row_pos[r] - window + 1 : 0;
    }
    const float scale_log2 = scale * 1.4426950408889634f;
    const int warp_last = min(pos0 + warp * 16 + 15, last_pos);        // highest position among the warp's rows
    const int warp_first_pos = pos0 + warp * 16;                        // lowest
    const int warp_first_key = (window > 0 && warp_first_pos - window + 1 > 0) ? warp_first_pos - window + 1 : 0;
    const bool warp_has_rows = warp * 16 < valid;

    for (int t = t_begin; t < t_end; ++t) {
        const int stage = (t - t_begin) & 1;
        if (t + 1 < t_end) {
            const uint32_t next = stage_base + (stage ^ 1) * 2 * kTileBytes;
            load_tile(next, k_pool, table[t + 1], kv_head, kv_heads);
            load_tile(next + kTileBytes, v_pool, table[t + 1], kv_head, kv_heads);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t k_tile = stage_base + stage * 2 * kTileBytes, v_tile = k_tile + kTileBytes;
        const int key_base = t * kTile;
        if (warp_has_rows && key_base <= warp_last && key_base + kTile - 1 >= warp_first_key) {
            // every key of the tile is visible to every row of the warp: no mask needed
            const bool full = key_base + kTile - 1 <= warp_first_pos && key_base >= ((window > 0) ? max(0, warp_last - window + 1) : 0)
                              && warp * 16 + 15 < valid;
            // scores of the whole tile first, so that the running maximum moves once per 64 keys
            float s[kTile / 8][4];
#pragma unroll
            for (int part = 0; part < kTile / 16; ++part) {
                float two[2][4];
                scores_16_keys(two, a, k_tile, part * 16);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s[2 * part][i] = two[0][i];
                    s[2 * part + 1][i] = two[1][i];
                }
            }
            // scores stay raw; the scale (times log2 e) is folded into the exponent: 2^(s*c - m*c)
            float part_max[2] = {-CUDART_INF_F, -CUDART_INF_F};
            if (full) {
#pragma unroll
                for (int nt = 0; nt < kTile / 8; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) part_max[i >> 1] = fmaxf(part_max[i >> 1], s[nt][i]);
            } else {
#pragma unroll
                for (int nt = 0; nt < kTile / 8; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int key = key_base + nt * 8 + tid4 * 2 + (i & 1);
                        const int r = i >> 1;
                        if (!(key <= row_pos[r] && key >= row_first[r])) s[nt][i] = -CUDART_INF_F;
                        part_max[r] = fmaxf(part_max[r], s[nt][i]);
                    }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float new_max = fmaxf(run_max[r], quad_max(part_max[r]));  // in raw score units
                // a row that has seen nothing yet keeps -inf; subtract 0 then so that the exponent is -inf, not NaN
                const float safe_max = new_max == -CUDART_INF_F ? 0.0f : new_max;
                const float correction = fast_exp2((run_max[r] - safe_max) * scale_log2);
                const float offset = -safe_max * scale_log2;
                run_max[r] = new_max;
                float local = 0.0f;
#pragma unroll
                for (int nt = 0; nt < kTile / 8; ++nt)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const float e = fast_exp2(fmaf(s[nt][2 * r + c], scale_log2, offset));
                        s[nt][2 * r + c] = e;
                        local += e;
                    }
                run_sum[r] = run_sum[r] * correction + local;
#pragma unroll
                for (int i = 0; i < HD / 8; ++i) {
                    o[i][2 * r] *= correction;
                    o[i][2 * r + 1] *= correction;
                }
            }
#pragma unroll
            for (int part = 0; part < kTile / 16; ++part) {
                uint32_t p[4];
                p[0] = pack_bf16(s[2 * part][0], s[2 * part][1]);
                p[1] = pack_bf16(s[2 * part][2], s[2 * part][3]);
                p[2] = pack_bf16(s[2 * part + 1][0], s[2 * part + 1][1]);
                p[3] = pack_bf16(s[2 * part + 1][2], s[2 * part + 1][3]);
                accumulate_16_keys(o, p, v_tile, part * 16);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + group_id + 8 * r;
        const float total = quad_sum(run_sum[r]);
        if (row >= valid) continue;
        const float inv = 1.0f / total;
        bf16* dst = out + (size_t)(q_begin + t0 + row) * out_row_stride + (size_t)head * HD;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8 + tid4 * 2) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
}

constexpr size_t decode_smem(int stages) {
    const size_t tiles = 2 * stages * (size_t)kTileBytes;  // (the queries lie in the last stage)
    const size_t merge = (4 * 16 * HD + 4 * 16 * 2 + 16 * HD + 16 * 2) * sizeof(float);
    return tiles > merge ? tiles : merge;
}
constexpr size_t prefill_smem() { return (size_t)kQRowsPrefill * kRowBytes + 4 * (size_t)kTileBytes; }

static int check_common(const char* what, int heads, int kv_heads, int page_size, int q_row_stride, int out_row_stride,
                        const void* q, const void* out) {
    if (kv_heads <= 0 || heads % kv_heads) return fail("%s: %d heads are no multiple of %d kv heads", what, heads, kv_heads);
    if (page_size != kTile) return fail("%s: the cache page must hold %d positions, got %d", what, kTile, page_size);
    if (q_row_stride % 8 || out_row_stride % 2 || ((uintptr_t)q & 15) || ((uintptr_t)out & 3))
        return fail("%s: query rows must start on 16-byte boundaries (row stride %d elements)", what, q_row_stride);
    return 0;
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_attention_head_dim() { return HD; }

// Page stages a decode call with `splits` blocks per sequence runs with at least (see the note on page stages above;
// a call whose blocks all fit the multiprocessors with three stages gets three), and the shared memory of one block
// with so many stages: for callers that plan how many blocks are resident at once.
MB_EXPORT int mb_decode_stages(int splits) { return (HD >= 96 || splits >= 4) ? 3 : 2; }
// More than a cluster's eight splits are for long contexts.  While the call's blocks are so few that at most two
// share a multiprocessor, pages of 8 KB (heads up to 64) are fetched five ahead instead of two: one sequence of
// 32,768 positions, 32 splits, 26.4 -> 24.2 us; of 131,072 positions 80.9 -> 71.4 us.  With more blocks the
// shared memory is worth more as room for further blocks (8 sequences of 65,536 positions: 195 us with three
// stages, 242 us with six), and pages of wider heads gain nothing from a deeper ring.
constexpr int kLongStages = HD <= 64 ? 6 : 3;
constexpr int kMaxDevices = 64;  // per-device facts below are kept for devices 0..63

// The current device, or -1 (with the message set) when it cannot be told or lies beyond the per-device tables.
static int current_device(const char* what) {
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) { fail("%s: cudaGetDevice: %s", what, cudaGetErrorString(status)); return -1; }
    if (device < 0 || device >= kMaxDevices) { fail("%s: device %d is outside 0..%d", what, device, kMaxDevices - 1); return -1; }
    return device;
}

static int multiprocessor_count(int device) {
    static int multiprocessors[kMaxDevices] = {0};  // of each device, asked once
    if (!multiprocessors[device] &&
        cudaDeviceGetAttribute(&multiprocessors[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        multiprocessors[device] = 1;  // unknown: the deep ring only for a handful of blocks
    return multiprocessors[device];
}

static int decode_stages(int splits, long blocks, int device) {
    const int sms = multiprocessor_count(device);
    if (splits > 8 && blocks <= 2L * sms) return kLongStages;
    // Few splits mean long walks per block (64 sequences: ten pages each), and with two stages a block waits for every
    // page: a third stage, as long as all blocks of the call still fit the multiprocessors at once with it.
    const long resident_with_three = (long)((227 * 1024) / (decode_smem(3) + 1024)) * sms;
    if (splits < 4 && blocks <= resident_with_three) return 3;
    return mb_decode_stages(splits);
}
MB_EXPORT size_t mb_decode_block_bytes(int stages) { return decode_smem(stages); }

// Scratch floats a decode call with `splits` > 1 needs: partial outputs and (maximum, sum) pairs.
MB_EXPORT size_t mb_decode_scratch_floats(int sequences, int heads, int splits) {
    return splits > 1 ? (size_t)sequences * heads * splits * (HD + 2) : 0;
}

MB_EXPORT int mb_decode_attention(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_pool,
                                  const void* v_pool, const int* block_table, int max_blocks, const int* cu_q,
                                  const int* kv_lens, int sequences, int heads, int kv_heads, int page_size, int window,
                                  float scale, int splits, float* scratch, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    if (int status = check_common("decode_attention", heads, kv_heads, page_size, q_row_stride, out_row_stride, q, out)) return status;
    if (splits < 1) return fail("decode_attention: splits %d must be at least 1", splits);
    const int group = heads / kv_heads;
    const int head_chunks = (group + 15) / 16;
    if (sequences > 65535 || kv_heads * head_chunks > 65535) return fail("decode_attention: grid too large");
    const int device = current_device("decode_attention");
    if (device < 0) return 1;
    const int stages = decode_stages(splits, (long)splits * kv_heads * head_chunks * sequences, device);
    static bool configured_devices[kMaxDevices] = {false};  // the attribute is a device's, not the process's
    bool& configured = configured_devices[device];
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(decode_attention_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(2));
        if (status == cudaSuccess)
            status = cudaFuncSetAttribute(decode_attention_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (status == cudaSuccess)
            status = cudaFuncSetAttribute(decode_attention_kernel<false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(3));
        if (status == cudaSuccess)
            status = cudaFuncSetAttribute(decode_attention_kernel<true, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (status == cudaSuccess && kLongStages > 3)
            status = cudaFuncSetAttribute(decode_attention_kernel<false, kLongStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(kLongStages));
        if (status != cudaSuccess) return fail("decode_attention: cannot reserve %zu bytes of shared memory: %s", decode_smem(kLongStages), cudaGetErrorString(status));
        configured = true;
    }
    const dim3 grid(splits, kv_heads * head_chunks, sequences);
    if (splits > 1 && !scratch) {
        // no scratch given: the splits of a sequence meet inside a thread-block cluster
        if (splits > 8) return fail("decode_attention: %d splits without scratch memory exceed the cluster limit of 8", splits);
        cudaLaunchConfig_t config = {};
        config.gridDim = grid;
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = decode_smem(stages);
        {
            // The blocks of a cluster are placed on as few multiprocessors as will hold them, where they share what one
            // multiprocessor can load.  Asking for as much shared memory as still lets all blocks of the call be resident
            // at once spreads them (8 sequences, 256 blocks: 0.792 ms per decode step at four blocks to a multiprocessor,
            // 0.762 at two; one sequence, 64 blocks: 0.722 and 0.703 with one; 16 sequences, 512 blocks, need all four).
            const long blocks = (long)splits * kv_heads * head_chunks * sequences;
            const int sms = multiprocessor_count(device);
            long share = (blocks + sms - 1) / sms;  // blocks a multiprocessor has to hold
            // (clusters of eight do not find eight multiprocessors of their own at once while the kernel before them still
            // holds some: they are packed at least two to a multiprocessor, three when there are more blocks than
            // multiprocessors -- 4 sequences: 0.746 ms per step with three, 0.777 with two)
            if (splits > 4) share = blocks <= sms ? 2 : (share < 3 ? 3 : share);
            const size_t room = (size_t)(227 * 1024) / (size_t)(share < 1 ? 1 : share) - 1024;
            const size_t want = room < (size_t)200 * 1024 ? room : (size_t)200 * 1024;
            if (want > config.dynamicSmemBytes) config.dynamicSmemBytes = want;
        }
        config.stream = stream;
        cudaLaunchAttribute attribute[2];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = splits;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attribute;
        config.numAttrs = dependent_launches_allowed() ? 2 : 1;
        auto kernel = stages == 3 ? decode_attention_kernel<true, 3> : decode_attention_kernel<true, 2>;
        cudaError_t status = cudaLaunchKernelEx(&config, kernel, (const bf16*)q, q_row_stride, (bf16*)out,
                                                out_row_stride, (const bf16*)k_pool, (const bf16*)v_pool, block_table, max_blocks,
                                                cu_q, kv_lens, heads, kv_heads, head_chunks, window, scale, splits,
                                                (float*)nullptr, (float*)nullptr);
        if (status != cudaSuccess) return fail("decode_attention: launch failed: %s", cudaGetErrorString(status));
        return check_launch("decode_attention");
    }
    float* partial_o = scratch;
    float* partial_ml = scratch ? scratch + (size_t)sequences * heads * splits * HD : nullptr;
    auto kernel = stages == kLongStages ? decode_attention_kernel<false, kLongStages>
                                        : (stages == 3 ? decode_attention_kernel<false, 3> : decode_attention_kernel<false, 2>);
    if (int status = launch_dependent("decode_attention", kernel, grid, dim3(kThreads), decode_smem(stages), stream, true,
                                      (const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_pool,
                                      (const bf16*)v_pool, block_table, max_blocks, cu_q, kv_lens, heads, kv_heads, head_chunks,
                                      window, scale, splits, partial_o, partial_ml))
        return status;
    if (splits > 1)
        return launch_dependent("combine_splits", combine_splits_kernel, dim3(heads, sequences), dim3(HD < 64 ? 32 : 64), 0, stream,
                                true, (const float*)partial_o, (const float*)partial_ml, (bf16*)out, out_row_stride, cu_q, heads,
                                splits);
    return 0;
}

MB_EXPORT int mb_prefill_attention(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_pool,
                                   const void* v_pool, const int* block_table, int max_blocks, const int* cu_q,
                                   const int* kv_lens, int sequences, int max_q_len, int heads, int kv_heads,
                                   int page_size, int window, float scale, cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0) return 0;
    if (int status = check_common("prefill_attention", heads, kv_heads, page_size, q_row_stride, out_row_stride, q, out)) return status;
    if (sequences > 65535 || heads > 65535) return fail("prefill_attention: grid too large");
    const int device = current_device("prefill_attention");
    if (device < 0) return 1;
    static bool configured_devices[kMaxDevices] = {false};
    bool& configured = configured_devices[device];
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(prefill_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_smem());
        if (status != cudaSuccess) return fail("prefill_attention: cannot reserve %zu bytes of shared memory: %s", prefill_smem(), cudaGetErrorString(status));
        configured = true;
    }
    const dim3 grid((max_q_len + kQRowsPrefill - 1) / kQRowsPrefill, heads, sequences);
    return launch_dependent("prefill_attention", prefill_attention_kernel, grid, dim3(kThreads), prefill_smem(), stream, true,
                            (const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,
                            block_table, max_blocks, cu_q, kv_lens, heads, kv_heads, window, scale);
}

// ------------------------------------------------------------------------------------------------
// Decode attention that allocates nothing (declared in attention_tc.h; integrallis/models has no
// counterpart of it).
//
// mb_decode_attention() takes its scratch from the caller, and the Python face of this library gets
// it from the framework's allocator.  A plain C or C++ host that runs these kernels by itself may
// not be able to do that: one that handed all device memory to an arena of its own when it started,
// or one that serves requests in a loop in which cudaMalloc -- which can fail once memory is
// committed, and synchronises the device -- must not appear.  For such a caller the partial results
// of the split keys live in the file-scope array below instead.  It is part of the library's image:
// every GPU that loads this library holds kStaticScratchFloats * 4 bytes for it until the process
// exits.
//
// The array's name is usable in device code only; host code sees a stand-in for it, not a device
// address.  So the entry point asks the runtime for the address once per device, with that device
// current (cudaGetSymbolAddress), keeps it, and hands it to the kernels.  The first call on a
// device does this set-up; make that first call outside any stream capture, and from one thread:
// the per-device tables are plain statics, so two first calls on one device must not run at once.
//
// Every call uses the same array, and it keeps what the last call left.  Nothing in it has to be
// zero at the start: each block writes its (maximum, sum) pair, and a partial output is read only
// where that pair says the block saw keys.  Two calls that overlap on the GPU (different streams,
// no ordering between them) race on the array; order them.
constexpr size_t kStaticScratchFloats = 1u << 20;  // 4 MiB
static __device__ __align__(256) float g_static_decode_scratch[kStaticScratchFloats];
static float* g_static_scratch_address[kMaxDevices] = {nullptr};

MB_EXPORT size_t mb_decode_attention_static_capacity() { return kStaticScratchFloats; }

MB_EXPORT int mb_decode_attention_static(const void* q, int q_row_stride, void* out, int out_row_stride,
                                         const void* k_pool, const void* v_pool, const int* block_table, int max_blocks,
                                         const int* cu_q, const int* kv_lens, int sequences, int heads, int kv_heads,
                                         int page_size, int window, float scale, int splits, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    if (splits < 1) return fail("decode_attention_static: splits %d must be at least 1", splits);
    const size_t need = mb_decode_scratch_floats(sequences, heads, splits);
    if (need > kStaticScratchFloats)
        return fail("decode_attention_static: %d sequences x %d heads x %d splits need %zu floats of scratch, the built-in "
                    "array holds %zu; use fewer splits or mb_decode_attention with scratch of your own",
                    sequences, heads, splits, need, (size_t)kStaticScratchFloats);
    const int device = current_device("decode_attention_static");
    if (device < 0) return 1;
    if (!g_static_scratch_address[device]) {
        float* address = nullptr;
        cudaError_t status = cudaGetSymbolAddress((void**)&address, g_static_decode_scratch);
        if (status != cudaSuccess || !address)
            return fail("decode_attention_static: cudaGetSymbolAddress on device %d: %s", device, cudaGetErrorString(status));
        g_static_scratch_address[device] = address;
    }
    return mb_decode_attention(q, q_row_stride, out, out_row_stride, k_pool, v_pool, block_table, max_blocks, cu_q, kv_lens,
                               sequences, heads, kv_heads, page_size, window, scale, splits,
                               splits > 1 ? g_static_scratch_address[device] : nullptr, stream);
}
