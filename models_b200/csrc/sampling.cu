// Next-token selection on the device: greedy argmax and the sampling pipeline of
// integrallis/models (models-runtime/.../Sampler.java:37-151,174-205,244-252):
//   repetition penalty once per earlier occurrence (positive logit / r, otherwise * r),
//   divide by the temperature, softmax over the whole vocabulary (max subtracted, exp, / sum),
//   the k most probable tokens with ties going to the lower id, the shortest prefix of these (most
//   probable first) whose mass reaches top_p, crossing token included, then an inverse-CDF draw
//   r = u * kept mass.  Temperature 0 is argmax, first maximum wins.
// The uniform u comes from Philox4x32-10 keyed by the request's seed, with the request's draw
// counter as the counter, 24 random bits as Java's Random.nextFloat() uses; the stream is
// reproducible but not the Java generator's.
//
// One block of 1024 threads per row.  `work` is caller-provided scratch of rows * vocab floats
// and `counts` rows * vocab ints (only touched by rows whose penalty is > 1).
#include "common.cuh"

#include <cooperative_groups.h>
#include <math_constants.h>

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kThreads = 1024;
constexpr int kMaxSorted = 1024;

struct Best {
    float value;
    int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    // greater value wins; equal values: the lower index (first maximum wins)
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

__device__ Best block_best(Best mine, Best* scratch /* 32 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        Best other;
        other.value = __shfl_xor_sync(0xffffffffu, mine.value, offset);
        other.index = __shfl_xor_sync(0xffffffffu, mine.index, offset);
        mine = better(mine, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    Best total = scratch[lane < (int)(blockDim.x >> 5) ? lane : 0];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        Best other;
        other.value = __shfl_xor_sync(0xffffffffu, total.value, offset);
        other.index = __shfl_xor_sync(0xffffffffu, total.index, offset);
        total = better(total, other);
    }
    return total;
}

// Exclusive prefix sum of a 0/1 flag over the block (thread order); *total gets the block's sum.
__device__ int block_flag_scan(bool flag, int* warp_totals /* 32 */, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned ballot = __ballot_sync(0xffffffffu, flag);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    __syncthreads();
    if (lane == 0) warp_totals[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, all = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
        const int t = warp_totals[w];
        if (w < warp) before += t;
        all += t;
    }
    *total = all;
    return before + in_warp;
}

// Inclusive prefix sum of floats over the block in thread order (a fixed order of additions).
__device__ float block_float_scan(float v, float* warp_totals /* 32 */, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, v, offset);
        if (lane >= offset) v += up;
    }
    __syncthreads();
    if (lane == 31) warp_totals[warp] = v;
    __syncthreads();
    float before = 0.0f, all = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
        const float t = warp_totals[w];
        if (w < warp) before += t;
        all += t;
    }
    *total = all;
    return before + v;
}

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t (&k)[2]) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k[0], n1 = lo1, n2 = hi0 ^ c[3] ^ k[1], n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k[0] += 0x9E3779B9u;
    k[1] += 0xBB67AE85u;
}

__device__ float philox_uniform(unsigned long long seed, unsigned long long counter) {
    uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32), 0u, 0u};
    uint32_t k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
#pragma unroll
    for (int round = 0; round < 10; ++round) philox_round(c, k);
    return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

constexpr int kArgmaxBlocks = 8;  // blocks of a cluster that share one row

// grid (kArgmaxBlocks, rows), clusters of kArgmaxBlocks along x: each block scans an eighth of the
// row, the first block of the cluster picks among the eight candidates (distributed shared memory).
__global__ void __launch_bounds__(kThreads)
argmax_rows_kernel(const float* __restrict__ logits, int row_stride, int vocab, int* __restrict__ out) {
    grid_launch_dependents();
    grid_dependency_wait();
    namespace cg = cooperative_groups;
    __shared__ Best scratch[32];
    __shared__ Best block_result;
    cg::cluster_group cluster = cg::this_cluster();
    const int part = cluster.block_rank();
    const float* row = logits + (size_t)blockIdx.y * row_stride;
    const int per_block = (vocab + kArgmaxBlocks - 1) / kArgmaxBlocks;
    const int begin = part * per_block, end = min(vocab, begin + per_block);
    Best mine = {-CUDART_INF_F, 0x7fffffff};
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (v > mine.value) mine = {v, i};  // ascending i per thread: the first maximum stays
    }
    const Best best = block_best(mine, scratch);
    if (threadIdx.x == 0) block_result = best;
    cluster.sync();
    if (part == 0 && threadIdx.x == 0) {
        Best total = block_result;
        for (int r = 1; r < kArgmaxBlocks; ++r) total = better(total, *cluster.map_shared_rank(&block_result, r));
        out[blockIdx.y] = total.index == 0x7fffffff ? 0 : total.index;
    }
    cluster_leave_together();  // (the first block has read the others' results)
}

// The candidates (probability, id) in shared memory, unused entries (-1, max int): sorted by probability
// descending and id ascending (bitonic over the smallest power of two that holds k), cut at the shortest prefix whose mass
// reaches `nucleus` (crossing token included), then the inverse-CDF draw r = u * kept mass.
// `grown`: where the picked id is stored a second time (the end of the row's history), or null.
__device__ void sort_and_pick(float* sorted_p, int* sorted_id, int k, float nucleus, float u, int* out, int* grown) {
    const int tid = threadIdx.x;
    int span = 32;  // the candidates lie in the first k entries: a power of two that holds them is all that is sorted
    while (span < k) span <<= 1;
    for (int size = 2; size <= span; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int partner = tid ^ stride;
            if (partner > tid && partner < span) {
                const bool descending_block = (tid & size) == 0;
                const float pa = sorted_p[tid], pb = sorted_p[partner];
                const int ia = sorted_id[tid], ib = sorted_id[partner];
                const bool a_first = pa > pb || (pa == pb && ia < ib);
                if (a_first != descending_block) {
                    sorted_p[tid] = pb; sorted_p[partner] = pa;
                    sorted_id[tid] = ib; sorted_id[partner] = ia;
                }
            }
            __syncthreads();
        }
    }
    if (tid == 0) {
        float cumulative = 0.0f;
        int cutoff = k;
        for (int i = 0; i < k; ++i) {
            cumulative += sorted_p[i];
            if (cumulative >= nucleus) {
                cutoff = i + 1;
                break;
            }
        }
        const float target = u * cumulative;  // the kept mass: the same additions in the same order
        float acc = 0.0f;
        int pick = sorted_id[cutoff - 1];
        for (int i = 0; i < cutoff; ++i) {
            acc += sorted_p[i];
            if (acc >= target) {
                pick = sorted_id[i];
                break;
            }
        }
        *out = pick;
        if (grown) *grown = pick;
    }
}

__global__ void __launch_bounds__(kThreads)
sample_rows_kernel(const float* __restrict__ logits, int row_stride, int vocab, float* __restrict__ work,
                   int* __restrict__ counts, const float* __restrict__ temperature, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, const float* __restrict__ penalty,
                   const int* __restrict__ history, int history_stride, const long long* __restrict__ history_rows, int append,
                   const int* __restrict__ history_len,
                   const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
                   const float* __restrict__ uniforms, int* __restrict__ out) {
    __shared__ Best best_scratch[32];
    __shared__ float float_scratch[32];
    __shared__ int int_scratch[32];
    __shared__ int histogram[256];
    __shared__ float sorted_p[kMaxSorted];
    __shared__ int sorted_id[kMaxSorted];
    __shared__ int shared_int[4];

    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    float* w = work + (size_t)r * vocab;
    const float temp = temperature[r];
    const float pen = penalty[r];
    // the row's earlier tokens: a row of the `history` matrix, or the array whose address history_rows[r] holds (0: none)
    int* h_row = history_rows ? reinterpret_cast<int*>(history_rows[r])
                              : (history ? const_cast<int*>(history) + (size_t)r * history_stride : nullptr);
    const bool penalised = pen > 1.0f && h_row && history_len[r] > 0;

    if (penalised) {
        int* cnt = counts + (size_t)r * vocab;
        for (int i = tid; i < vocab; i += kThreads) cnt[i] = 0;
        __syncthreads();
        const int* h = h_row;
        for (int j = tid; j < history_len[r]; j += kThreads) {
            const int token = h[j];
            if (token >= 0 && token < vocab) atomicAdd(&cnt[token], 1);
        }
        __syncthreads();
    }

    // adjusted logits, and their first maximum
    Best mine = {-CUDART_INF_F, 0x7fffffff};
    for (int i = tid; i < vocab; i += kThreads) {
        float v = row[i];
        if (penalised) {
            const int c = counts[(size_t)r * vocab + i];
            for (int n = 0; n < c; ++n) v = v > 0.0f ? v / pen : v * pen;
        }
        if (temp > 0.0f) v = v / temp;
        w[i] = v;
        if (v > mine.value) mine = {v, i};
    }
    const Best top = block_best(mine, best_scratch);
    if (temp <= 0.0f) {
        if (tid == 0) {
            const int token = top.index == 0x7fffffff ? 0 : top.index;
            out[r] = token;
            if (append && h_row) h_row[history_len[r]] = token;  // the row's history grows on the device
        }
        return;
    }

    // softmax over the whole vocabulary
    float local = 0.0f;
    for (int i = tid; i < vocab; i += kThreads) {
        const float e = expf(w[i] - top.value);
        w[i] = e;
        local += e;
    }
    const float sum = block_sum(local, float_scratch);
    for (int i = tid; i < vocab; i += kThreads) w[i] = w[i] / sum;
    __syncthreads();

    const float u = uniforms ? uniforms[r] : philox_uniform(seeds[r], counters[r]);
    int k = top_k[r];
    if (k <= 0 || k > vocab) k = vocab;
    const float nucleus = top_p[r];

    // k-th largest probability by radix select over the float bit patterns (all are >= 0)
    uint32_t kth_bits = 0;
    int need_ties = 0, tie_count = 0;
    if (k < vocab) {
        uint32_t prefix = 0, mask = 0;
        int remaining = k;
        for (int pass = 3; pass >= 0; --pass) {
            const int shift = pass * 8;
            if (tid < 256) histogram[tid] = 0;
            __syncthreads();
            for (int i = tid; i < vocab; i += kThreads) {
                const uint32_t key = __float_as_uint(w[i]);
                if ((key & mask) == prefix) atomicAdd(&histogram[(key >> shift) & 255u], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int cumulative = 0, digit = 0;
                for (int b = 255; b >= 0; --b) {
                    if (cumulative + histogram[b] >= remaining) {
                        digit = b;
                        break;
                    }
                    cumulative += histogram[b];
                }
                shared_int[0] = digit;
                shared_int[1] = remaining - cumulative;
                shared_int[2] = histogram[digit];
            }
            __syncthreads();
            prefix |= (uint32_t)shared_int[0] << shift;
            mask |= 255u << shift;
            remaining = shared_int[1];
            tie_count = shared_int[2];
            __syncthreads();
        }
        kth_bits = prefix;
        need_ties = remaining;
    }

    if (k <= kMaxSorted) {
        // gather the k candidates, sort them (probability descending, id ascending), walk them
        if (tid == 0) shared_int[3] = 0;
        for (int i = tid; i < kMaxSorted; i += kThreads) {
            sorted_p[i] = -1.0f;
            sorted_id[i] = 0x7fffffff;
        }
        __syncthreads();
        const bool all_ties = (k == vocab) || tie_count == need_ties;
        for (int i = tid; i < vocab; i += kThreads) {
            const uint32_t key = __float_as_uint(w[i]);
            if (k == vocab || key > kth_bits || (all_ties && key == kth_bits)) {
                const int at = atomicAdd(&shared_int[3], 1);
                sorted_p[at] = w[i];
                sorted_id[at] = i;
            }
        }
        __syncthreads();
        if (!all_ties) {
            // more tokens tie at the k-th probability than fit: the lower ids go in
            int taken = 0;
            const int base_count = shared_int[3];
            for (int base = 0; base < vocab && taken < need_ties; base += kThreads) {
                const int i = base + tid;
                const bool tie = i < vocab && __float_as_uint(w[i]) == kth_bits;
                int chunk_total;
                const int rank = taken + block_flag_scan(tie, int_scratch, &chunk_total);
                if (tie && rank < need_ties) {
                    sorted_p[base_count + rank] = w[i];
                    sorted_id[base_count + rank] = i;
                }
                taken += chunk_total;
            }
            __syncthreads();
        }
        sort_and_pick(sorted_p, sorted_id, k, nucleus, u, out + r, (append && h_row) ? h_row + history_len[r] : nullptr);
        return;
    }

    // More than kMaxSorted candidates (the host admits this only with top_p == 1): the draw walks
    // the kept tokens in id order, which draws from the same distribution.
    float kept_local = 0.0f;
    {
        // ties at the k-th probability: the first need_ties ids are kept; find the id bound
        int tie_bound = vocab;  // ids < tie_bound that tie are kept
        if (k < vocab && tie_count != need_ties) {
            int taken = 0;
            tie_bound = 0;
            for (int base = 0; base < vocab && taken < need_ties; base += kThreads) {
                const int i = base + tid;
                const bool tie = i < vocab && __float_as_uint(w[i]) == kth_bits;
                int chunk_total;
                const int rank = taken + block_flag_scan(tie, int_scratch, &chunk_total);
                if (tie && rank == need_ties - 1) shared_int[3] = i + 1;
                taken += chunk_total;
            }
            __syncthreads();
            tie_bound = shared_int[3];
        }
        for (int i = tid; i < vocab; i += kThreads) {
            const uint32_t key = __float_as_uint(w[i]);
            const bool kept = k == vocab || key > kth_bits || (key == kth_bits && i < tie_bound);
            if (!kept) w[i] = 0.0f;
            kept_local += w[i];
        }
    }
    const float total = block_sum(kept_local, float_scratch);
    const float target = u * total;
    if (tid == 0) {
        shared_int[1] = 0x7fffffff;  // lowest id whose running mass reaches the target
        shared_int[2] = -1;          // highest kept id, taken if rounding leaves the target unreached
    }
    __syncthreads();
    int last_kept = -1;
    for (int i = tid; i < vocab; i += kThreads)
        if (w[i] > 0.0f) last_kept = i;
    if (last_kept >= 0) atomicMax(&shared_int[2], last_kept);
    float running = 0.0f;
    for (int base = 0; base < vocab; base += kThreads) {
        const int i = base + tid;
        const float v = i < vocab ? w[i] : 0.0f;
        float chunk_total;
        const float inclusive = running + block_float_scan(v, float_scratch, &chunk_total);
        if (v > 0.0f && inclusive >= target) atomicMin(&shared_int[1], i);
        running += chunk_total;  // the same value in every thread
        if (running >= target) break;
    }
    __syncthreads();
    if (tid == 0) {
        const int token = shared_int[1] != 0x7fffffff ? shared_int[1] : (shared_int[2] >= 0 ? shared_int[2] : 0);
        out[r] = token;
        if (append && h_row) h_row[history_len[r]] = token;
    }
}


// The same pipeline for rows with at most kMaxSorted candidates, with the row spread over a cluster of
// kSampleBlocks blocks: block b owns the ids [b * slice, (b + 1) * slice).  Every pass over the vocabulary
// runs on all blocks at once; maxima, sums and the radix histograms meet through distributed shared memory
// (always added in block order, so the result does not depend on timing); the candidates are gathered into
// the first block's shared memory, which sorts them and draws.  grid (kSampleBlocks, rows).
constexpr int kSampleBlocks = 8;

__global__ void __launch_bounds__(kThreads)
sample_rows_cluster_kernel(const float* __restrict__ logits, int row_stride, int vocab, float* __restrict__ work,
                           int* __restrict__ counts, const float* __restrict__ temperature, const int* __restrict__ top_k,
                           const float* __restrict__ top_p, const float* __restrict__ penalty,
                           const int* __restrict__ history, int history_stride, const long long* __restrict__ history_rows, int append,
                   const int* __restrict__ history_len,
                           const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
                           const float* __restrict__ uniforms, int* __restrict__ out) {
    __shared__ Best best_scratch[32];
    __shared__ float float_scratch[32];
    __shared__ int int_scratch[32];
    __shared__ int histogram[256];      // of this block's ids
    __shared__ int histogram_all[256];  // of the whole row
    __shared__ float sorted_p[kMaxSorted];  // the candidates: filled and used in the cluster's first block only
    __shared__ int sorted_id[kMaxSorted];
    __shared__ Best slot_best;
    __shared__ float slot_sum;
    __shared__ int slot_ties;
    __shared__ int gathered;            // first block: candidates gathered so far
    __shared__ int shared_int[4];

    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int part = cluster.block_rank();
    const int r = blockIdx.y, tid = threadIdx.x;
    const int slice = (vocab + kSampleBlocks - 1) / kSampleBlocks;
    const int begin = min(vocab, part * slice), end = min(vocab, begin + slice);
    const float* row = logits + (size_t)r * row_stride;
    // the block's part of the row lives in shared memory from the first pass to the last: w[i] for begin <= i < end
    extern __shared__ float slice_values[];
    float* w = slice_values - begin;
    const float temp = temperature[r];
    const float pen = penalty[r];
    // the row's earlier tokens: a row of the `history` matrix, or the array whose address history_rows[r] holds (0: none)
    int* h_row = history_rows ? reinterpret_cast<int*>(history_rows[r])
                              : (history ? const_cast<int*>(history) + (size_t)r * history_stride : nullptr);
    const bool penalised = pen > 1.0f && h_row && history_len[r] > 0;

    if (part == 0) {
        if (tid == 0) gathered = 0;
        for (int i = tid; i < kMaxSorted; i += kThreads) {
            sorted_p[i] = -1.0f;
            sorted_id[i] = 0x7fffffff;
        }
    }
    if (penalised) {
        int* cnt = counts + (size_t)r * vocab;
        for (int i = begin + tid; i < end; i += kThreads) cnt[i] = 0;
        __threadfence();
        cluster.sync();
        const int* h = h_row;
        for (int j = part * kThreads + tid; j < history_len[r]; j += kSampleBlocks * kThreads) {
            const int token = h[j];
            if (token >= 0 && token < vocab) atomicAdd(&cnt[token], 1);
        }
        __threadfence();
        cluster.sync();
    }

    // adjusted logits, and their first maximum
    Best mine = {-CUDART_INF_F, 0x7fffffff};
    int scalar_from = begin;
    if (!penalised && !(begin & 3) && !((uintptr_t)row & 15)) {
        // four logits a load where the block's part starts on a 16-byte boundary (every thread still walks ascending ids,
        // so the first maximum stays the first)
        const int whole = begin + ((end - begin) & ~3);
        for (int i = begin + 4 * tid; i < whole; i += 4 * kThreads) {
            const float4 q = *reinterpret_cast<const float4*>(row + i);
            float v4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float v = temp > 0.0f ? v4[j] / temp : v4[j];
                w[i + j] = v;
                if (v > mine.value) mine = {v, i + j};
            }
        }
        scalar_from = whole;
    }
    for (int i = scalar_from + tid; i < end; i += kThreads) {
        float v = row[i];
        if (penalised) {
            const int c = counts[(size_t)r * vocab + i];
            for (int n = 0; n < c; ++n) v = v > 0.0f ? v / pen : v * pen;
        }
        if (temp > 0.0f) v = v / temp;
        w[i] = v;
        if (v > mine.value) mine = {v, i};
    }
    {
        const Best block = block_best(mine, best_scratch);
        if (tid == 0) slot_best = block;
    }
    cluster.sync();
    Best top = *cluster.map_shared_rank(&slot_best, 0);
    for (int b = 1; b < kSampleBlocks; ++b) top = better(top, *cluster.map_shared_rank(&slot_best, b));
    if (temp <= 0.0f) {
        if (part == 0 && tid == 0) {
            const int token = top.index == 0x7fffffff ? 0 : top.index;
            out[r] = token;
            if (append && h_row) h_row[history_len[r]] = token;
        }
        cluster.sync();  // nobody leaves while its shared memory may still be read
        return;
    }

    // softmax over the whole vocabulary
    float local = 0.0f;
    for (int i = begin + tid; i < end; i += kThreads) {
        const float e = expf(w[i] - top.value);
        w[i] = e;
        local += e;
    }
    {
        const float block = block_sum(local, float_scratch);
        if (tid == 0) slot_sum = block;
    }
    cluster.sync();
    float sum = 0.0f;
    for (int b = 0; b < kSampleBlocks; ++b) sum += *cluster.map_shared_rank(&slot_sum, b);
    for (int i = begin + tid; i < end; i += kThreads) w[i] = w[i] / sum;
    __syncthreads();

    const float u = uniforms ? uniforms[r] : philox_uniform(seeds[r], counters[r]);
    int k = top_k[r];
    if (k <= 0 || k > vocab) k = vocab;
    const float nucleus = top_p[r];

    if (k == vocab && nucleus >= 1.0f && vocab > kMaxSorted) {
        // Nothing is cut: the draw walks the whole vocabulary in id order (the same distribution as walking it by
        // probability).  The blocks' masses are added in block order; the block whose range holds the target walks
        // its ids, 1,024 at a time.
        float mass = 0.0f;
        for (int i = begin + tid; i < end; i += kThreads) mass += w[i];
        {
            const float block = block_sum(mass, float_scratch);
            __syncthreads();
            if (tid == 0) slot_sum = block;
        }
        cluster.sync();
        float prefix[kSampleBlocks + 1];
        prefix[0] = 0.0f;
        for (int b = 0; b < kSampleBlocks; ++b) prefix[b + 1] = prefix[b] + *cluster.map_shared_rank(&slot_sum, b);
        const float target = u * prefix[kSampleBlocks];
        int owner = 0;  // the first block whose range reaches the target; else the last block that has ids
        for (int b = 0; b < kSampleBlocks; ++b) {
            if (min(vocab, b * slice) >= min(vocab, (b + 1) * slice)) continue;  // no ids
            owner = b;
            if (prefix[b + 1] >= target) break;
        }
        const float before = prefix[owner];
        cluster.sync();  // every block has read every mass
        if (part != owner) return;
        if (tid == 0) {
            shared_int[1] = 0x7fffffff;  // lowest id whose running mass reaches the target
            shared_int[2] = -1;          // highest id with any mass, taken if rounding leaves the target unreached
        }
        __syncthreads();
        int last_kept = -1;
        for (int i = begin + tid; i < end; i += kThreads)
            if (w[i] > 0.0f) last_kept = i;
        if (last_kept >= 0) atomicMax(&shared_int[2], last_kept);
        // every thread takes a run of neighbouring ids; one scan over the runs' masses finds the run that holds
        // the target, and its thread walks it
        const int per_thread = (end - begin + kThreads - 1) / kThreads;
        const int first = min(end, begin + tid * per_thread), last = min(end, first + per_thread);
        float run_mass = 0.0f;
        for (int i = first; i < last; ++i) run_mass += w[i];
        float all_runs;
        const float inclusive = before + block_float_scan(run_mass, float_scratch, &all_runs);
        if (inclusive >= target) {  // this run or an earlier one holds the target: the lowest id that reaches it wins
            float running = inclusive - run_mass;
            for (int i = first; i < last; ++i) {
                running += w[i];
                if (w[i] > 0.0f && running >= target) {
                    atomicMin(&shared_int[1], i);
                    break;
                }
            }
        }
        __syncthreads();
        if (tid == 0) {
            const int token = shared_int[1] != 0x7fffffff ? shared_int[1] : (shared_int[2] >= 0 ? shared_int[2] : 0);
            out[r] = token;
            if (append && h_row) h_row[history_len[r]] = token;
        }
        return;
    }
    if (k > kMaxSorted) k = kMaxSorted;  // the host sends only rows that fit; never write past the arrays

    // k-th largest probability by radix select over the float bit patterns (all are >= 0)
    uint32_t kth_bits = 0;
    int need_ties = 0, tie_count = 0;
    int sort_span = 32;  // what sort_and_pick sorts for this k
    while (sort_span < k) sort_span <<= 1;
    if (k < vocab) {
        uint32_t prefix = 0, mask = 0;
        int remaining = k;
        for (int pass = 3; pass >= 0; --pass) {
            const int shift = pass * 8;
            if (tid < 256) histogram[tid] = 0;
            __syncthreads();
            for (int i = begin + tid; i < end; i += kThreads) {
                const uint32_t key = __float_as_uint(w[i]);
                const bool counted = (key & mask) == prefix;
                const uint32_t digit = (key >> shift) & 255u;
                // lanes with the same digit add once: most of a row shares its leading digits
                const unsigned peers = __match_any_sync(__activemask(), counted ? digit : 256u);
                if (counted && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&histogram[digit], __popc(peers));
            }
            cluster.sync();
            if (tid < 256) {
                int total = 0;
                for (int b = 0; b < kSampleBlocks; ++b) total += cluster.map_shared_rank(histogram, b)[tid];
                histogram_all[tid] = total;
            }
            __syncthreads();
            if (tid < 32) {
                // the digit at which the count from the top reaches `remaining`: lane l takes bins 255 - 8l down to
                // 248 - 8l, a scan over the lanes finds the lane, the lane finds the bin
                int bins[8], mine_total = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    bins[j] = histogram_all[255 - 8 * tid - j];
                    mine_total += bins[j];
                }
                int inclusive = mine_total;
#pragma unroll
                for (int offset = 1; offset < 32; offset <<= 1) {
                    const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
                    if (tid >= offset) inclusive += other;
                }
                const unsigned reached = __ballot_sync(0xffffffffu, inclusive >= remaining);
                const int lane_of_digit = reached ? __ffs(reached) - 1 : 31;
                if (tid == lane_of_digit) {
                    int cumulative = inclusive - mine_total, digit = 255 - 8 * tid - 7;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (cumulative + bins[j] >= remaining || j == 7) {
                            digit = 255 - 8 * tid - j;
                            break;
                        }
                        cumulative += bins[j];
                    }
                    shared_int[0] = digit;
                    shared_int[1] = remaining - cumulative;
                    shared_int[2] = histogram_all[digit];
                }
            }
            cluster.sync();  // every block has read every histogram before the next pass clears them
            prefix |= (uint32_t)shared_int[0] << shift;
            mask |= 255u << shift;
            remaining = shared_int[1];
            tie_count = shared_int[2];
            // Everything above the chosen digit is in for certain (k - remaining ids), and the digit's own ids number
            // tie_count.  If all of them together fit what the sort below takes anyway, the remaining passes are not
            // needed: all ids from the digit's lower bound up become candidates and the sort cuts at k.
            if (pass > 0 && k - remaining + tie_count <= sort_span) {
                remaining = tie_count;  // (all of the digit's ids are gathered: see `all_ties` below)
                break;
            }
        }
        kth_bits = prefix;
        need_ties = remaining;
    }

    // gather the candidates into the first block
    float* first_p = cluster.map_shared_rank(sorted_p, 0);
    int* first_id = cluster.map_shared_rank(sorted_id, 0);
    int* first_gathered = cluster.map_shared_rank(&gathered, 0);
    const bool all_ties = (k == vocab) || tie_count == need_ties;
    int my_ties = 0;
    for (int i = begin + tid; i < end; i += kThreads) {
        const uint32_t key = __float_as_uint(w[i]);
        if (k == vocab || key > kth_bits || (all_ties && key == kth_bits)) {
            const int at = atomicAdd(first_gathered, 1);
            if (at < kMaxSorted) {
                first_p[at] = w[i];
                first_id[at] = i;
            }
        } else if (key == kth_bits) {
            ++my_ties;
        }
    }
    if (!all_ties) {
        // more tokens tie at the k-th probability than fit: the lower ids go in.  Blocks own ascending id
        // ranges, so a block's ties rank after all ties of the blocks before it.
        __syncthreads();
        int_scratch[0] = 0;
        __syncthreads();
        if (my_ties) atomicAdd(&int_scratch[0], my_ties);
        __syncthreads();
        if (tid == 0) slot_ties = int_scratch[0];
        cluster.sync();  // all candidates above the k-th are in; the tie counts are known
        int taken = 0;
        for (int b = 0; b < part; ++b) taken += *cluster.map_shared_rank(&slot_ties, b);
        const int base_count = *first_gathered;
        for (int base = begin; base < end && taken < need_ties; base += kThreads) {
            const int i = base + tid;
            const bool tie = i < end && __float_as_uint(w[i]) == kth_bits;
            int chunk_total;
            const int rank = taken + block_flag_scan(tie, int_scratch, &chunk_total);
            if (tie && rank < need_ties && base_count + rank < kMaxSorted) {
                first_p[base_count + rank] = w[i];
                first_id[base_count + rank] = i;
            }
            taken += chunk_total;
        }
    }
    cluster.sync();  // the first block's arrays are complete; the others are done
    if (part != 0) return;
    sort_and_pick(sorted_p, sorted_id, k, nucleus, u, out + r, (append && h_row) ? h_row + history_len[r] : nullptr);
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_argmax_rows(const float* logits, int row_stride, int rows, int vocab, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || row_stride < vocab) return fail("argmax_rows: vocab %d, row stride %d", vocab, row_stride);
    if (rows > 65535) return fail("argmax_rows: %d rows exceed the grid limit 65535", rows);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(kArgmaxBlocks, rows);
    config.blockDim = dim3(kThreads);
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = kArgmaxBlocks;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent_launches_allowed() ? 2 : 1;
    cudaError_t status = cudaLaunchKernelEx(&config, argmax_rows_kernel, logits, row_stride, vocab, out);
    if (status != cudaSuccess) return fail("argmax_rows: launch failed: %s", cudaGetErrorString(status));
    return check_launch("argmax_rows");
}

// Per-row arrays live on the device.  `uniforms` (optional) overrides the generator, for tests.
// The host guarantees top_p == 1 for rows whose candidate count (top_k, or the vocabulary when
// top_k <= 0) exceeds `mb_sample_max_sorted()`.
// max_candidates: the host's bound on min(top_k, vocab) over the rows that cut anything (a row with top_k >= vocab and
// top_p >= 1 cuts nothing and does not count); 0: unknown.  When it is at most mb_sample_max_sorted(), the rows take the
// kernel that spreads a row over a cluster of blocks.
MB_EXPORT int mb_sample_rows(const float* logits, int row_stride, int rows, int vocab, float* work, int* counts,
                             const float* temperature, const int* top_k, const float* top_p, const float* penalty,
                             const int* history, int history_stride, const long long* history_rows, int append, const int* history_len,
                             const unsigned long long* seeds, const unsigned long long* counters,
                             const float* uniforms, int* out, int max_candidates, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || row_stride < vocab) return fail("sample_rows: vocab %d, row stride %d", vocab, row_stride);
    if (!work) return fail("sample_rows: needs rows * vocab floats of scratch");
    if (!uniforms && (!seeds || !counters)) return fail("sample_rows: needs seeds and counters, or uniforms");
    // a block of the cluster kernel keeps its eighth of a row in shared memory; a vocabulary too large for that (more
    // than 400,000 ids) takes the kernel that works in the scratch array
    const size_t slice_bytes = (size_t)((vocab + kSampleBlocks - 1) / kSampleBlocks) * sizeof(float);
    if (max_candidates > 0 && max_candidates <= kMaxSorted && slice_bytes <= 200 * 1024) {
        static size_t reserved = 0;
        if (slice_bytes > reserved) {
            cudaError_t status = cudaFuncSetAttribute(sample_rows_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)slice_bytes);
            if (status != cudaSuccess) return fail("sample_rows: cannot reserve %zu bytes of shared memory: %s", slice_bytes, cudaGetErrorString(status));
            reserved = slice_bytes;
        }
        if (rows > 65535) return fail("sample_rows: %d rows exceed the grid limit 65535", rows);
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(kSampleBlocks, rows);
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = slice_bytes;
        config.stream = stream;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = kSampleBlocks;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        cudaError_t status = cudaLaunchKernelEx(&config, sample_rows_cluster_kernel, logits, row_stride, vocab, work, counts,
                                                temperature, top_k, top_p, penalty, history, history_stride, history_rows, append, history_len, seeds,
                                                counters, uniforms, out);
        if (status != cudaSuccess) return fail("sample_rows: launch failed: %s", cudaGetErrorString(status));
        return check_launch("sample_rows");
    }
    sample_rows_kernel<<<rows, kThreads, 0, stream>>>(logits, row_stride, vocab, work, counts, temperature, top_k, top_p,
                                                      penalty, history, history_stride, history_rows, append, history_len, seeds, counters,
                                                      uniforms, out);
    return check_launch("sample_rows");
}

MB_EXPORT int mb_sample_max_sorted() { return kMaxSorted; }
