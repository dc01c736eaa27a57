// Row-wise and element-wise kernels of the decoder: embedding gather, residual add fused with
// RMSNorm, rotary position encoding fused with the cache write, the gated activation and bias add.
// Each is instantiated for float and bfloat16 storage; all arithmetic is float.
//
// Formulas follow integrallis/models (paths inside that project):
//   RMSNorm    backend-java/.../ops/TensorOps.java:45-58
//   rotation   backend-java/.../ops/TensorOps.java:1474-1486 (pair rotation), RotaryTable.java:177-186
//   SwiGLU     backend-java/.../ops/TensorOps.java:1407-1425
//   cache write after rotation, values unrotated: backend-java/.../llama/LlamaForwardPass.java:1070-1086
#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

// ------------------------------------------------------------------------------------ embedding

template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ out, int width, int vocab, float scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int row = blockIdx.x;
    int token = tokens[row];
    token = token < 0 ? 0 : (token >= vocab ? vocab - 1 : token);  // ids are validated on the host
    const TW* src = table + (size_t)token * width;
    float* dst = out + (size_t)row * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) dst[d] = Num<TW>::load(src + d) * scale;
}

// ------------------------------------------------------------------------------------ add + RMSNorm

// One block per output row.  x is the float residual stream.  With `delta` the sum x + delta is
// formed in float; it is written back to x when write_x is set.  `rows` (optional) picks input rows.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps, int write_x) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ float row_cache[];  // the row, width floats
    __shared__ float scratch[32];
    const int out_row = blockIdx.x;
    const int in_row = rows ? rows[out_row] : out_row;
    float* xr = x + (size_t)in_row * width;
    const TD* dr = delta ? delta + (size_t)in_row * width : nullptr;
    float sum_sq = 0.0f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float v = xr[d];
        if (dr) {
            v += Num<TD>::load(dr + d);
            if (write_x) xr[d] = v;
        }
        row_cache[d] = v;
        sum_sq += v * v;
    }
    sum_sq = block_sum(sum_sq, scratch);
    const float rms = sqrtf(sum_sq / (float)width + eps);
    const float scale = 1.0f / rms;
    TO* o = out + (size_t)out_row * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) Num<TO>::store(o + d, row_cache[d] * scale * weight[d]);
}

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                       __uint_as_float(raw.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

// The same with four elements per thread and step; width a multiple of 4, rows 16-byte aligned.
template <typename TD, typename TO>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                        const float* __restrict__ weight, TO* __restrict__ out,
                                        const int* __restrict__ rows, int width, float eps, int write_x) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ float row_cache[];
    __shared__ float scratch[32];
    const int out_row = blockIdx.x;
    const int in_row = rows ? rows[out_row] : out_row;
    float* xr = x + (size_t)in_row * width;
    const TD* dr = delta ? delta + (size_t)in_row * width : nullptr;
    float sum_sq = 0.0f;
    for (int d = threadIdx.x * 4; d < width; d += blockDim.x * 4) {
        float4 v = load4(xr + d);
        if (dr) {
            const float4 e = load4(dr + d);
            v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
            if (write_x) store4(xr + d, v);
        }
        store4(row_cache + d, v);
        sum_sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    sum_sq = block_sum(sum_sq, scratch);
    const float rms = sqrtf(sum_sq / (float)width + eps);
    const float scale = 1.0f / rms;
    TO* o = out + (size_t)out_row * width;
    for (int d = threadIdx.x * 4; d < width; d += blockDim.x * 4) {
        const float4 v = load4(row_cache + d), w = load4(weight + d);
        store4(o + d, make_float4(v.x * scale * w.x, v.y * scale * w.y, v.z * scale * w.z, v.w * scale * w.w));
    }
}

// Many rows (a prompt's): one warp per row and the row in registers, kVec groups of four elements per lane.  All of a
// row's loads are in flight at once and nothing waits at a block barrier; with one block per row a step of 2,048
// rows of 2,048 spent most of its time between its two passes.  width <= 128 * kVec.
template <typename TD, typename TO, int kVec>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ x, const TD* __restrict__ delta, const float* __restrict__ weight,
                        TO* __restrict__ out, const int* __restrict__ rows, int out_rows, int width, float eps, int write_x) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int out_row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (out_row >= out_rows) return;
    const int in_row = rows ? rows[out_row] : out_row;
    float* xr = x + (size_t)in_row * width;
    const TD* dr = delta ? delta + (size_t)in_row * width : nullptr;
    float4 v[kVec];
    float sum_sq = 0.0f;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
        const int d = (i * 32 + lane) * 4;
        v[i] = d < width ? load4(xr + d) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (dr) {
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
            const int d = (i * 32 + lane) * 4;
            if (d < width) {
                const float4 e = load4(dr + d);
                v[i].x += e.x; v[i].y += e.y; v[i].z += e.z; v[i].w += e.w;
                if (write_x) store4(xr + d, v[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kVec; ++i) sum_sq += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    sum_sq = warp_sum(sum_sq);
    const float rms = sqrtf(sum_sq / (float)width + eps);
    const float scale = 1.0f / rms;
    TO* o = out + (size_t)out_row * width;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
        const int d = (i * 32 + lane) * 4;
        if (d < width) {
            const float4 w = load4(weight + d);
            store4(o + d, make_float4(v[i].x * scale * w.x, v[i].y * scale * w.y, v[i].z * scale * w.z, v[i].w * scale * w.w));
        }
    }
}

// ------------------------------------------------------------------------------------ rotary + cache

// grid (tokens, heads + 2*kv_heads).  Query heads are rotated in place; key heads are rotated and
// written to the cache; value heads are copied to the cache.  slot_mapping[t] is the flat position
// (page * page_size + offset) of token t in this layer's pools, or < 0 for a row that is padding.
template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                        const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                        T* __restrict__ k_pool, T* __restrict__ v_pool,
                                        const int* __restrict__ slot_mapping, int heads, int kv_heads, int head_dim,
                                        int rotary_dim, int interleaved, int page_size, int write_cache) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const int h = blockIdx.y;
    T* vec = qkv + (size_t)t * row_stride + (size_t)h * head_dim;
    const bool is_query = h < heads;
    const bool is_key = !is_query && h < heads + kv_heads;
    T* dst = nullptr;
    if (!is_query) {
        if (!write_cache) return;
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const int kvh = is_key ? h - heads : h - heads - kv_heads;
        const size_t page = slot / page_size, offset = slot % page_size;
        dst = (is_key ? k_pool : v_pool) + ((page * kv_heads + kvh) * page_size + offset) * head_dim;
    }
    if (is_query || is_key) {
        const int pairs = rotary_dim / 2;
        const int pos = positions[t];
        const float* c = cos_table + (size_t)pos * pairs;
        const float* s = sin_table + (size_t)pos * pairs;
        for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
            const int i0 = interleaved ? 2 * i : i;
            const int i1 = interleaved ? 2 * i + 1 : i + pairs;
            const float x0 = Num<T>::load(vec + i0), x1 = Num<T>::load(vec + i1);
            const float r0 = x0 * c[i] - x1 * s[i];
            const float r1 = x0 * s[i] + x1 * c[i];
            if (is_query) {
                Num<T>::store(vec + i0, r0);
                Num<T>::store(vec + i1, r1);
            } else {
                Num<T>::store(dst + i0, r0);
                Num<T>::store(dst + i1, r1);
            }
        }
        if (is_key)
            for (int d = rotary_dim + threadIdx.x; d < head_dim; d += blockDim.x) dst[d] = vec[d];
    } else {
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x) dst[d] = vec[d];
    }
}

// The common case -- split-half pairs over the whole head, head size a multiple of 16 -- eight
// elements per thread: grid (tokens), a block walks the (head, eighth-of-a-half) items of its token.
template <typename T>
__global__ void rope_cache_write_vec8_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                             const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                             T* __restrict__ k_pool, T* __restrict__ v_pool,
                                             const int* __restrict__ slot_mapping, int heads, int kv_heads, int head_dim,
                                             int page_size, int write_cache) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const int half = head_dim / 2, pieces = half / 8;  // pieces of 8 pairs per head
    const int pos = positions[t];
    const float* c = cos_table + (size_t)pos * half;
    const float* s = sin_table + (size_t)pos * half;
    const int slot = write_cache ? slot_mapping[t] : -1;
    const size_t page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot % page_size : 0;
    T* row = qkv + (size_t)t * row_stride;
    const int rotated_heads = write_cache ? heads + kv_heads : heads;
    const int rotate_items = rotated_heads * pieces;
    const int copy_items = write_cache ? kv_heads * (head_dim / 8) : 0;
    for (int item = threadIdx.x; item < rotate_items + copy_items; item += blockDim.x) {
        if (item < rotate_items) {
            const int h = item / pieces, piece = item % pieces;
            T* vec = row + (size_t)h * head_dim + piece * 8;
            float x0[8], x1[8], cs[8], sn[8], r0[8], r1[8];
            load8(vec, x0);
            load8(vec + half, x1);
            load8(c + piece * 8, cs);
            load8(s + piece * 8, sn);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                r0[i] = x0[i] * cs[i] - x1[i] * sn[i];
                r1[i] = x0[i] * sn[i] + x1[i] * cs[i];
            }
            T* dst = vec;
            if (h >= heads) {
                if (slot < 0) continue;
                dst = k_pool + ((page * kv_heads + (h - heads)) * page_size + offset) * head_dim + piece * 8;
            }
            store8(dst, r0);
            store8(dst + half, r1);
        } else {
            if (slot < 0) continue;
            const int copy = item - rotate_items;
            const int h = copy / (head_dim / 8), piece = copy % (head_dim / 8);
            float v[8];
            load8(row + (size_t)(heads + kv_heads + h) * head_dim + piece * 8, v);
            store8(v_pool + ((page * kv_heads + h) * page_size + offset) * head_dim + piece * 8, v);
        }
    }
}

// ------------------------------------------------------------------------------------ logits

__global__ void logit_epilogue_kernel(float* __restrict__ logits, int ld, int vocab, size_t total, float scale, float softcap) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float* at = logits + (i / vocab) * ld + (i % vocab);
        float value = *at * scale;
        if (softcap != 0.0f) value = softcap * tanhf(value / softcap);
        *at = value;
    }
}

// ------------------------------------------------------------------------------------ gated activation

// gate_up: [rows, 2*width] with the gate in columns [0, width) and up in [width, 2*width).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int width, size_t total, int activation) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t row = i / width, col = i % width;
        const float g = Num<T>::load(gate_up + row * 2 * width + col);
        const float u = Num<T>::load(gate_up + row * 2 * width + width + col);
        Num<T>::store(out + i, gate_activation(activation, g) * u);
    }
}

// Eight elements per thread; width a multiple of 8, rows 16-byte (bf16) or 32-byte (float) aligned.
template <typename T>
__global__ void swiglu_vec8_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int width, size_t total8, int activation) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int per_row = width / 8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += stride) {
        const size_t row = i / per_row, col = (i % per_row) * 8;
        float g[8], u[8], r[8];
        load8(gate_up + row * 2 * width + col, g);
        load8(gate_up + row * 2 * width + width + col, u);
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = gate_activation(activation, g[j]) * u[j];
        store8(out + row * width + col, r);
    }
}

template <typename T>
__global__ void bias_add_kernel(T* __restrict__ x, const float* __restrict__ bias, int width, size_t total) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
        Num<T>::store(x + i, Num<T>::load(x + i) + bias[i % width]);
}

// x (float residual) += delta
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t total) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
        x[i] += Num<TD>::load(delta + i);
}

inline int grid_for(size_t total, int block) {
    size_t blocks = (total + block - 1) / block;
    return (int)(blocks > 148 * 16 ? 148 * 16 : (blocks ? blocks : 1));
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_embed_gather(const void* table, int table_dtype, const int* tokens, float* out, int rows, int width,
                              int vocab, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || vocab <= 0) return fail("embed_gather: width %d and vocab %d must be positive", width, vocab);
    const int block = width >= 1024 ? 256 : 128;
    // the first kernel of a step follows a copy, not a kernel: an ordinary launch
    if (table_dtype == MB_F32)
        embed_gather_kernel<float><<<rows, block, 0, stream>>>((const float*)table, tokens, out, width, vocab, scale);
    else if (table_dtype == MB_BF16)
        embed_gather_kernel<__nv_bfloat16><<<rows, block, 0, stream>>>((const __nv_bfloat16*)table, tokens, out, width, vocab, scale);
    else
        return fail("embed_gather: unknown dtype code %d", table_dtype);
    return check_launch("embed_gather");
}

constexpr int kRowsPerWarpFrom = 256;  // from so many rows on, a warp per row (add_rmsnorm_rows_kernel)

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* x, const void* delta, const float* weight, void* out, const int* rows,
                              int out_rows, int width, float eps, int write_x, cudaStream_t stream) {
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return fail("add_rmsnorm: a row of %d floats does not fit shared memory (limit 51200)", width);
    auto kernel = add_rmsnorm_kernel<TD, TO>;
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("add_rmsnorm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
    }
    const int block = width >= 4096 ? 512 : (width >= 1024 ? 256 : 128);
    const bool aligned = width % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)delta & 7) && !((uintptr_t)weight & 15) &&
                         !((uintptr_t)out & 7);
    if (aligned && out_rows >= kRowsPerWarpFrom && width <= 4096) {
        const int warps = out_rows >= 2048 ? 8 : (out_rows >= 1024 ? 4 : 2);  // a few hundred rows: smaller blocks, so that every multiprocessor has some
        const int grid = (out_rows + warps - 1) / warps;
#define MB_ROWS_KERNEL(kVec)                                                                                              \
    return launch_dependent("add_rmsnorm", add_rmsnorm_rows_kernel<TD, TO, kVec>, dim3(grid), dim3(32 * warps), 0, stream, \
                            true, x, (const TD*)delta, weight, (TO*)out, rows, out_rows, width, eps, write_x)
        if (width <= 512) MB_ROWS_KERNEL(4);
        if (width <= 1024) MB_ROWS_KERNEL(8);
        if (width <= 2048) MB_ROWS_KERNEL(16);
        MB_ROWS_KERNEL(32);
#undef MB_ROWS_KERNEL
    }
    if (aligned) {
        auto vec = add_rmsnorm_vec4_kernel<TD, TO>;
        if (smem > 48 * 1024) {
            cudaError_t status = cudaFuncSetAttribute(vec, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (status != cudaSuccess) return fail("add_rmsnorm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
        }
        return launch_dependent("add_rmsnorm", vec, dim3(out_rows), dim3(block), smem, stream, true, x, (const TD*)delta, weight,
                                (TO*)out, rows, width, eps, write_x);
    }
    return launch_dependent("add_rmsnorm", kernel, dim3(out_rows), dim3(block), smem, stream, true, x, (const TD*)delta, weight,
                            (TO*)out, rows, width, eps, write_x);
}

// delta may be null (then delta_dtype is ignored).  out_dtype selects the storage of `out`.
MB_EXPORT int mb_add_rmsnorm(float* x, const void* delta, int delta_dtype, const float* weight, void* out,
                             int out_dtype, const int* rows, int out_rows, int width, float eps, int write_x,
                             cudaStream_t stream) {
    if (out_rows <= 0) return 0;
    if (width <= 0) return fail("add_rmsnorm: width %d must be positive", width);
    if (!delta) delta_dtype = out_dtype;
    if (delta_dtype == MB_F32 && out_dtype == MB_F32)
        return launch_add_rmsnorm<float, float>(x, delta, weight, out, rows, out_rows, width, eps, write_x, stream);
    if (delta_dtype == MB_BF16 && out_dtype == MB_BF16)
        return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(x, delta, weight, out, rows, out_rows, width, eps, write_x, stream);
    if (delta_dtype == MB_F32 && out_dtype == MB_BF16)
        return launch_add_rmsnorm<float, __nv_bfloat16>(x, delta, weight, out, rows, out_rows, width, eps, write_x, stream);
    if (delta_dtype == MB_BF16 && out_dtype == MB_F32)
        return launch_add_rmsnorm<__nv_bfloat16, float>(x, delta, weight, out, rows, out_rows, width, eps, write_x, stream);
    return fail("add_rmsnorm: unknown dtype codes %d, %d", delta_dtype, out_dtype);
}

MB_EXPORT int mb_rope_cache_write(void* qkv, int dtype, int row_stride, const int* positions, const float* cos_table,
                                  const float* sin_table, void* k_pool, void* v_pool, const int* slot_mapping,
                                  int tokens, int heads, int kv_heads, int head_dim, int rotary_dim, int interleaved,
                                  int page_size, int write_cache, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
        return fail("rope_cache_write: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    if (rotary_dim > 0 && (!cos_table || !sin_table || !positions))
        return fail("rope_cache_write: a rotation needs positions and cos/sin tables");
    if (write_cache && (!k_pool || !v_pool || !slot_mapping || page_size <= 0))
        return fail("rope_cache_write: a cache write needs pools, a slot mapping and a page size");
    const bool wide = !interleaved && rotary_dim == head_dim && head_dim % 16 == 0 && row_stride % 8 == 0 &&
                      !((uintptr_t)qkv & 31) && !((uintptr_t)k_pool & 31) && !((uintptr_t)v_pool & 31) &&
                      !((uintptr_t)cos_table & 31) && !((uintptr_t)sin_table & 31);
    if (wide) {
        const int items = (heads + kv_heads) * (head_dim / 16) + kv_heads * (head_dim / 8);
        const int threads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
        if (dtype == MB_F32)
            return launch_dependent("rope_cache_write", rope_cache_write_vec8_kernel<float>, dim3(tokens), dim3(threads), 0, stream,
                                    true, (float*)qkv, row_stride, positions, cos_table, sin_table, (float*)k_pool, (float*)v_pool,
                                    slot_mapping, heads, kv_heads, head_dim, page_size, write_cache);
        if (dtype == MB_BF16)
            return launch_dependent("rope_cache_write", rope_cache_write_vec8_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0,
                                    stream, true, (__nv_bfloat16*)qkv, row_stride, positions, cos_table, sin_table,
                                    (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, slot_mapping, heads, kv_heads, head_dim,
                                    page_size, write_cache);
        return fail("rope_cache_write: unknown dtype code %d", dtype);
    }
    const dim3 grid(tokens, write_cache ? heads + 2 * kv_heads : heads);
    const int block = head_dim >= 128 ? 64 : 32;
    if (dtype == MB_F32)
        return launch_dependent("rope_cache_write", rope_cache_write_kernel<float>, grid, dim3(block), 0, stream, true, (float*)qkv,
                                row_stride, positions, cos_table, sin_table, (float*)k_pool, (float*)v_pool, slot_mapping, heads,
                                kv_heads, head_dim, rotary_dim, interleaved, page_size, write_cache);
    if (dtype == MB_BF16)
        return launch_dependent("rope_cache_write", rope_cache_write_kernel<__nv_bfloat16>, grid, dim3(block), 0, stream, true,
                                (__nv_bfloat16*)qkv, row_stride, positions, cos_table, sin_table, (__nv_bfloat16*)k_pool,
                                (__nv_bfloat16*)v_pool, slot_mapping, heads, kv_heads, head_dim, rotary_dim, interleaved, page_size,
                                write_cache);
    return fail("rope_cache_write: unknown dtype code %d", dtype);
}

// out [rows, width] = act(gate) * up for gate_up [rows, 2 * width]; activation: MB_ACT_*.
MB_EXPORT int mb_swiglu(const void* gate_up, void* out, int dtype, int rows, int width, int activation, cudaStream_t stream) {
    const size_t total = (size_t)rows * width;
    if (total == 0) return 0;
    if (activation < 0 || activation >= MB_ACT_COUNT) return fail("swiglu: unknown gate activation code %d", activation);
    if (width % 8 == 0 && !((uintptr_t)gate_up & 31) && !((uintptr_t)out & 31)) {
        const size_t total8 = total / 8;
        const size_t blocks = (total8 + 255) / 256;
        const int grid = (int)(blocks > 148 * 32 ? 148 * 32 : blocks);
        if (dtype == MB_F32)
            return launch_dependent("swiglu", swiglu_vec8_kernel<float>, dim3(grid), dim3(256), 0, stream, true, (const float*)gate_up,
                                    (float*)out, width, total8, activation);
        if (dtype == MB_BF16)
            return launch_dependent("swiglu", swiglu_vec8_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, true,
                                    (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, width, total8, activation);
        return fail("swiglu: unknown dtype code %d", dtype);
    }
    if (dtype == MB_F32)
        swiglu_kernel<float><<<grid_for(total, 256), 256, 0, stream>>>((const float*)gate_up, (float*)out, width, total, activation);
    else if (dtype == MB_BF16)
        swiglu_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, width, total, activation);
    else
        return fail("swiglu: unknown dtype code %d", dtype);
    return check_launch("swiglu");
}

// logits = logits * scale; with softcap c != 0 then c * tanh(logits / c)
// (integrallis/models, backend-java/.../llama/LlamaForwardPass.java:1751-1764).  In place, float32.
MB_EXPORT int mb_logit_epilogue(float* logits, int ld, int rows, int vocab, float scale, float softcap, cudaStream_t stream) {
    const size_t total = (size_t)rows * vocab;
    if (total == 0) return 0;
    logit_epilogue_kernel<<<grid_for(total, 256), 256, 0, stream>>>(logits, ld, vocab, total, scale, softcap);
    return check_launch("logit_epilogue");
}

MB_EXPORT int mb_bias_add(void* x, int dtype, const float* bias, int rows, int width, cudaStream_t stream) {
    const size_t total = (size_t)rows * width;
    if (total == 0) return 0;
    if (dtype == MB_F32)
        bias_add_kernel<float><<<grid_for(total, 256), 256, 0, stream>>>((float*)x, bias, width, total);
    else if (dtype == MB_BF16)
        bias_add_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, stream>>>((__nv_bfloat16*)x, bias, width, total);
    else
        return fail("bias_add: unknown dtype code %d", dtype);
    return check_launch("bias_add");
}

MB_EXPORT int mb_residual_add(float* x, const void* delta, int delta_dtype, size_t total, cudaStream_t stream) {
    if (total == 0) return 0;
    if (delta_dtype == MB_F32)
        residual_add_kernel<float><<<grid_for(total, 256), 256, 0, stream>>>(x, (const float*)delta, total);
    else if (delta_dtype == MB_BF16)
        residual_add_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, stream>>>(x, (const __nv_bfloat16*)delta, total);
    else
        return fail("residual_add: unknown dtype code %d", delta_dtype);
    return check_launch("residual_add");
}
