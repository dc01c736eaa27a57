// Shared helpers of every kernel library of this package: the exported-symbol macro, the
// per-library error message, storage-type conversion and block reductions with a fixed order.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define MB_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes that cross the C boundary
#define MB_F32 0
#define MB_BF16 1

// Gate activations of a gated feed-forward.  A launcher takes the code in bits 8 and up of its
// epilogue argument (0, the default, is SiLU).
#define MB_ACT_SILU 0
#define MB_ACT_GELU_TANH 1
#define MB_ACT_COUNT 2

namespace mb {

// act(gate): silu(z) = z / (1 + exp(-z)) (integrallis/models, backend-java/.../ops/TensorOps.java:1407-1425);
// gelu_tanh(z) = 0.5 z (1 + tanh(0.7978845608 z (1 + 0.044715 z^2))) (:1427-1449).  `activation` is the
// same for every thread of a launch, so the branch does not diverge.
__device__ __forceinline__ float gate_activation(int activation, float z) {
    if (activation == MB_ACT_GELU_TANH)
        return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * z * (1.0f + 0.044715f * z * z)));
    return z / (1.0f + expf(-z));
}

// The cluster barrier a block passes before it leaves, so that its shared memory outlives the other blocks' reads
// of it.  The arrival is relaxed: nothing this block wrote has to be visible to the others any more (they have read
// what they needed), and a releasing arrival would wait here for the block's last global stores to be performed.
__device__ __forceinline__ void cluster_leave_together() {
    asm volatile("barrier.cluster.arrive.relaxed;\n\tbarrier.cluster.wait;" ::: "memory");
}

// One message per library and host thread; read by mb_last_error() after a non-zero return.
inline char* error_buffer() {
    static thread_local char buffer[1024] = {0};
    return buffer;
}

inline int fail(const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(error_buffer(), 1024, format, args);
    va_end(args);
    return 1;
}

inline int check_launch(const char* what) {
    cudaError_t status = cudaPeekAtLastError();
    if (status != cudaSuccess) {
        cudaGetLastError();
        return fail("%s: %s", what, cudaGetErrorString(status));
    }
    return 0;
}

template <typename T>
struct Num;

template <>
struct Num<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};

template <>
struct Num<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// Loads 8 consecutive elements (address must be 16-byte aligned for bf16, 32-byte for float).
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of the
// additions depends on the block size only, never on the data or on other blocks.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < warps) ? scratch[lane] : 0.0f;
    total = warp_sum(total);
    return total;
}

// Programmatic dependent launch.  A kernel launched with launch_dependent() may start while the
// kernel before it in the stream is still draining; everything it does before grid_dependency_wait()
// must not touch what that kernel writes.  Without such a launch both calls do nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// MODELS_B200_NO_PDL=1 in the environment turns every programmatic dependent launch into an ordinary
// one (a switch for debugging launch-order problems).
inline bool dependent_launches_allowed() {
    static const bool allowed = getenv("MODELS_B200_NO_PDL") == nullptr;
    return allowed;
}

template <typename... KernelArgs, typename... Args>
inline int launch_dependent(const char* what, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, bool dependent, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = (dependent && dependent_launches_allowed()) ? 1 : 0;
    cudaError_t status = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
    if (status != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(status));
    return check_launch(what);
}

}  // namespace mb

#define MB_DEFINE_LAST_ERROR() \
    MB_EXPORT const char* mb_last_error() { return mb::error_buffer(); }
