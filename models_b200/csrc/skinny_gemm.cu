// Matrix products for decode: few activation rows (one per live sequence, up to 32) against a large
// bfloat16 weight matrix W[N, K] that is read exactly once, straight from global memory into
// tensor-core fragments.  The work is bound by the weight stream, so everything around the product
// is folded into the same kernel:
//   prologue  NORM: the activations are the float32 residual rows; RMSNorm (gain, epsilon) is applied
//             on the fly -- the rows are multiplied by the gain while they are loaded, their sums of
//             squares are gathered by the same loads, and 1/rms scales the accumulators at the end
//             (sumSq/size + eps, sqrt, 1/rms: integrallis/models, backend-java/.../ops/TensorOps.java:45-58).
//   epilogue  BF16 / F32: store.  RESIDUAL: add into the float32 residual stream
//             (x = x + W.h, backend-java/.../llama/LlamaForwardPass.java:1131-1138,1172-1178).
//             SWIGLU: the block computes a gate tile and the matching up tile and stores
//             silu(gate) * up (backend-java/.../ops/TensorOps.java:1407-1425).
//
// Layout of the work: a block owns 16 weight rows (two such tiles, `pair_offset` rows apart, for
// SWIGLU); its warps split K.  A warp walks its K slice 64 columns at a time.  In an
// m16n8k16 MMA the weights are the 16-row operand and up to 8 activation rows the 8-column one.  The
// order of k inside an MMA is free as long as both operands agree, so each lane loads 16-byte
// pieces: columns [k0 + 16*tid4, +16) of weight rows groupID and groupID+8, and the same columns of
// activation row groupID.  Partial sums of the warps are added in warp order in shared memory.
#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

using bf16 = __nv_bfloat16;

enum { PRO_NONE = 0, PRO_NORM = 1 };
enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3 };

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_weights(const bf16* p) {
    uint4 v;
    // streamed once: do not keep in L1
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct SkinnyArgs {
    const bf16* w;
    int ldw, n, k, batch;
    const bf16* x;        // PRO_NONE: [batch, k]
    int ldx;
    const float* xf;      // PRO_NORM: float rows
    int ldxf;
    const float* gain;    // PRO_NORM: [k]
    float eps;
    const int* rows;      // optional: activation row b is xf row rows[b]
    bf16* out_bf16;
    float* out_f32;       // EPI_F32 output, or the residual stream for EPI_RESIDUAL
    int ld_out;
    int pair_offset;      // EPI_SWIGLU: the up tile starts pair_offset rows after the gate tile
    int k_per_warp;       // multiple of 64
};

// NT: tiles of 8 activation rows.  TILES: 1, or 2 for paired row tiles.
template <int NT, int PRO, int EPI>
__global__ void __launch_bounds__(512)
skinny_gemm_kernel(const SkinnyArgs args) {
    constexpr int TILES = EPI == EPI_SWIGLU ? 2 : 1;
    extern __shared__ float reduce_smem[];  // [warps][TILES][16][NT*8] then [warps][NT*8] sums of squares
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int group_id = lane >> 2, tid4 = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int k_begin = warp * args.k_per_warp;
    const int k_end = min(args.k, k_begin + args.k_per_warp);

    // weight rows of this lane (clamped: rows beyond N are computed and dropped)
    const bf16* w_rows[TILES][2];
#pragma unroll
    for (int t = 0; t < TILES; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = min(args.n - 1 + t * args.pair_offset, n0 + t * args.pair_offset + group_id + 8 * h);
            w_rows[t][h] = args.w + (size_t)row * args.ldw;
        }
    // activation rows of this lane: batch index nt*8 + group_id
    const bf16* x_rows[NT];
    const float* xf_rows[NT];
    bool x_live[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int b = nt * 8 + group_id;
        x_live[nt] = b < args.batch;
        const int src = x_live[nt] ? (args.rows ? args.rows[b] : b) : 0;
        x_rows[nt] = PRO == PRO_NONE ? args.x + (size_t)src * args.ldx : nullptr;
        xf_rows[nt] = PRO == PRO_NORM ? args.xf + (size_t)src * args.ldxf : nullptr;
    }

    float acc[TILES][NT][4];
#pragma unroll
    for (int t = 0; t < TILES; ++t)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[t][nt][0] = acc[t][nt][1] = acc[t][nt][2] = acc[t][nt][3] = 0.0f;
    float sum_sq[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) sum_sq[nt] = 0.0f;

    // weights are fetched one step ahead of the products that use them
    uint4 wv_next[TILES][2][2];
    auto fetch = [&](int k0) {
        const int kc = k0 + 16 * tid4;  // two 16-byte pieces per row: columns k0 + 16*tid4 + {0, 8}
#pragma unroll
        for (int t = 0; t < TILES; ++t)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    wv_next[t][h][c] = (kc + 8 * c < k_end) ? load_weights(w_rows[t][h] + kc + 8 * c) : make_uint4(0u, 0u, 0u, 0u);
    };
    if (k_begin < k_end) fetch(k_begin);
    for (int k0 = k_begin; k0 < k_end; k0 += 64) {
        const int kc = k0 + 16 * tid4;
        uint4 wv[TILES][2][2];
#pragma unroll
        for (int t = 0; t < TILES; ++t)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c = 0; c < 2; ++c) wv[t][h][c] = wv_next[t][h][c];
        if (k0 + 64 < k_end) fetch(k0 + 64);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint4 xv[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int kk = kc + 8 * c;
                xv[c] = make_uint4(0u, 0u, 0u, 0u);
                if (kk < k_end && x_live[nt]) {
                    if (PRO == PRO_NONE) {
                        xv[c] = *reinterpret_cast<const uint4*>(x_rows[nt] + kk);
                    } else {
                        const float4 a = *reinterpret_cast<const float4*>(xf_rows[nt] + kk);
                        const float4 b = *reinterpret_cast<const float4*>(xf_rows[nt] + kk + 4);
                        const float4 ga = *reinterpret_cast<const float4*>(args.gain + kk);
                        const float4 gb = *reinterpret_cast<const float4*>(args.gain + kk + 4);
                        sum_sq[nt] += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
                        xv[c] = make_uint4(pack2(a.x * ga.x, a.y * ga.y), pack2(a.z * ga.z, a.w * ga.w),
                                           pack2(b.x * gb.x, b.y * gb.y), pack2(b.z * gb.z, b.w * gb.w));
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < TILES; ++t) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    mma_bf16(acc[t][nt], wv[t][0][c].x, wv[t][1][c].x, wv[t][0][c].y, wv[t][1][c].y, xv[c].x, xv[c].y);
                    mma_bf16(acc[t][nt], wv[t][0][c].z, wv[t][1][c].z, wv[t][0][c].w, wv[t][1][c].w, xv[c].z, xv[c].w);
                }
            }
        }
    }

    // partial results of the warps -> shared memory
    constexpr int COLS = NT * 8;
    float* part = reduce_smem + (size_t)warp * TILES * 16 * COLS;
#pragma unroll
    for (int t = 0; t < TILES; ++t)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = group_id + 8 * (i >> 1), col = nt * 8 + tid4 * 2 + (i & 1);
                part[(t * 16 + row) * COLS + col] = acc[t][nt][i];
            }
    float* sq = reduce_smem + (size_t)warps * TILES * 16 * COLS;
    if (PRO == PRO_NORM) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float s = sum_sq[nt];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (tid4 == 0) sq[warp * COLS + nt * 8 + group_id] = s;
        }
    }
    __syncthreads();

    for (int i = threadIdx.x; i < 16 * COLS; i += blockDim.x) {
        const int col = i / 16, row = i % 16;  // row fastest: neighbouring threads store neighbouring columns of the output
        if (col >= args.batch || n0 + row >= args.n) continue;
        float value[TILES];
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
            float s = 0.0f;
            for (int w = 0; w < warps; ++w) s += reduce_smem[((size_t)w * TILES + t) * 16 * COLS + row * COLS + col];
            value[t] = s;
        }
        if (PRO == PRO_NORM) {
            float s = 0.0f;
            for (int w = 0; w < warps; ++w) s += sq[w * COLS + col];
            const float inv_rms = 1.0f / sqrtf(s / (float)args.k + args.eps);
#pragma unroll
            for (int t = 0; t < TILES; ++t) value[t] *= inv_rms;
        }
        const size_t at = (size_t)col * args.ld_out + n0 + row;
        if (EPI == EPI_BF16) args.out_bf16[at] = __float2bfloat16_rn(value[0]);
        if (EPI == EPI_F32) args.out_f32[at] = value[0];
        if (EPI == EPI_RESIDUAL) args.out_f32[at] += value[0];
        if (EPI == EPI_SWIGLU) {
            const float g = value[0], u = value[TILES - 1];
            args.out_bf16[at] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
        }
    }
}

template <int NT, int PRO, int EPI>
static int launch(const SkinnyArgs& args, int warps, cudaStream_t stream) {
    constexpr int TILES = EPI == EPI_SWIGLU ? 2 : 1;
    const size_t smem = ((size_t)warps * TILES * 16 * NT * 8 + (size_t)warps * NT * 8) * sizeof(float);
    auto kernel = skinny_gemm_kernel<NT, PRO, EPI>;
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("skinny_gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(status));
    }
    const int rows = EPI == EPI_SWIGLU ? args.pair_offset : args.n;
    kernel<<<(rows + 15) / 16, warps * 32, smem, stream>>>(args);
    return check_launch("skinny_gemm");
}

template <int PRO, int EPI>
static int launch_nt(const SkinnyArgs& args, int warps, cudaStream_t stream) {
    if (args.batch <= 8) return launch<1, PRO, EPI>(args, warps, stream);
    if (args.batch <= 16) return launch<2, PRO, EPI>(args, warps, stream);
    if (PRO == PRO_NORM) return fail("skinny_gemm: the norm prologue takes at most 16 rows, got %d", args.batch);
    if (args.batch <= 32) return launch<4, PRO_NONE, EPI>(args, warps, stream);
    return fail("skinny_gemm: takes at most 32 activation rows, got %d", args.batch);
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_skinny_max_rows(int with_norm) { return with_norm ? 16 : 32; }

// w: bfloat16 [n, k] (row stride ldw).  Activations: x (bfloat16 [batch, k]) when gain is null,
// else xf (float32 rows, optionally picked by `rows`) normalised with `gain` and `eps`.
// epilogue 0: out bfloat16 [batch, n]; 1: out float32; 2: out float32 += ; 3: w holds gate rows
// [0, n/2) and up rows [n/2, n), out bfloat16 [batch, n/2] = silu(gate) * up.
MB_EXPORT int mb_skinny_gemm(const void* w, int ldw, int n, int k, int batch, const void* x, int ldx, const float* xf,
                             int ldxf, const float* gain, float eps, const int* rows, void* out, int ld_out,
                             int epilogue, int multiprocessors, cudaStream_t stream) {
    if (batch <= 0 || n <= 0) return 0;
    if (batch > 32) return fail("skinny_gemm: takes at most 32 activation rows, got %d", batch);
    if (k <= 0 || k % 8 || ldw % 8) return fail("skinny_gemm: k (%d) and the weight row stride (%d) must be multiples of 8", k, ldw);
    if ((uintptr_t)w & 15) return fail("skinny_gemm: the weight matrix must start on a 16-byte boundary");
    const bool norm = gain != nullptr;
    if (norm && (!xf || ldxf % 4 || ((uintptr_t)xf & 15) || ((uintptr_t)gain & 15)))
        return fail("skinny_gemm: the norm prologue needs 16-byte aligned float rows and gain");
    if (!norm && (!x || ldx % 8 || ((uintptr_t)x & 15))) return fail("skinny_gemm: activations need 16-byte aligned bfloat16 rows");
    if (epilogue == EPI_SWIGLU && n % 2) return fail("skinny_gemm: the gated epilogue needs an even number of weight rows, got %d", n);
    SkinnyArgs args{};
    args.w = (const bf16*)w; args.ldw = ldw; args.n = n; args.k = k; args.batch = batch;
    args.x = (const bf16*)x; args.ldx = ldx; args.xf = xf; args.ldxf = ldxf; args.gain = gain; args.eps = eps; args.rows = rows;
    args.out_bf16 = (bf16*)out; args.out_f32 = (float*)out; args.ld_out = ld_out;
    args.pair_offset = epilogue == EPI_SWIGLU ? n / 2 : 0;
    if (epilogue == EPI_SWIGLU) args.n = n / 2;
    // warps per block: enough blocks x warps to keep every multiprocessor streaming, K slices of >= 128
    const int tiles = (args.n + 15) / 16;
    int warps = 1;
    while (warps < 16 && tiles * warps < multiprocessors * 16 && k / (warps * 2) >= 128) warps *= 2;
    args.k_per_warp = ((k + warps - 1) / warps + 63) / 64 * 64;
#define MB_CASE(PRO, EPI) \
    if ((norm ? PRO_NORM : PRO_NONE) == PRO && epilogue == EPI) return launch_nt<PRO, EPI>(args, warps, stream);
    MB_CASE(PRO_NONE, EPI_BF16)
    MB_CASE(PRO_NONE, EPI_F32)
    MB_CASE(PRO_NONE, EPI_RESIDUAL)
    MB_CASE(PRO_NORM, EPI_BF16)
    MB_CASE(PRO_NORM, EPI_F32)
    MB_CASE(PRO_NORM, EPI_SWIGLU)
    MB_CASE(PRO_NONE, EPI_SWIGLU)
#undef MB_CASE
    return fail("skinny_gemm: no kernel for prologue %d with epilogue %d", norm ? 1 : 0, epilogue);
}
