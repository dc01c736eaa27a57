// True 32-bit matrix product: C[M, N] = A[M, K] . W[N, K]^T with float operands and float FMAs
// on the CUDA cores -- no tensor-core mode, no reduced-precision inputs.  It is the matrix
// product of the 32-bit path of the whole model.
//
// out[r] = sum_c W[r, c] * x[c] (integrallis/models, backend-java/.../ops/TensorOps.java:61-63).
// Every output element is one chain of FMAs over c = 0..K-1 in ascending order, so a row's result
// does not depend on how many other rows the call carries or on where the row sits in a tile.
#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, int lda, const float* __restrict__ w, int ldw, float* __restrict__ c,
                int ldc, int m, int n, int k) {
    __shared__ float a_tile[kTileK][kTileM + 4];
    __shared__ float w_tile[kTileK][kTileN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
    const int row0 = blockIdx.y * kTileM, col0 = blockIdx.x * kTileN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k; k0 += kTileK) {
        // 64 rows x 16 columns of each operand; 256 threads, 4 elements each
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int index = threadIdx.x + i * 256;
            const int r = index / kTileK, kk = index % kTileK;
            const int gr = row0 + r, gc = col0 + r, gk = k0 + kk;
            a_tile[kk][r] = (gr < m && gk < k) ? a[(size_t)gr * lda + gk] : 0.0f;
            w_tile[kk][r] = (gc < n && gk < k) ? w[(size_t)gc * ldw + gk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTileK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = a_tile[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = w_tile[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc < n) c[(size_t)gr * ldc + gc] = acc[i][j];
        }
    }
}

// Few rows (decode): one warp per output column, lanes stride over K, rows kept in registers.
// The per-lane partial sums are combined in a fixed butterfly, so results are reproducible; the
// order differs from the tiled kernel's single chain, which is rounding only.
template <int kRows>
__global__ void __launch_bounds__(256)
gemv_f32_kernel(const float* __restrict__ a, int lda, const float* __restrict__ w, int ldw, float* __restrict__ c,
                int ldc, int m, int n, int k) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n) return;
    const float* w_row = w + (size_t)warp * ldw;
    float acc[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;
    for (int kk = lane; kk < k; kk += 32) {
        const float wv = w_row[kk];
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            if (r < m) acc[r] = fmaf(a[(size_t)r * lda + kk], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const float total = warp_sum(acc[r]);
        if (lane == 0 && r < m) c[(size_t)r * ldc + warp] = total;
    }
}

}  // namespace mb

using namespace mb;

// A: [m, k] with row stride lda; W: [n, k] with row stride ldw; C: [m, n] with row stride ldc.
// `row_invariant` != 0 always takes the tiled kernel, whose result for a row does not depend on m.
MB_EXPORT int mb_gemm_f32(const float* a, int lda, const float* w, int ldw, float* c, int ldc, int m, int n, int k,
                          int row_invariant, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return fail("gemm_f32: k %d must be positive", k);
    if (lda < k || ldw < k || ldc < n) return fail("gemm_f32: row strides (%d, %d, %d) are shorter than the rows (%d, %d, %d)", lda, ldw, ldc, k, k, n);
    if (!row_invariant && m <= 8) {
        const int blocks = (n * 32 + 255) / 256;
        gemv_f32_kernel<8><<<blocks, 256, 0, stream>>>(a, lda, w, ldw, c, ldc, m, n, k);
        return check_launch("gemv_f32");
    }
    const dim3 grid((n + kTileN - 1) / kTileN, (m + kTileM - 1) / kTileM);
    if (grid.y > 65535) return fail("gemm_f32: %d rows exceed the grid limit", m);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(a, lda, w, ldw, c, ldc, m, n, k);
    return check_launch("gemm_f32");
}
