// Random weights on the device: normal variates from Philox4x32-10, bit for bit those of
// weights/philox_normal.py on the host.
//
// Element i of a tensor keyed (k0, k1) comes from counter i / 4; the four output words make two
// Box-Muller pairs.  Logarithm, sine and cosine are polynomials in float64 built from separately
// rounded multiplications and additions (__dmul_rn / __dadd_rn: the compiler must not fuse them),
// division and square root are the IEEE ones, so every step has one correct result and the host
// twin gets the same bits.  integrallis/models seeds a test model from java.util.Random in tensor
// order (models-test/.../NanoGgufModel.java:42-49,91); a keyed counter makes each tensor
// reproducible on its own, wherever it is drawn.

#include "common.cuh"

MB_DEFINE_LAST_ERROR()

namespace mb {

__device__ __forceinline__ void philox4x32_10(uint64_t counter, uint32_t k0, uint32_t k1, uint32_t (&c)[4]) {
    c[0] = (uint32_t)counter; c[1] = (uint32_t)(counter >> 32); c[2] = 0u; c[3] = 0u;
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
        c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

__device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }

// s = terms[0]; s = s * x2 + terms[i] ... with every product and sum rounded on its own
template <int N>
__device__ __forceinline__ double horner(double x2, const double (&terms)[N]) {
    double s = terms[0];
#pragma unroll
    for (int i = 1; i < N; ++i) s = add(mul(s, x2), terms[i]);
    return s;
}

__device__ __forceinline__ void box_muller(uint32_t a, uint32_t b, double& z_cos, double& z_sin) {
    const double kLn2 = 0.6931471805599453, kQuarterPi = 3.141592653589793 / 4.0, kSqrtHalf = 0.7071067811865476;
    const double log_terms[7] = {1.0 / 15, 1.0 / 13, 1.0 / 11, 1.0 / 9, 1.0 / 7, 1.0 / 5, 1.0 / 3};
    const double sin_terms[7] = {-1.0 / 1307674368000.0, 1.0 / 6227020800.0, -1.0 / 39916800.0, 1.0 / 362880.0,
                                 -1.0 / 5040.0, 1.0 / 120.0, -1.0 / 6.0};
    const double cos_terms[8] = {1.0 / 20922789888000.0, -1.0 / 87178291200.0, 1.0 / 479001600.0, -1.0 / 3628800.0,
                                 1.0 / 40320.0, -1.0 / 720.0, 1.0 / 24.0, -1.0 / 2.0};
    // u1 = n / 2^32, n = a + 1 in 1 ... 2^32; n = m 2^e with m in [0.5, 1)
    const uint64_t n = (uint64_t)a + 1ull;
    int e = 64 - __clzll((long long)n);
    double m = mul((double)n, __longlong_as_double((long long)(1023 - e) << 52));  // exact: a power of two
    if (m < kSqrtHalf) {
        m = mul(m, 2.0);
        e -= 1;
    }
    const double t = __ddiv_rn(add(m, -1.0), add(m, 1.0));
    const double t2 = mul(t, t);
    const double series = add(mul(horner(t2, log_terms), t2), 1.0);
    const double log_u = add(mul((double)(e - 32), kLn2), mul(mul(2.0, t), series));
    const double radius = __dsqrt_rn(mul(-2.0, log_u));
    const uint32_t octant = b >> 29;
    const double fraction = mul((double)(b & 0x1FFFFFFFu), 1.0 / 536870912.0);
    const double x = mul((octant & 1u) ? add(1.0, -fraction) : fraction, kQuarterPi);
    const double x2 = mul(x, x);
    const double sin_x = mul(add(mul(horner(x2, sin_terms), x2), 1.0), x);
    const double cos_x = add(mul(horner(x2, cos_terms), x2), 1.0);
    const bool swap = ((octant + 1u) & 2u) != 0u;
    double c = swap ? sin_x : cos_x, s = swap ? cos_x : sin_x;
    if (octant >= 2u && octant <= 5u) c = -c;
    if (octant >= 4u) s = -s;
    z_cos = mul(radius, c);
    z_sin = mul(radius, s);
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, size_t count, uint32_t k0, uint32_t k1, float mean, float std,
                                     int shift) {
    const size_t blocks = (count + 3) / 4;
    for (size_t block = (size_t)blockIdx.x * blockDim.x + threadIdx.x; block < blocks; block += (size_t)gridDim.x * blockDim.x) {
        uint32_t w[4];
        philox4x32_10(block, k0, k1, w);
        double z[4];
        box_muller(w[0], w[1], z[0], z[1]);
        box_muller(w[2], w[3], z[2], z[3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const size_t index = block * 4 + i;
            if (index < count) {
                float value = __fmul_rn(__double2float_rn(z[i]), std);
                if (shift) value = __fadd_rn(value, mean);
                Num<T>::store(out + index, value);
            }
        }
    }
}

}  // namespace mb

// out[i] = mean + std * z_i for count elements of float (dtype 0) or bfloat16 (dtype 1); the mean is added
// only when it is not 0 (as the host twin does).
MB_EXPORT int mb_random_normal(void* out, int dtype, size_t count, uint32_t k0, uint32_t k1, float mean, float std,
                               cudaStream_t stream) {
    if (count == 0) return 0;
    const size_t blocks = (count + 3) / 4;
    const int threads = 256;
    const unsigned grid = (unsigned)((blocks + threads - 1) / threads < 148 * 16 ? (blocks + threads - 1) / threads : 148 * 16);
    const int shift = mean != 0.0f ? 1 : 0;
    if (dtype == MB_F32)
        mb::random_normal_kernel<float><<<grid, threads, 0, stream>>>((float*)out, count, k0, k1, mean, std, shift);
    else if (dtype == MB_BF16)
        mb::random_normal_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((__nv_bfloat16*)out, count, k0, k1, mean, std, shift);
    else
        return mb::fail("mb_random_normal: unknown dtype code %d", dtype);
    return mb::check_launch("mb_random_normal");
}
