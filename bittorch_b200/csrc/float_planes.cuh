// Floating-point activations through the integer kernels, exactly: the two small kernels around the tensor-core GEMM.
//
// bt_gemv_tiled_float (gemv_tiled.cuh) turns each activation row into 32-bit fixed point (a power-of-two scaling from
// the row maximum), splits it into four balanced signed-byte digit planes and runs them through the integer pipeline
// as four int8 rows.  The same construction serves any batch size with the tcgen05 GEMM in the middle:
//
//     float_planes_quant     X [M,K] float  ->  int8 planes [4M,K] (row 4m+p = digit p of row m), their row sums,
//                                               the power of two that undoes the scaling, a flag for non-finite rows
//     bt_gemm_tiled_i8       the planes as 4M int8 rows -> exact int32 accumulators [4M,N]
//     float_planes_combine   acc -> ((a3*256 + a2)*256 + a1)*256 + a0 in 64 bits, one rounding to float, the exact
//                            power of two, scale, bias -> Y [M,N]
//
// so that the reference's float semantics (csrc/kernels/ternary_gemm_production.cu:53-250,
// csrc/kernels/ternary_gemm_tensor_core.cu:120-271: fp32-accumulated Y = (X . T) * scale + bias) come out of the
// 5th-generation tensor cores as the correctly rounded exact sum, at a quarter of the int8 rate.
#pragma once

#include "common.cuh"
#include "fused_elementwise.cuh"

namespace bt {

// v = b3 2^24 + b2 2^16 + b1 2^8 + b0 with b0..b2 in [-128, 127]; |v| <= 2^30 leaves |b3| <= 64.
__device__ __forceinline__ void balanced_digits(int v, int (&b)[4]) {
#pragma unroll
    for (int d = 0; d < 3; ++d) {
        b[d] = static_cast<int>(static_cast<int8_t>(v & 0xff));
        v = (v - b[d]) >> 8;
    }
    b[3] = v;
}

// Exponent e with max|x| < 2^e (clamped so that 2^(30-e) and 2^(e-30) are normal floats).
__device__ __forceinline__ int planes_exponent(float amax) {
    int e = 0;
    frexpf(amax, &e);
    return max(-96, min(127, e));
}

// rint(x * 2^(30-e)) clamped to +-2^30; NaN gives 0 (the row is flagged separately).
__device__ __forceinline__ int planes_fixed_point(float x, float mult) {
    const int v = __float2int_rn(__fmul_rn(x, mult));
    return max(-(1 << 30), min(1 << 30, v));
}

template <typename T>
__global__ void __launch_bounds__(FE_THREADS)
float_planes_quant_kernel(const T* __restrict__ X, int64_t K, int64_t ldx, int8_t* __restrict__ planes,
                          float* __restrict__ pw, int32_t* __restrict__ xsum, int32_t* __restrict__ bad) {
    __shared__ float s_redf[FE_THREADS / 32];
    __shared__ int s_redi[FE_THREADS / 32];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t m = blockIdx.x;
    const T* row = X + m * ldx;
    float mx = 0.0f;
    int nonfinite = 0;
    for (int64_t k = threadIdx.x; k < K; k += FE_THREADS) {
        const float a = fabsf(to_float<T>(row[k]));
        mx = fmaxf(mx, a);
        nonfinite |= !(a <= 3.402823466e38f);
    }
    mx = block_max(mx, s_redf);
    nonfinite = block_sum(nonfinite, s_redi);
    const int e = planes_exponent(mx);
    const float mult = ldexpf(1.0f, 30 - e);
    int sums[4] = {0, 0, 0, 0};
    for (int64_t k = threadIdx.x; k < K; k += FE_THREADS) {
        int b[4];
        balanced_digits(planes_fixed_point(to_float<T>(row[k]), mult), b);
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            planes[(4 * m + d) * K + k] = static_cast<int8_t>(b[d]);
            sums[d] += b[d];
        }
    }
#pragma unroll
    for (int d = 0; d < 4; ++d) {
        const int total = block_sum(sums[d], s_redi);
        if (threadIdx.x == 0) xsum[4 * m + d] = total;
    }
    if (threadIdx.x == 0) {
        pw[m] = ldexpf(1.0f, e - 30);
        bad[m] = nonfinite != 0;
    }
}

// grid = (ceil(N / 256), M), block = 256: thread (m, n) reads the four plane accumulators of its output.
__global__ void __launch_bounds__(256)
float_planes_combine_kernel(const int32_t* __restrict__ acc, int64_t N, const float* __restrict__ pw,
                            const int32_t* __restrict__ bad, const float* __restrict__ scale,
                            const float* __restrict__ bias, void* __restrict__ Y, int y_dtype, int64_t ldy) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t m = blockIdx.y;
    const int64_t n = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (n >= N) return;
    long long total = 0;
#pragma unroll
    for (int d = 3; d >= 0; --d) total = total * 256 + acc[(4 * m + d) * N + n];
    float y = __fmul_rn(__fmul_rn(__ll2float_rn(total), pw[m]), scale[n]);
    if (bias != nullptr) y = __fadd_rn(y, bias[n]);
    if (bad[m]) y = __int_as_float(0x7fc00000);
    store_out_dt(Y, y_dtype, m * ldy + n, y);
}

template <typename T>
static int launch_float_planes_quant(const void* X, int64_t M, int64_t K, int64_t ldx, int8_t* planes, float* pw,
                                     int32_t* xsum, int32_t* bad, cudaStream_t st) {
    BT_LAUNCH(float_planes_quant_kernel<T>, static_cast<unsigned>(M), FE_THREADS, 0, st, static_cast<const T*>(X), K, ldx,
              planes, pw, xsum, bad);
    BT_LAUNCH_OK("float_planes_quant_kernel");
    return BT_OK;
}

}  // namespace bt

extern "C" int bt_float_planes_quant(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* planes, float* pw,
                                     int32_t* xsum, int32_t* bad, void* stream) {
    using namespace bt;
    BT_REQUIRE(X && planes && pw && xsum && bad, "bt_float_planes_quant: NULL pointer");
    BT_REQUIRE(valid_dtype(x_dtype), "bt_float_planes_quant: unknown dtype %d", x_dtype);
    BT_REQUIRE(M > 0 && K > 0, "bt_float_planes_quant: X is empty");
    BT_REQUIRE(ldx >= K, "bt_float_planes_quant: row stride %lld < K %lld", (long long)ldx, (long long)K);
    BT_REQUIRE(M < (int64_t{1} << 29), "bt_float_planes_quant: M too large");
    BT_UNSUPPORTED_IF(K > BT_MAX_K / 2, "bt_float_planes_quant: K=%lld exceeds %d", (long long)K, BT_MAX_K / 2);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_dtype == BT_F32) return launch_float_planes_quant<float>(X, M, K, ldx, planes, pw, xsum, bad, st);
    if (x_dtype == BT_F16) return launch_float_planes_quant<__half>(X, M, K, ldx, planes, pw, xsum, bad, st);
    return launch_float_planes_quant<__nv_bfloat16>(X, M, K, ldx, planes, pw, xsum, bad, st);
}

extern "C" int bt_float_planes_combine(const int32_t* acc, int64_t M, int64_t N, const float* pw, const int32_t* bad,
                                       const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                                       void* stream) {
    using namespace bt;
    BT_REQUIRE(acc && pw && bad && scale && Y, "bt_float_planes_combine: NULL pointer");
    BT_REQUIRE(valid_dtype(y_dtype), "bt_float_planes_combine: unknown output dtype %d", y_dtype);
    BT_REQUIRE(M > 0 && N > 0, "bt_float_planes_combine: empty output");
    BT_REQUIRE(ldy >= N, "bt_float_planes_combine: output row stride %lld < N %lld", (long long)ldy, (long long)N);
    BT_UNSUPPORTED_IF(M > 65535, "bt_float_planes_combine: more than 65535 rows per call");
    const dim3 grid(static_cast<unsigned>(ceil_div<int64_t>(N, 256)), static_cast<unsigned>(M));
    BT_LAUNCH(float_planes_combine_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), acc, N, pw, bad, scale, bias, Y,
              y_dtype, ldy);
    BT_LAUNCH_OK("float_planes_combine_kernel");
    return BT_OK;
}
