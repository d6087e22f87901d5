// Floating-point-activation linear kernels (fp32 accumulation): the reference's exact
// float semantics, kept for callers that need its 1e-4 agreement (training forward of
// the unpacked API, float mode of the packed API).  Classic shared-memory tiling,
// 64x64 output tile, 4x4 outputs per thread; not the bandwidth- or tensor-bound path.
#pragma once

#include "common.cuh"

namespace bt {

constexpr int LF_TILE = 64;
constexpr int LF_BK = 32;
constexpr int LF_THREADS = 256;

// PACKED = false: W is int8 [N,K] (csrc/kernels/ternary_gemm.cu:41-73 semantics).
// PACKED = true : W is the public uint8 [ceil(K/4), N] buffer
//                 (csrc/kernels/ternary_gemm_production.cu:53-142 semantics).
template <typename T, bool PACKED>
__global__ void __launch_bounds__(LF_THREADS)
linear_float_kernel(const T* __restrict__ X, int M, int K, const void* __restrict__ Wv, int N,
                    const float* __restrict__ scale, const float* __restrict__ bias, T* __restrict__ Y) {
    __shared__ float s_x[LF_BK][LF_TILE + 4];
    __shared__ float s_w[LF_BK][LF_TILE + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * LF_TILE, n0 = blockIdx.x * LF_TILE;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += LF_BK) {
        // X tile: 64 rows x 32 k, k fastest in global memory
        for (int idx = threadIdx.x; idx < LF_TILE * LF_BK; idx += LF_THREADS) {
            const int r = idx / LF_BK, kk = idx % LF_BK;
            const int m = m0 + r, k = k0 + kk;
            s_x[kk][r] = (m < M && k < K) ? to_float<T>(X[static_cast<int64_t>(m) * K + k]) : 0.0f;
        }
        if (PACKED) {
            const uint8_t* W = static_cast<const uint8_t*>(Wv);
            // 8 packed rows x 64 columns, n fastest in global memory
            for (int idx = threadIdx.x; idx < (LF_BK / 4) * LF_TILE; idx += LF_THREADS) {
                const int kbl = idx / LF_TILE, c = idx % LF_TILE;
                const int kb = k0 / 4 + kbl, n = n0 + c;
                uint32_t byte = 0;
                if (n < N && kb * 4 < K) byte = W[static_cast<int64_t>(kb) * N + n];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t code = (byte >> (2 * j)) & 3u;
                    s_w[kbl * 4 + j][c] = static_cast<float>(static_cast<int>(code == 1u) - static_cast<int>(code == 2u));
                }
            }
        } else {
            const int8_t* W = static_cast<const int8_t*>(Wv);
            for (int idx = threadIdx.x; idx < LF_TILE * LF_BK; idx += LF_THREADS) {
                const int c = idx / LF_BK, kk = idx % LF_BK;
                const int n = n0 + c, k = k0 + kk;
                s_w[kk][c] = (n < N && k < K) ? static_cast<float>(W[static_cast<int64_t>(n) * K + k]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < LF_BK; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = s_x[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = s_w[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float r = acc[i][j] * scale[n];
            if (bias != nullptr) r += bias[n];
            Y[static_cast<int64_t>(m) * N + n] = from_float<T>(r);
        }
    }
}

template <bool PACKED>
static int launch_linear_float(const char* who, const void* X, int x_dtype, int64_t M, int64_t K, const void* W, int64_t N,
                               const float* scale, const float* bias, void* Y, void* stream) {
    BT_REQUIRE(X && W && scale && Y, "%s: NULL pointer", who);
    BT_REQUIRE(valid_dtype(x_dtype) || x_dtype == BT_F64, "%s: unknown dtype %d", who, x_dtype);
    BT_REQUIRE(M > 0 && K > 0, "%s: X is empty", who);
    BT_REQUIRE(N > 0, "%s: weight is empty", who);
    BT_UNSUPPORTED_IF(M > (int64_t{1} << 30) || N > (int64_t{1} << 30) || K > (int64_t{1} << 30), "%s: shape too large", who);
    const dim3 grid(static_cast<unsigned>(ceil_div<int64_t>(N, LF_TILE)), static_cast<unsigned>(ceil_div<int64_t>(M, LF_TILE)));
    BT_UNSUPPORTED_IF(grid.y > 65535, "%s: M too large for one launch", who);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int m = static_cast<int>(M), k = static_cast<int>(K), n = static_cast<int>(N);
    if (x_dtype == BT_F32)
        BT_LAUNCH((linear_float_kernel<float, PACKED>), grid, LF_THREADS, 0, st, static_cast<const float*>(X), m, k, W, n, scale, bias, static_cast<float*>(Y));
    else if (x_dtype == BT_F64)   // float64 containers, float32 arithmetic (csrc/kernels/ternary_gemm.cu:56-61)
        BT_LAUNCH((linear_float_kernel<double, PACKED>), grid, LF_THREADS, 0, st, static_cast<const double*>(X), m, k, W, n, scale, bias, static_cast<double*>(Y));
    else if (x_dtype == BT_F16)
        BT_LAUNCH((linear_float_kernel<__half, PACKED>), grid, LF_THREADS, 0, st, static_cast<const __half*>(X), m, k, W, n, scale, bias, static_cast<__half*>(Y));
    else
        BT_LAUNCH((linear_float_kernel<__nv_bfloat16, PACKED>), grid, LF_THREADS, 0, st, static_cast<const __nv_bfloat16*>(X), m, k, W, n, scale, bias, static_cast<__nv_bfloat16*>(Y));
    BT_LAUNCH_OK("linear_float_kernel");
    return BT_OK;
}

}  // namespace bt

extern "C" int bt_linear_unpacked(const void* X, int x_dtype, int64_t M, int64_t K, const int8_t* W, int64_t N,
                                  const float* scale, const float* bias, void* Y, void* stream) {
    return bt::launch_linear_float<false>("bt_linear_unpacked", X, x_dtype, M, K, W, N, scale, bias, Y, stream);
}

extern "C" int bt_linear_packed_float(const void* X, int x_dtype, int64_t M, int64_t K, const uint8_t* packed_T, int64_t N,
                                      const float* scale, const float* bias, void* Y, void* stream) {
    return bt::launch_linear_float<true>("bt_linear_packed_float", X, x_dtype, M, K, packed_T, N, scale, bias, Y, stream);
}
