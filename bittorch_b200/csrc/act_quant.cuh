// Per-token int8 activation quantizer: one CTA per row of X.
//
// Pass 1 reads the row for its absmax, pass 2 re-reads it (L1/L2-resident: a row is
// at most a few tens of KB) and writes int8.  Algorithmic traffic: sizeof(T) bytes
// read + 1 byte written per element, + 4 bytes of scale per row.
#pragma once

#include "common.cuh"

namespace bt {

constexpr int AQ_THREADS = 256;

// csrc/kernels/ternary_gemm_tensor_core.cu:343-347 — multiply by the reciprocal,
// roundf (half away from zero), clamp to +-127.
__device__ __forceinline__ int quantize_i8(float v, float inv) {
    float s = roundf(__fmul_rn(v, inv));
    s = fmaxf(-127.0f, fminf(127.0f, s));
    return static_cast<int>(s);
}

template <typename T>
__global__ void __launch_bounds__(AQ_THREADS)
act_quant_kernel(const T* __restrict__ X, int64_t K, int64_t ldx, int8_t* __restrict__ Xq,
                 float* __restrict__ sx, int32_t* __restrict__ xsum, bool vec_in, bool vec_out) {
    __shared__ float s_red[AQ_THREADS / 32];
    __shared__ int s_sum[AQ_THREADS / 32];
    __shared__ float s_inv;
    pdl_launch_dependents();   // the consumer kernel may start prefetching its weights
    pdl_wait();                // X may be the previous kernel's output
    const int64_t m = blockIdx.x;
    const T* row = X + m * ldx;
    const int64_t KB = (K + 3) / 4;

    float mx = 0.0f;
    for (int64_t kb = threadIdx.x; kb < KB; kb += AQ_THREADS) {
        float v[4];
        const int64_t k = kb * 4;
        const int valid = (K - k >= 4) ? 4 : static_cast<int>(K - k);
        load4<T>(row + k, vec_in, valid, v);
#pragma unroll
        for (int i = 0; i < 4; ++i) mx = fmaxf(mx, fabsf(v[i]));
    }
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = s_red[0];
#pragma unroll
        for (int i = 1; i < AQ_THREADS / 32; ++i) t = fmaxf(t, s_red[i]);
        // ternary_gemm_tensor_core.cu:438-440 (scale rule) and :456 (reciprocal).
        const float s = (t > 1e-6f) ? __fdiv_rn(t, 127.0f) : 1.0f;
        sx[m] = s;
        s_inv = __fdiv_rn(1.0f, s);
    }
    __syncthreads();
    const float inv = s_inv;

    int8_t* out = Xq + m * K;
    int qsum = 0;
    for (int64_t kb = threadIdx.x; kb < KB; kb += AQ_THREADS) {
        float v[4];
        const int64_t k = kb * 4;
        const int valid = (K - k >= 4) ? 4 : static_cast<int>(K - k);
        load4<T>(row + k, vec_in, valid, v);
        int q[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            q[i] = quantize_i8(v[i], inv);
            if (i < valid) qsum += q[i];
        }
        if (vec_out && valid == 4) {
            const uint32_t w = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((q[3] & 0xff) << 24);
            *reinterpret_cast<uint32_t*>(out + k) = w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < valid) out[k + i] = static_cast<int8_t>(q[i]);
        }
    }
    if (xsum != nullptr) {      // row sum of the int8 codes: the tensor-core kernel stores weights as t+1
        qsum = warp_sum(qsum);
        if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = qsum;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
#pragma unroll
            for (int i = 0; i < AQ_THREADS / 32; ++i) t += s_sum[i];
            xsum[m] = t;
        }
    }
}

template <typename T>
static int launch_act_quant(const void* X, int64_t M, int64_t K, int64_t ldx, int8_t* Xq, float* sx, int32_t* xsum,
                            cudaStream_t st) {
    const bool vec_in = (K % 4 == 0) && (ldx % 4 == 0) && aligned(X, 4 * sizeof(T));
    const bool vec_out = (K % 4 == 0) && aligned(Xq, 4);
    BT_LAUNCH(act_quant_kernel<T>, static_cast<unsigned>(M), AQ_THREADS, 0, st, static_cast<const T*>(X), K, ldx, Xq, sx,
                                                                         xsum, vec_in, vec_out);
    BT_LAUNCH_OK("act_quant_kernel");
    return BT_OK;
}

}  // namespace bt

extern "C" int bt_act_quant_i8(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* Xq, float* sx,
                               int32_t* xsum, void* stream) {
    using namespace bt;
    BT_REQUIRE(X != nullptr && Xq != nullptr && sx != nullptr, "bt_act_quant_i8: NULL pointer");
    BT_REQUIRE(valid_dtype(x_dtype), "bt_act_quant_i8: unknown dtype %d", x_dtype);
    BT_REQUIRE(M > 0 && K > 0, "bt_act_quant_i8: X is empty");
    BT_REQUIRE(ldx >= K, "bt_act_quant_i8: row stride %lld < K %lld", (long long)ldx, (long long)K);
    BT_REQUIRE(M < (int64_t{1} << 31), "bt_act_quant_i8: M too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_dtype == BT_F32) return launch_act_quant<float>(X, M, K, ldx, Xq, sx, xsum, st);
    if (x_dtype == BT_F16) return launch_act_quant<__half>(X, M, K, ldx, Xq, sx, xsum, st);
    return launch_act_quant<__nv_bfloat16>(X, M, K, ldx, Xq, sx, xsum, st);
}
