// Elementwise steps of a decoder block fused with the per-token int8 activation quantizer, so that the packed
// linear layer behind them starts from int8 rows + scales (bt_gemv_tiled_i8 / bt_gemm_tiled_i8) and the
// floating-point intermediate never travels through global memory twice:
//
//   silu_mul_quant      h = silu(gate) * up                      -> int8 h, scale, row sum      (SwiGLU: the reference's
//                                                                    runtime, js/src/models/TernaryTransformer.ts:520-550)
//   add_rmsnorm_quant   x += delta;  y = x / rms(x) * weight      -> new x, int8 y, scale, row sum (pre-norm residual
//                                                                    blocks, :366-464; RMSNorm js/src/core/RMSNorm.ts:10-38)
//
// One CTA per row.  The arithmetic is spelled out operation by operation (round-to-nearest multiplies and adds that
// the compiler may not contract, an exponential built from them, a fixed reduction order), so a CPU restatement
// reproduces every bit: values are rounded to the activation type T wherever the unfused sequence of framework
// operations would have stored them.
#pragma once

#include "act_quant.cuh"
#include "common.cuh"

namespace bt {

constexpr int FE_THREADS = 1024;    // a decode step has one row per sequence: many threads per row keep it short

// exp(x) from IEEE multiplies, adds and one rint only: x = n ln2 + r, a degree-7 polynomial in r, exact scaling by 2^n.
// Relative error below 2e-7 on [-87, 88]; arguments outside are clamped (the results are then 0 or huge in any case).
__device__ __forceinline__ float exp_plain(float x) {
    x = fminf(fmaxf(x, -87.0f), 88.0f);
    const float n = rintf(__fmul_rn(x, 1.44269504088896341f));
    float r = __fadd_rn(x, -__fmul_rn(n, 0.693359375f));                  // ln2, high part (exact product)
    r = __fadd_rn(r, __fmul_rn(n, 2.12194440e-4f));                       // ln2, low part (ln2 = hi - 2.1219444e-4)
    float p = 1.0f / 5040.0f;
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 720.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 120.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 24.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 6.0f);
    p = __fadd_rn(__fmul_rn(p, r), 0.5f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    return __fmul_rn(p, __int_as_float((static_cast<int>(n) + 127) << 23));   // n in [-126, 127]
}

// silu(g) * u as a framework would leave it in type T: silu rounded to T, the product rounded to T.
template <typename T>
__device__ __forceinline__ float silu_mul_as_stored(float g, float u) {
    const float s = round_through<T>(__fdiv_rn(g, __fadd_rn(1.0f, exp_plain(-g))));
    return round_through<T>(__fmul_rn(s, u));
}

// Block-wide maximum / integer sum of one value per thread (FE_THREADS threads), result in every thread.
__device__ __forceinline__ float block_max(float v, float* s_red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = s_red[0];
#pragma unroll
    for (int i = 1; i < FE_THREADS / 32; ++i) r = fmaxf(r, s_red[i]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ int block_sum(int v, int* s_red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    int r = 0;
#pragma unroll
    for (int i = 0; i < FE_THREADS / 32; ++i) r += s_red[i];
    __syncthreads();
    return r;
}

// Quantizes the row `value(k)`, k < K (a pure function of k, evaluated twice) with the rule of bt_act_quant_i8.
template <typename F>
__device__ __forceinline__ void quantize_row(F value, int64_t K, int8_t* __restrict__ out, float* sx, int32_t* xsum,
                                             float* s_redf, int* s_redi) {
    float mx = 0.0f;
    for (int64_t k = threadIdx.x; k < K; k += FE_THREADS) mx = fmaxf(mx, fabsf(value(k)));
    mx = block_max(mx, s_redf);
    // csrc/kernels/ternary_gemm_tensor_core.cu:438-440 (scale rule) and :456 (reciprocal)
    const float s = (mx > 1e-6f) ? __fdiv_rn(mx, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, s);
    int qsum = 0;
    for (int64_t k = threadIdx.x; k < K; k += FE_THREADS) {
        const int q = quantize_i8(value(k), inv);
        out[k] = static_cast<int8_t>(q);
        qsum += q;
    }
    qsum = block_sum(qsum, s_redi);
    if (threadIdx.x == 0) {
        *sx = s;
        if (xsum != nullptr) *xsum = qsum;
    }
}

// GU [M, ld]: gate in columns [0, F), up in [F, 2F).  Hq int8 [M, F]; H (optional) the unquantized product in T.
template <typename T>
__global__ void __launch_bounds__(FE_THREADS)
silu_mul_quant_kernel(const T* __restrict__ GU, int64_t F, int64_t ld, int8_t* __restrict__ Hq, float* __restrict__ sx,
                      int32_t* __restrict__ xsum, T* __restrict__ H) {
    __shared__ float s_redf[FE_THREADS / 32];
    __shared__ int s_redi[FE_THREADS / 32];
    pdl_launch_dependents();
    pdl_wait();                                               // GU is the preceding kernel's output
    const int64_t m = blockIdx.x;
    const T* gate = GU + m * ld;
    const T* up = gate + F;
    auto value = [&](int64_t k) { return silu_mul_as_stored<T>(to_float<T>(gate[k]), to_float<T>(up[k])); };
    if (H != nullptr)
        for (int64_t k = threadIdx.x; k < F; k += FE_THREADS) H[m * F + k] = from_float<T>(value(k));
    quantize_row(value, F, Hq + m * F, sx + m, xsum ? xsum + m : nullptr, s_redf, s_redi);
}

// X [M, ldx] (updated in place when delta is given), delta [M, ldd] or NULL, weight [D].  The sum of squares is taken
// in double precision in a fixed order: thread t adds elements t, t + 1024, ...; lanes combine by xor 16, 8, 4, 2, 1;
// warps in index order.  Squares of floats are exact in double.
template <typename T>
__global__ void __launch_bounds__(FE_THREADS)
add_rmsnorm_quant_kernel(T* __restrict__ X, const T* __restrict__ delta, int64_t D, int64_t ldx, int64_t ldd,
                         const T* __restrict__ weight, float eps, int8_t* __restrict__ Yq, float* __restrict__ sx,
                         int32_t* __restrict__ xsum, T* __restrict__ Y) {
    __shared__ float s_redf[FE_THREADS / 32];
    __shared__ int s_redi[FE_THREADS / 32];
    __shared__ double s_redd[FE_THREADS / 32];
    __shared__ float s_rms;
    pdl_launch_dependents();
    pdl_wait();
    const int64_t m = blockIdx.x;
    T* x = X + m * ldx;
    double ss = 0.0;
    for (int64_t k = threadIdx.x; k < D; k += FE_THREADS) {
        float v = to_float<T>(x[k]);
        if (delta != nullptr) {
            v = round_through<T>(__fadd_rn(v, to_float<T>(delta[m * ldd + k])));       // the residual stream, as stored
            x[k] = from_float<T>(v);
        }
        ss += static_cast<double>(v) * static_cast<double>(v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const long long bits = __double_as_longlong(ss);
        const int lo = __shfl_xor_sync(0xffffffffu, static_cast<int>(bits & 0xffffffffll), o);
        const int hi = __shfl_xor_sync(0xffffffffu, static_cast<int>(bits >> 32), o);
        ss += __longlong_as_double((static_cast<long long>(hi) << 32) | static_cast<unsigned int>(lo));
    }
    if ((threadIdx.x & 31) == 0) s_redd[threadIdx.x >> 5] = ss;
    __syncthreads();                                          // also orders this thread's x[k] stores before the reads below
    if (threadIdx.x == 0) {
        double total = 0.0;
#pragma unroll
        for (int i = 0; i < FE_THREADS / 32; ++i) total += s_redd[i];
        const float ms = static_cast<float>(total / static_cast<double>(D));
        s_rms = sqrtf(__fadd_rn(ms, eps));                    // js/src/core/RMSNorm.ts:24-30: eps inside the root
    }
    __syncthreads();
    const float rms = s_rms;
    auto value = [&](int64_t k) {
        return round_through<T>(__fmul_rn(__fdiv_rn(to_float<T>(x[k]), rms), to_float<T>(weight[k])));
    };
    if (Y != nullptr)
        for (int64_t k = threadIdx.x; k < D; k += FE_THREADS) Y[m * D + k] = from_float<T>(value(k));
    quantize_row(value, D, Yq + m * D, sx + m, xsum ? xsum + m : nullptr, s_redf, s_redi);
}

template <typename T>
static int launch_silu_mul_quant(const void* GU, int64_t M, int64_t F, int64_t ld, int8_t* Hq, float* sx, int32_t* xsum,
                                 void* H, cudaStream_t st) {
    BT_LAUNCH(silu_mul_quant_kernel<T>, static_cast<unsigned>(M), FE_THREADS, 0, st, static_cast<const T*>(GU), F, ld, Hq, sx,
              xsum, static_cast<T*>(H));
    BT_LAUNCH_OK("silu_mul_quant_kernel");
    return BT_OK;
}

template <typename T>
static int launch_add_rmsnorm_quant(void* X, const void* delta, int64_t M, int64_t D, int64_t ldx, int64_t ldd,
                                    const void* weight, float eps, int8_t* Yq, float* sx, int32_t* xsum, void* Y,
                                    cudaStream_t st) {
    BT_LAUNCH(add_rmsnorm_quant_kernel<T>, static_cast<unsigned>(M), FE_THREADS, 0, st, static_cast<T*>(X),
              static_cast<const T*>(delta), D, ldx, ldd, static_cast<const T*>(weight), eps, Yq, sx, xsum, static_cast<T*>(Y));
    BT_LAUNCH_OK("add_rmsnorm_quant_kernel");
    return BT_OK;
}

}  // namespace bt

extern "C" int bt_silu_mul_quant(const void* GU, int dtype, int64_t M, int64_t F, int64_t ld, int8_t* Hq, float* sx,
                                 int32_t* xsum, void* H, void* stream) {
    using namespace bt;
    BT_REQUIRE(GU != nullptr && Hq != nullptr && sx != nullptr, "bt_silu_mul_quant: NULL pointer");
    BT_REQUIRE(valid_dtype(dtype), "bt_silu_mul_quant: unknown dtype %d", dtype);
    BT_REQUIRE(M > 0 && F > 0, "bt_silu_mul_quant: input is empty");
    BT_REQUIRE(ld >= 2 * F, "bt_silu_mul_quant: row stride %lld < 2F %lld", (long long)ld, (long long)(2 * F));
    BT_REQUIRE(M < (int64_t{1} << 31), "bt_silu_mul_quant: M too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == BT_F32) return launch_silu_mul_quant<float>(GU, M, F, ld, Hq, sx, xsum, H, st);
    if (dtype == BT_F16) return launch_silu_mul_quant<__half>(GU, M, F, ld, Hq, sx, xsum, H, st);
    return launch_silu_mul_quant<__nv_bfloat16>(GU, M, F, ld, Hq, sx, xsum, H, st);
}

extern "C" int bt_add_rmsnorm_quant(void* X, const void* delta, int dtype, int64_t M, int64_t D, int64_t ldx, int64_t ldd,
                                    const void* weight, float eps, int8_t* Yq, float* sx, int32_t* xsum, void* Y,
                                    void* stream) {
    using namespace bt;
    BT_REQUIRE(X != nullptr && weight != nullptr && Yq != nullptr && sx != nullptr, "bt_add_rmsnorm_quant: NULL pointer");
    BT_REQUIRE(valid_dtype(dtype), "bt_add_rmsnorm_quant: unknown dtype %d", dtype);
    BT_REQUIRE(M > 0 && D > 0, "bt_add_rmsnorm_quant: input is empty");
    BT_REQUIRE(ldx >= D && (delta == nullptr || ldd >= D), "bt_add_rmsnorm_quant: row stride smaller than D %lld", (long long)D);
    BT_REQUIRE(eps >= 0.0f, "bt_add_rmsnorm_quant: eps must not be negative");
    BT_REQUIRE(M < (int64_t{1} << 31), "bt_add_rmsnorm_quant: M too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == BT_F32) return launch_add_rmsnorm_quant<float>(X, delta, M, D, ldx, ldd, weight, eps, Yq, sx, xsum, Y, st);
    if (dtype == BT_F16) return launch_add_rmsnorm_quant<__half>(X, delta, M, D, ldx, ldd, weight, eps, Yq, sx, xsum, Y, st);
    return launch_add_rmsnorm_quant<__nv_bfloat16>(X, delta, M, D, ldx, ldd, weight, eps, Yq, sx, xsum, Y, st);
}
