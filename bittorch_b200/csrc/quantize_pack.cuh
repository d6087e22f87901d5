// Fused weight ternarizer + 2-bit packer, and the stand-alone packer / unpacker.
//
// One CTA owns 32 consecutive output rows (n) of the master weight.  Pass 1 streams
// the rows from HBM to find each row's absmax; pass 2 re-reads the same rows (now in
// L2: 32 rows are far smaller than the CTA's share of the 126 MB L2 for the shapes of
// interest), ternarizes, packs four k per byte and transposes 32x32-byte tiles through
// shared memory so that the [ceil(K/4), N] buffer is written in 32-byte runs along n.
// Algorithmic traffic: sizeof(T) bytes read + 1/4 byte written per weight.
#pragma once

#include "common.cuh"

namespace bt {

constexpr int QP_ROWS = 32;      // output rows per CTA
constexpr int QP_THREADS = 512;  // 16 warps, 2 rows each
constexpr int QP_KB_TILE = 32;   // packed bytes (along k) per transposed tile

// bittorch/quant/ternary.py:137-142 — sign where |w| > thr, else 0.
__device__ __forceinline__ int ternary_code(float w, float thr) {
    return (fabsf(w) > thr) ? ((w > 0.0f) - (w < 0.0f)) : 0;
}
// bittorch/quant/ternary_packed.py:57-61 — 0 -> 0, +1 -> 1, -1 -> 2.
__device__ __forceinline__ uint32_t two_bit(int t) { return t == 1 ? 1u : (t == -1 ? 2u : 0u); }

template <typename T>
__global__ void __launch_bounds__(QP_THREADS)
quantize_pack_kernel(const T* __restrict__ W, int64_t N, int64_t K, int64_t ldw, float threshold_factor,
                     uint8_t* __restrict__ packed_T, float* __restrict__ scale_out,
                     int8_t* __restrict__ codes_out, T* __restrict__ tern_out, bool vec_in) {
    __shared__ float s_thr[QP_ROWS];
    __shared__ __align__(16) uint8_t s_tile[QP_KB_TILE][QP_ROWS + 4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * QP_ROWS;
    const int64_t KB = (K + 3) / 4;
    constexpr int NWARPS = QP_THREADS / 32;

    // ---- pass 1: per-row absmax -> scale, threshold (quant/ternary.py:125-134) ----
    for (int r = warp; r < QP_ROWS; r += NWARPS) {
        const int64_t n = n0 + r;
        if (n >= N) { if (lane == 0) s_thr[r] = 0.0f; continue; }
        const T* row = W + n * ldw;
        float m = 0.0f;
        int nan_seen = 0;
        for (int64_t kb = lane; kb < KB; kb += 32) {
            float v[4];
            const int64_t k = kb * 4;
            const int valid = (K - k >= 4) ? 4 : static_cast<int>(K - k);
            load4<T>(row + k, vec_in, valid, v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = fabsf(v[i]);
                nan_seen |= (a != a);
                m = fmaxf(m, a);
            }
        }
        m = warp_max(m);
        nan_seen = warp_or(nan_seen);
        // clamp(min=1e-8) in the storage type; torch.max propagates NaN.
        const float floor_ = round_through<T>(1e-8f);
        float s = nan_seen ? __int_as_float(0x7fc00000) : fmaxf(m, floor_);
        if (lane == 0) {
            scale_out[n] = s;
            s_thr[r] = round_through<T>(__fmul_rn(threshold_factor, s));
        }
    }
    __syncthreads();

    // ---- pass 2: ternarize, pack, transpose, store ------------------------------------
    const bool n_vec = (N % 4 == 0);   // 4-byte stores along n
    for (int64_t kb0 = 0; kb0 < KB; kb0 += QP_KB_TILE) {
        for (int r = warp; r < QP_ROWS; r += NWARPS) {
            const int64_t n = n0 + r;
            const int64_t kb = kb0 + lane;
            uint32_t byte = 0;
            if (n < N && kb < KB) {
                const int64_t k = kb * 4;
                const int valid = (K - k >= 4) ? 4 : static_cast<int>(K - k);
                float v[4];
                load4<T>(W + n * ldw + k, vec_in, valid, v);
                const float thr = s_thr[r];
                int t[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    t[i] = (i < valid) ? ternary_code(v[i], thr) : 0;
                    byte |= two_bit(t[i]) << (2 * i);
                }
                if (codes_out != nullptr) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (i < valid) codes_out[n * K + k + i] = static_cast<int8_t>(t[i]);
                }
                if (tern_out != nullptr) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (i < valid) tern_out[n * K + k + i] = from_float<T>(static_cast<float>(t[i]));
                }
            }
            s_tile[lane][r] = static_cast<uint8_t>(byte);
        }
        __syncthreads();
        if (packed_T != nullptr) {
            // 32 (kb) x 32 (n) bytes; 256 threads store 4 bytes each along n.
            if (threadIdx.x < QP_KB_TILE * (QP_ROWS / 4)) {
                const int kbl = threadIdx.x / (QP_ROWS / 4);
                const int nl = (threadIdx.x % (QP_ROWS / 4)) * 4;
                const int64_t kb = kb0 + kbl;
                const int64_t n = n0 + nl;
                if (kb < KB && n < N) {
                    if (n_vec) {
                        *reinterpret_cast<uint32_t*>(packed_T + kb * N + n) =
                            *reinterpret_cast<const uint32_t*>(&s_tile[kbl][nl]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (n + i < N) packed_T[kb * N + n + i] = s_tile[kbl][nl + i];
                    }
                }
            }
        }
        __syncthreads();
    }
}

// Packs int8 codes [N,K] into the public [ceil(K/4), N] buffer (same tiling as above).
__global__ void __launch_bounds__(QP_THREADS)
pack_codes_kernel(const int8_t* __restrict__ codes, int64_t N, int64_t K, uint8_t* __restrict__ packed_T) {
    __shared__ uint8_t s_tile[QP_KB_TILE][QP_ROWS + 4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * QP_ROWS;
    const int64_t KB = (K + 3) / 4;
    constexpr int NWARPS = QP_THREADS / 32;
    for (int64_t kb0 = 0; kb0 < KB; kb0 += QP_KB_TILE) {
        for (int r = warp; r < QP_ROWS; r += NWARPS) {
            const int64_t n = n0 + r, kb = kb0 + lane;
            uint32_t byte = 0;
            if (n < N && kb < KB) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int64_t k = kb * 4 + i;
                    if (k < K) byte |= two_bit(codes[n * K + k]) << (2 * i);
                }
            }
            s_tile[lane][r] = static_cast<uint8_t>(byte);
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < QP_KB_TILE * QP_ROWS; idx += QP_THREADS) {
            const int kbl = idx / QP_ROWS, nl = idx % QP_ROWS;
            const int64_t kb = kb0 + kbl, n = n0 + nl;
            if (kb < KB && n < N) packed_T[kb * N + n] = s_tile[kbl][nl];
        }
        __syncthreads();
    }
}

// Inverse: public packed buffer -> int8 codes [N,K]; reserved pattern 11 -> 0
// (bittorch/quant/ternary_packed.py:112-115).
__global__ void unpack_codes_kernel(const uint8_t* __restrict__ packed_T, int64_t N, int64_t K,
                                    int8_t* __restrict__ codes) {
    const int64_t total = N * K;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t n = idx / K, k = idx % K;
        const uint32_t c = (packed_T[(k >> 2) * N + n] >> (2 * (k & 3))) & 3u;
        codes[idx] = static_cast<int8_t>((c == 1u) - (c == 2u));
    }
}

template <typename T>
static int launch_quantize_pack(const void* W, int64_t N, int64_t K, int64_t ldw, float tf, uint8_t* packed_T,
                                float* scale, int8_t* codes, void* tern, cudaStream_t st) {
    const bool vec = (K % 4 == 0) && (ldw % 4 == 0) && aligned(W, 4 * sizeof(T));
    const unsigned grid = static_cast<unsigned>(ceil_div<int64_t>(N, QP_ROWS));
    quantize_pack_kernel<T><<<grid, QP_THREADS, 0, st>>>(static_cast<const T*>(W), N, K, ldw, tf, packed_T, scale,
                                                          codes, static_cast<T*>(tern), vec);
    BT_LAUNCH_OK("quantize_pack_kernel");
    return BT_OK;
}

}  // namespace bt

extern "C" int bt_quantize_pack(const void* W, int w_dtype, int64_t N, int64_t K, int64_t ldw, float threshold_factor,
                                uint8_t* packed_T, float* scale, int8_t* codes, void* tern, void* stream) {
    using namespace bt;
    BT_REQUIRE(W != nullptr && scale != nullptr, "bt_quantize_pack: W and scale must not be NULL");
    BT_REQUIRE(valid_dtype(w_dtype), "bt_quantize_pack: unknown dtype %d", w_dtype);
    BT_REQUIRE(N > 0 && K > 0, "bt_quantize_pack: empty weight [%lld,%lld]", (long long)N, (long long)K);
    BT_REQUIRE(ldw >= K, "bt_quantize_pack: row stride %lld < K %lld", (long long)ldw, (long long)K);
    BT_REQUIRE(N <= (int64_t{1} << 31) * QP_ROWS / 2, "bt_quantize_pack: N too large");
    BT_REQUIRE(packed_T == nullptr || N % 4 != 0 || aligned(packed_T, 4), "bt_quantize_pack: packed_T must be 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (w_dtype == BT_F32) return launch_quantize_pack<float>(W, N, K, ldw, threshold_factor, packed_T, scale, codes, tern, st);
    if (w_dtype == BT_F16) return launch_quantize_pack<__half>(W, N, K, ldw, threshold_factor, packed_T, scale, codes, tern, st);
    return launch_quantize_pack<__nv_bfloat16>(W, N, K, ldw, threshold_factor, packed_T, scale, codes, tern, st);
}

extern "C" int bt_pack_codes(const int8_t* codes, int64_t N, int64_t K, uint8_t* packed_T, void* stream) {
    using namespace bt;
    BT_REQUIRE(codes != nullptr && packed_T != nullptr, "bt_pack_codes: NULL pointer");
    BT_REQUIRE(N > 0 && K > 0, "bt_pack_codes: empty weight");
    const unsigned grid = static_cast<unsigned>(ceil_div<int64_t>(N, QP_ROWS));
    pack_codes_kernel<<<grid, QP_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(codes, N, K, packed_T);
    BT_LAUNCH_OK("pack_codes_kernel");
    return BT_OK;
}

extern "C" int bt_unpack_codes(const uint8_t* packed_T, int64_t N, int64_t K, int8_t* codes, void* stream) {
    using namespace bt;
    BT_REQUIRE(codes != nullptr && packed_T != nullptr, "bt_unpack_codes: NULL pointer");
    BT_REQUIRE(N > 0 && K > 0, "bt_unpack_codes: empty weight");
    const int64_t total = N * K;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(ceil_div<int64_t>(total, 256), sm_count() * 16));
    unpack_codes_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(packed_T, N, K, codes);
    BT_LAUNCH_OK("unpack_codes_kernel");
    return BT_OK;
}
