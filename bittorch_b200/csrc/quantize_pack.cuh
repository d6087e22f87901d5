// Fused weight ternarizer + 2-bit packer, and the stand-alone packer / unpacker.
//
// One CTA owns 16 consecutive output rows (n) of the master weight.  Pass 1 streams
// the rows from HBM to find each row's absmax; pass 2 re-reads the same rows (now in
// L2: 16 rows are far smaller than the CTA's share of the 126 MB L2 for the shapes of
// interest), ternarizes, packs four k per byte and transposes 128x16-byte tiles through
// shared memory so that the [ceil(K/4), N] buffer is written in 16-byte runs along n.
// Algorithmic traffic: sizeof(T) bytes read + 1/4 byte written per weight.
#pragma once

#include "common.cuh"

namespace bt {

constexpr int QP_ROWS = 16;      // output rows per CTA: keeps the rows of all resident CTAs inside L2 for pass 2
constexpr int QP_THREADS = 512;  // 16 warps, 1 row each
constexpr int QP_KB_TILE = 128;  // packed bytes (along k) per transposed tile: 4 loads in flight per lane and row

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
        // max over the bit patterns of |w|: for non-negative floats unsigned order is numeric
        // order, and every NaN pattern sorts above +inf, so a NaN propagates like torch.max
        uint32_t mbits = 0;
        for (int64_t kb0 = lane; kb0 < KB; kb0 += 32 * 8) {
            float v[8][4];
#pragma unroll
            for (int u = 0; u < 8; ++u) {                 // eight independent loads in flight per lane
                const int64_t kb = kb0 + 32 * u;
                const int64_t k = kb * 4;
                const int valid = (kb < KB) ? ((K - k >= 4) ? 4 : static_cast<int>(K - k)) : 0;
                if (valid > 0) load4<T>(row + k, vec_in, valid, v[u]);
                else v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int i = 0; i < 4; ++i) mbits = max(mbits, __float_as_uint(v[u][i]) & 0x7fffffffu);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mbits = max(mbits, __shfl_xor_sync(0xffffffffu, mbits, o));
        const float m = __uint_as_float(mbits);
        // clamp(min=1e-8) in the storage type (NaN stays NaN)
        const float floor_ = round_through<T>(1e-8f);
        const float s = (m != m) ? m : fmaxf(m, floor_);
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
            const float thr = s_thr[r];
            float v[QP_KB_TILE / 32][4];
            int valid[QP_KB_TILE / 32];
#pragma unroll
            for (int u = 0; u < QP_KB_TILE / 32; ++u) {    // independent loads first
                const int64_t kb = kb0 + lane + 32 * u;
                const int64_t k = kb * 4;
                valid[u] = (n < N && kb < KB) ? ((K - k >= 4) ? 4 : static_cast<int>(K - k)) : 0;
                if (valid[u] > 0) load4<T>(W + n * ldw + k, vec_in, valid[u], v[u]);
            }
#pragma unroll
            for (int u = 0; u < QP_KB_TILE / 32; ++u) {
                const int64_t k = (kb0 + lane + 32 * u) * 4;
                uint32_t byte = 0;
                if (valid[u] > 0) {
                    // |w| > thr ? sign(w) : 0 as two compares: code bit 0 = (w > thr), bit 1 = (w < -thr)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (i < valid[u])
                            byte |= ((v[u][i] > thr ? 1u : 0u) | (v[u][i] < -thr ? 2u : 0u)) << (2 * i);
                    if (codes_out != nullptr || tern_out != nullptr) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (i >= valid[u]) continue;
                            const uint32_t c = (byte >> (2 * i)) & 3u;
                            const int t = static_cast<int>(c & 1u) - static_cast<int>(c >> 1);
                            if (codes_out != nullptr) codes_out[n * K + k + i] = static_cast<int8_t>(t);
                            if (tern_out != nullptr) tern_out[n * K + k + i] = from_float<T>(static_cast<float>(t));
                        }
                    }
                }
                s_tile[lane + 32 * u][r] = static_cast<uint8_t>(byte);
            }
        }
        __syncthreads();
        if (packed_T != nullptr) {
            // QP_KB_TILE (kb) x 32 (n) bytes, 4-byte stores along n
            for (int idx = threadIdx.x; idx < QP_KB_TILE * (QP_ROWS / 4); idx += QP_THREADS) {
                const int kbl = idx / (QP_ROWS / 4);
                const int nl = (idx % (QP_ROWS / 4)) * 4;
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
constexpr int PC_KB_TILE = 32;   // packed bytes (along k) per transposed tile of the stand-alone packer

__global__ void __launch_bounds__(QP_THREADS)
pack_codes_kernel(const int8_t* __restrict__ codes, int64_t N, int64_t K, uint8_t* __restrict__ packed_T) {
    __shared__ uint8_t s_tile[PC_KB_TILE][QP_ROWS + 4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * QP_ROWS;
    const int64_t KB = (K + 3) / 4;
    constexpr int NWARPS = QP_THREADS / 32;
    for (int64_t kb0 = 0; kb0 < KB; kb0 += PC_KB_TILE) {
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
        for (int idx = threadIdx.x; idx < PC_KB_TILE * QP_ROWS; idx += QP_THREADS) {
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

// Row layout uint8 [N, ceil(K/4)] (bittorch/quant/ternary_packed.py:22-75): one thread per packed byte, codes read
// and bytes written along k, so both sides coalesce without a transpose.
__global__ void pack_codes_rows_kernel(const int8_t* __restrict__ codes, int64_t N, int64_t K, uint8_t* __restrict__ packed) {
    const int64_t KB = (K + 3) / 4, total = N * KB;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t n = idx / KB, kb = idx % KB;
        uint32_t byte = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t k = kb * 4 + i;
            if (k < K) byte |= two_bit(codes[n * K + k]) << (2 * i);
        }
        packed[idx] = static_cast<uint8_t>(byte);
    }
}

// Inverse of the row layout; reserved pattern 11 -> 0 (bittorch/quant/ternary_packed.py:112-115).
__global__ void unpack_codes_rows_kernel(const uint8_t* __restrict__ packed, int64_t N, int64_t K, int8_t* __restrict__ codes) {
    const int64_t KB = (K + 3) / 4, total = N * K;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t n = idx / K, k = idx % K;
        const uint32_t c = (packed[n * KB + (k >> 2)] >> (2 * (k & 3))) & 3u;
        codes[idx] = static_cast<int8_t>((c == 1u) - (c == 2u));
    }
}

template <typename T>
static int launch_quantize_pack(const void* W, int64_t N, int64_t K, int64_t ldw, float tf, uint8_t* packed_T,
                                float* scale, int8_t* codes, void* tern, cudaStream_t st) {
    const bool vec = (K % 4 == 0) && (ldw % 4 == 0) && aligned(W, 4 * sizeof(T));
    const unsigned grid = static_cast<unsigned>(ceil_div<int64_t>(N, QP_ROWS));
    BT_LAUNCH(quantize_pack_kernel<T>, grid, QP_THREADS, 0, st, static_cast<const T*>(W), N, K, ldw, tf, packed_T, scale,
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
    BT_LAUNCH(pack_codes_kernel, grid, QP_THREADS, 0, static_cast<cudaStream_t>(stream), codes, N, K, packed_T);
    BT_LAUNCH_OK("pack_codes_kernel");
    return BT_OK;
}

extern "C" int bt_unpack_codes(const uint8_t* packed_T, int64_t N, int64_t K, int8_t* codes, void* stream) {
    using namespace bt;
    BT_REQUIRE(codes != nullptr && packed_T != nullptr, "bt_unpack_codes: NULL pointer");
    BT_REQUIRE(N > 0 && K > 0, "bt_unpack_codes: empty weight");
    const int64_t total = N * K;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(ceil_div<int64_t>(total, 256), sm_count() * 16));
    BT_LAUNCH(unpack_codes_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), packed_T, N, K, codes);
    BT_LAUNCH_OK("unpack_codes_kernel");
    return BT_OK;
}

extern "C" int bt_pack_codes_rows(const int8_t* codes, int64_t N, int64_t K, uint8_t* packed, void* stream) {
    using namespace bt;
    BT_REQUIRE(codes != nullptr && packed != nullptr, "bt_pack_codes_rows: NULL pointer");
    BT_REQUIRE(N > 0 && K > 0, "bt_pack_codes_rows: empty weight");
    const int64_t total = N * ceil_div<int64_t>(K, 4);
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(ceil_div<int64_t>(total, 256), sm_count() * 16));
    BT_LAUNCH(pack_codes_rows_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), codes, N, K, packed);
    BT_LAUNCH_OK("pack_codes_rows_kernel");
    return BT_OK;
}

extern "C" int bt_unpack_codes_rows(const uint8_t* packed, int64_t N, int64_t K, int8_t* codes, void* stream) {
    using namespace bt;
    BT_REQUIRE(codes != nullptr && packed != nullptr, "bt_unpack_codes_rows: NULL pointer");
    BT_REQUIRE(N > 0 && K > 0, "bt_unpack_codes_rows: empty weight");
    const int64_t total = N * K;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(ceil_div<int64_t>(total, 256), sm_count() * 16));
    BT_LAUNCH(unpack_codes_rows_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), packed, N, K, codes);
    BT_LAUNCH_OK("unpack_codes_rows_kernel");
    return BT_OK;
}
