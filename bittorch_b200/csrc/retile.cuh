// Private "tiled" layout of the packed weights and its conversion kernels.
//
// The buffer is an array of 512-byte tiles, tile (nb, kt) at ((nb*KT)+kt)*512 with
// KT = ceil(K/128): 16 output columns x 128 inputs, so the tiles of one 16-column block
// are contiguous along K (a whole column block is one bulk copy).  Inside a tile, lane
// l = 4g+t of a warp owns 16 bytes = words q=0..3; byte j of word q holds four 2-bit
// fields, field i (bits 2i+1:2i) being the weight
//     n = 16 nb + g + 8 (q & 1),     k = 128 kt + 32 t + 8 i + 4 (q >> 1) + j
// stored as t+1 in {0,1,2} (padding outside N x K is 1, i.e. a zero weight).
// So masking plane i of word q (w & (0x03030303 << 2i)) yields four consecutive k of one
// column as bytes scaled by 4^i — a dp4a operand for the decode kernel — and a lane's
// eight (plane, word-half) pieces cover 32 consecutive activations.  For the tensor-core
// kernel, (w >> 2i) & 0x03030303 is four bytes of row n of a K-major 128-byte operand row.
#pragma once

#include "common.cuh"

namespace bt {

constexpr int TILE_N = 16;
constexpr int TILE_K = 128;
constexpr int TILE_BYTES = 512;

// Position of weight (n_local, k_local) inside a tile: 32-bit word index and bit shift.
__host__ __device__ inline void tile_slot(int n_local, int k_local, int& word, int& shift) {
    const int g = n_local & 7, qlo = n_local >> 3;
    const int t = k_local >> 5, r = k_local & 31;
    const int i = r >> 3, qhi = (r >> 2) & 1, j = r & 3;
    word = (4 * g + t) * 4 + (qlo | (qhi << 1));
    shift = 8 * j + 2 * i;
}

// grid = (KT, NB), block = 128: one thread per 32-bit word of the tile.
__global__ void __launch_bounds__(128)
retile_kernel(const uint8_t* __restrict__ packed_T, int K, int N, int KT, uint8_t* __restrict__ tiled) {
    const int kt = blockIdx.x, nb = blockIdx.y;
    const int lane = threadIdx.x >> 2, q = threadIdx.x & 3;
    const int g = lane >> 2, t = lane & 3;
    const int KB = (K + 3) / 4;
    const int n = TILE_N * nb + g + 8 * (q & 1);
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // public row kb holds k = 4kb .. 4kb+3 of every column
        const int kb = (TILE_K * kt + 32 * t + 8 * i + 4 * (q >> 1)) >> 2;
        uint32_t byte = 0;
        if (n < N && kb < KB) byte = packed_T[static_cast<int64_t>(kb) * N + n];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t c = (byte >> (2 * j)) & 3u;
            const int tv = (c == 1u) - (c == 2u);           // pattern 11 -> 0
            word |= static_cast<uint32_t>(tv + 1) << (8 * j + 2 * i);
        }
    }
    const int64_t tile = static_cast<int64_t>(nb) * KT + kt;
    reinterpret_cast<uint32_t*>(tiled + tile * TILE_BYTES)[lane * 4 + q] = word;
}

// One thread per public byte.
__global__ void untile_kernel(const uint8_t* __restrict__ tiled, int K, int N, int KT, uint8_t* __restrict__ packed_T) {
    const int KB = (K + 3) / 4;
    const int64_t total = static_cast<int64_t>(KB) * N;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int kb = static_cast<int>(idx / N), n = static_cast<int>(idx % N);
        const int nb = n / TILE_N, kt = (4 * kb) / TILE_K;
        const int64_t tile = static_cast<int64_t>(nb) * KT + kt;
        const uint32_t* words = reinterpret_cast<const uint32_t*>(tiled + tile * TILE_BYTES);
        uint32_t byte = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = 4 * kb + j;
            int word, shift;
            tile_slot(n % TILE_N, k % TILE_K, word, shift);
            const int tv = static_cast<int>((words[word] >> shift) & 3u) - 1;
            const uint32_t c = (k < K) ? (tv == 1 ? 1u : (tv == -1 ? 2u : 0u)) : 0u;
            byte |= c << (2 * j);
        }
        packed_T[idx] = static_cast<uint8_t>(byte);
    }
}

}  // namespace bt

extern "C" size_t bt_tiled_bytes(int64_t K, int64_t N) {
    if (K <= 0 || N <= 0) return 0;
    return static_cast<size_t>((N + bt::TILE_N - 1) / bt::TILE_N) * static_cast<size_t>((K + bt::TILE_K - 1) / bt::TILE_K) *
           bt::TILE_BYTES;
}

extern "C" int bt_retile_packed(const uint8_t* packed_T, int64_t K, int64_t N, uint8_t* tiled, void* stream) {
    using namespace bt;
    BT_REQUIRE(packed_T && tiled, "bt_retile_packed: NULL pointer");
    BT_REQUIRE(K > 0 && N > 0, "bt_retile_packed: empty weight");
    BT_REQUIRE(aligned(tiled, 16), "bt_retile_packed: tiled buffer must be 16-byte aligned");
    BT_UNSUPPORTED_IF(K > BT_MAX_K || N > (int64_t{1} << 30), "bt_retile_packed: shape too large");
    const int KT = static_cast<int>(ceil_div<int64_t>(K, TILE_K)), NB = static_cast<int>(ceil_div<int64_t>(N, TILE_N));
    BT_UNSUPPORTED_IF(NB > 65535, "bt_retile_packed: N too large for one launch");
    BT_LAUNCH(retile_kernel, dim3(KT, NB), 128, 0, static_cast<cudaStream_t>(stream), packed_T, static_cast<int>(K),
                                                                                static_cast<int>(N), KT, tiled);
    BT_LAUNCH_OK("retile_kernel");
    return BT_OK;
}

extern "C" int bt_untile_packed(const uint8_t* tiled, int64_t K, int64_t N, uint8_t* packed_T, void* stream) {
    using namespace bt;
    BT_REQUIRE(packed_T && tiled, "bt_untile_packed: NULL pointer");
    BT_REQUIRE(K > 0 && N > 0, "bt_untile_packed: empty weight");
    BT_UNSUPPORTED_IF(K > BT_MAX_K || N > (int64_t{1} << 30), "bt_untile_packed: shape too large");
    const int KT = static_cast<int>(ceil_div<int64_t>(K, TILE_K));
    const int64_t total = ceil_div<int64_t>(K, 4) * N;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(ceil_div<int64_t>(total, 256), sm_count() * 16));
    BT_LAUNCH(untile_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), tiled, static_cast<int>(K), static_cast<int>(N), KT,
                                                                       packed_T);
    BT_LAUNCH_OK("untile_kernel");
    return BT_OK;
}
