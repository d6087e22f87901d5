// Decode-size (M <= 16) packed ternary linear on int8 activations, compatibility path on the
// PUBLIC [ceil(K/4), N] buffer (used by the stateless functional API when no tiled copy of
// the weights exists; modules run gemv_tiled.cuh instead).
//
// A thread-block cluster of S CTAs splits K for one block of 128 output columns, every CTA
// accumulates an int32 partial tile in its own shared memory (shared-memory LUT decode +
// dp4a), and after a cluster barrier each CTA reduces a slice of the columns over
// distributed shared memory and applies the epilogue.  No global scratch.
#pragma once

#include "common.cuh"

namespace bt {

constexpr int GV_X_PAD = 16;                               // row padding of the activation slice (bank spread)

struct GemvParams {
    const int8_t* Xq;
    const float* sx;
    const uint8_t* W;      // public packed weights [ceil(K/4), N]
    const float* scale;
    const float* bias;
    void* Y;
    int32_t* acc_out;
    int64_t ldy;
    int M, K, N;
    int KT;                // packed rows in total
    int slice_max;         // max packed rows per CTA
    int y_dtype;
    int x_vec;             // activation rows can be copied 16 bytes at a time
};

// Copies this CTA's K slice of the int8 activations into shared memory (rows >= M and
// bytes past K are zero) and leaves the per-row sums of the slice in s_rowsum.
// Called by the `nthreads` consumer threads only; `bar_id` is their named barrier.
template <int M_PAD>
__device__ __forceinline__ void stage_activations(const GemvParams& p, int k_begin, int slice_bytes, int xstride,
                                                  int8_t* s_x, int* s_rowsum, int tid, int nthreads, int bar_id) {
    const int k_valid = min(slice_bytes, max(0, p.K - k_begin));   // bytes of real data per row
    if (p.x_vec) {
        const int vec_per_row = slice_bytes / 16;                   // slice_bytes is a multiple of 32
        for (int idx = tid; idx < M_PAD * vec_per_row; idx += nthreads) {
            const int m = idx / vec_per_row, v = idx % vec_per_row;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (m < p.M && v * 16 < k_valid)                        // K % 16 == 0 here, so vectors are all-or-nothing
                val = *reinterpret_cast<const uint4*>(p.Xq + static_cast<int64_t>(m) * p.K + k_begin + v * 16);
            *reinterpret_cast<uint4*>(s_x + m * xstride + v * 16) = val;
        }
    } else {
        for (int idx = tid; idx < M_PAD * slice_bytes; idx += nthreads) {
            const int m = idx / slice_bytes, b = idx % slice_bytes;
            int8_t val = 0;
            if (m < p.M && b < k_valid) val = p.Xq[static_cast<int64_t>(m) * p.K + k_begin + b];
            s_x[m * xstride + b] = val;
        }
    }
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    for (int m = warp; m < M_PAD; m += nwarps) {
        int s = 0;
        for (int w = lane; w < slice_bytes / 4; w += 32)
            s = __dp4a(*reinterpret_cast<const int*>(s_x + m * xstride + w * 4), 0x01010101, s);
        s = warp_sum(s);
        if (lane == 0) s_rowsum[m] = s;
    }
}

// Cluster reduction + epilogue.  s_acc is [cols][M_PAD] int32 in every CTA of the
// cluster; CTA `rank` finishes columns [rank*cols/S, (rank+1)*cols/S).
// `sub_rowsum`: the partial sums still contain +sum(x) per row (tiled kernel).
template <int M_PAD>
__device__ __forceinline__ void cluster_reduce_store(const GemvParams& p, const int* s_acc, const int* s_rowsum,
                                                     int cols, int n_base, uint32_t rank, uint32_t S,
                                                     bool sub_rowsum, int tid, int nthreads) {
    const int my_cols = cols / static_cast<int>(S);
    for (int idx = tid; idx < my_cols * M_PAD; idx += nthreads) {
        const int m = idx / my_cols;
        const int nl = static_cast<int>(rank) * my_cols + idx % my_cols;
        const int n = n_base + nl;
        if (m >= p.M || n >= p.N) continue;
        int acc = 0;
        for (uint32_t r = 0; r < S; ++r) {
            acc += ld_dsmem_s32(&s_acc[nl * M_PAD + m], r);
            if (sub_rowsum) acc -= ld_dsmem_s32(&s_rowsum[m], r);
        }
        if (p.acc_out != nullptr) p.acc_out[static_cast<int64_t>(m) * p.N + n] = acc;
        const float y = dequant(acc, p.sx[m], p.scale[n], p.bias ? p.bias[n] : 0.0f, p.bias != nullptr);
        store_out_dt(p.Y, p.y_dtype, static_cast<int64_t>(m) * p.ldy + n, y);
    }
}

// ------------------------------------------------------------------------------------
// Compatibility path: public [ceil(K/4), N] layout.
// grid = (S, ceil(N/128)), cluster = (S,1,1), block = 128 threads.
// ------------------------------------------------------------------------------------
constexpr int GP_COLS = 128;
constexpr int GP_THREADS = 128;

template <int M_PAD>
__global__ void __launch_bounds__(GP_THREADS)
gemv_packed_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int xstride = p.slice_max * 4 + GV_X_PAD;
    int8_t* s_x = reinterpret_cast<int8_t*>(smem);
    int* s_acc = reinterpret_cast<int*>(s_x + ((M_PAD * xstride + 15) / 16) * 16);
    int* s_rowsum = s_acc + GP_COLS * M_PAD;
    __shared__ uint32_t s_lut[256];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t S = cluster_nctarank(), rank = cluster_ctarank();
    const int n_base = blockIdx.y * GP_COLS;
    // K is split in units of 8 packed rows (32 activations bytes) so that every slice
    // of the activations starts 16-byte aligned.
    const int units = (p.KT + 7) / 8;
    const int kb0 = static_cast<int>((static_cast<int64_t>(rank) * units) / S) * 8;
    const int kb1 = min(static_cast<int>((static_cast<int64_t>(rank + 1) * units) / S) * 8, p.KT);
    const int nrows = max(kb1 - kb0, 0);

    // byte -> four int8 in {-1,0,+1}; pattern 11 decodes to 0 (quant/ternary_packed.py:112-115)
    for (int b = tid; b < 256; b += GP_THREADS) {
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = (b >> (2 * j)) & 3;
            const int tval = (c == 1) - (c == 2);
            v |= static_cast<uint32_t>(tval & 0xff) << (8 * j);
        }
        s_lut[b] = v;
    }
    for (int i = tid; i < GP_COLS * M_PAD; i += GP_THREADS) s_acc[i] = 0;
    pdl_launch_dependents();
    pdl_wait();
    // slice rows are 4 bytes (one packed row = 4 k); pad to a multiple of 32 bytes for the vector copy
    const int slice_bytes = ((nrows * 4 + 31) / 32) * 32;
    stage_activations<M_PAD>(p, kb0 * 4, slice_bytes, xstride, s_x, s_rowsum, tid, GP_THREADS, 1);
    __syncthreads();

    const int n = n_base + lane * 4;
    const bool vec = (p.N % 4 == 0);
    int acc[4][M_PAD];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int m = 0; m < M_PAD; ++m) acc[j][m] = 0;

    for (int r = warp; r < nrows; r += GP_THREADS / 32) {
        const uint8_t* rowp = p.W + static_cast<int64_t>(kb0 + r) * p.N;
        uint32_t w = 0;
        if (vec) {
            if (n < p.N) w = *reinterpret_cast<const uint32_t*>(rowp + n);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (n + j < p.N) w |= static_cast<uint32_t>(rowp[n + j]) << (8 * j);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int wt = static_cast<int>(s_lut[(w >> (8 * j)) & 0xff]);
#pragma unroll
            for (int m = 0; m < M_PAD; ++m)
                acc[j][m] = __dp4a(wt, *reinterpret_cast<const int*>(s_x + m * xstride + r * 4), acc[j][m]);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int m = 0; m < M_PAD; ++m) atomicAdd(&s_acc[(lane * 4 + j) * M_PAD + m], acc[j][m]);
    __syncthreads();
    cluster_sync_all();
    cluster_reduce_store<M_PAD>(p, s_acc, s_rowsum, GP_COLS, n_base, rank, S, false, tid, GP_THREADS);
    cluster_sync_all();
}

// ---- host side -------------------------------------------------------------------------

static int pick_split(int col_blocks, int k_units, int min_units_per_cta) {
    // Testing / tuning override (BT_TUNE_GEMV_SPLIT): 1, 2, 4 or 8.
    {
        const int v = tuning(BT_TUNE_GEMV_SPLIT);
        if (v == 1 || v == 2 || v == 4 || v == 8) return (k_units >= v) ? v : 1;
    }
    int S = 1;
    const int want = 3 * sm_count();
    while (S < 8 && col_blocks * S < want && k_units / (2 * S) >= min_units_per_cta) S *= 2;
    return S;
}

template <typename Kern>
static int launch_cluster(Kern kern, const char* name, dim3 grid, dim3 block, size_t smem, int S, cudaStream_t st,
                          const GemvParams& p) {
    BT_UNSUPPORTED_IF(smem > 227 * 1024, "%s: needs %zu bytes of shared memory (K too large for this M)", name, smem);
    static std::atomic<size_t> granted[BT_MAX_DEVICES];      // one array per kernel instantiation (Kern)
    if (const int rc = ensure_dynamic_smem(kern, smem, granted)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = S;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    BT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
    return BT_OK;
}

static int check_gemv_args(const char* who, const int8_t* Xq, const float* sx, int64_t M, int64_t K, const uint8_t* W,
                           int64_t N, const float* scale, void* Y, int y_dtype, int64_t ldy) {
    BT_REQUIRE(Xq && sx && W && scale && Y, "%s: NULL pointer", who);
    BT_REQUIRE(M > 0 && K > 0 && N > 0, "%s: X is empty or weight is empty", who);
    BT_REQUIRE(valid_dtype(y_dtype), "%s: unknown output dtype %d", who, y_dtype);
    BT_REQUIRE(ldy >= N, "%s: output row stride %lld < N %lld", who, (long long)ldy, (long long)N);
    BT_UNSUPPORTED_IF(K > BT_MAX_K, "%s: K=%lld exceeds %d", who, (long long)K, BT_MAX_K);
    BT_UNSUPPORTED_IF(N > (int64_t{1} << 30), "%s: N too large", who);
    return BT_OK;
}

static GemvParams make_params(const int8_t* Xq, const float* sx, int64_t M, int64_t K, const uint8_t* W, int64_t N,
                              const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                              int32_t* acc_out) {
    GemvParams p;
    p.Xq = Xq; p.sx = sx; p.W = W; p.scale = scale; p.bias = bias; p.Y = Y; p.acc_out = acc_out; p.ldy = ldy;
    p.M = static_cast<int>(M); p.K = static_cast<int>(K); p.N = static_cast<int>(N);
    p.y_dtype = y_dtype;
    p.x_vec = (K % 16 == 0) && aligned(Xq, 16);
    p.KT = 0; p.slice_max = 0;
    return p;
}

}  // namespace bt

extern "C" int bt_gemv_packed_i8(const int8_t* Xq, const float* sx, int64_t M, int64_t K, const uint8_t* packed_T,
                                 int64_t N, const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                                 int32_t* acc_out, void* stream) {
    using namespace bt;
    int rc = check_gemv_args("bt_gemv_packed_i8", Xq, sx, M, K, packed_T, N, scale, Y, y_dtype, ldy);
    if (rc != BT_OK) return rc;
    BT_UNSUPPORTED_IF(M > BT_GEMV_MAX_M, "bt_gemv_packed_i8: M=%lld exceeds %d", (long long)M, BT_GEMV_MAX_M);
    BT_REQUIRE(N % 4 != 0 || aligned(packed_T, 4), "bt_gemv_packed_i8: packed weights must be 4-byte aligned");
    GemvParams p = make_params(Xq, sx, M, K, packed_T, N, scale, bias, Y, y_dtype, ldy, acc_out);
    p.KT = static_cast<int>(ceil_div<int64_t>(K, 4));
    const int NBc = static_cast<int>(ceil_div<int64_t>(N, GP_COLS));
    const int m_pad = (M <= 4) ? 4 : ((M <= 8) ? 8 : 16);
    int S = pick_split(NBc, p.KT, 16);
    while (S < 8 && static_cast<int64_t>(m_pad) * ceil_div(p.KT, S) * 4 > 64 * 1024 && p.KT / (2 * S) >= 1) S *= 2;
    p.slice_max = ceil_div(ceil_div(p.KT, 8), S) * 8;             // packed rows per CTA, in units of 8 rows
    const int xstride = p.slice_max * 4 + GV_X_PAD;
    const size_t smem = ((static_cast<size_t>(m_pad) * xstride + 15) / 16) * 16 + sizeof(int) * (GP_COLS * m_pad + m_pad);
    dim3 grid(S, NBc), block(GP_THREADS);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (m_pad == 4) return launch_cluster(gemv_packed_kernel<4>, "gemv_packed_kernel<4>", grid, block, smem, S, st, p);
    if (m_pad == 8) return launch_cluster(gemv_packed_kernel<8>, "gemv_packed_kernel<8>", grid, block, smem, S, st, p);
    return launch_cluster(gemv_packed_kernel<16>, "gemv_packed_kernel<16>", grid, block, smem, S, st, p);
}
