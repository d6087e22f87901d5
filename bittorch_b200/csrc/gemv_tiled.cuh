// Decode-size packed ternary linear on the tiled layout: the HBM-bound fast path.
//
// One CTA per SM (grid = min(#SMs, column blocks)), no clusters, no global scratch.  Each
// CTA owns a contiguous run of 16-column blocks, i.e. one contiguous byte range of the
// tiled buffer, which a producer lane streams with 1-D TMA bulk copies into an mbarrier
// ring (32 KB stages, up to 96 KB) — starting BEFORE the programmatic-dependent-launch wait,
// because weights never depend on the preceding kernel, so with back-to-back layers the
// weight stream of layer i+1 overlaps the tail of layer i.
//
// After the wait the CTA (16 consumer warps) quantizes the activation rows itself (FUSED:
// per-row absmax over all of K, reciprocal scale, roundf, clamp — bit-identical to
// bt_act_quant_i8) or copies pre-quantized int8 rows, into shared memory.  Then warp w
// takes four consecutive tiles of every stage: one 16-byte vector per lane and tile, the four 2-bit planes masked in
// place (bytes (t+1)*4^i for planes 0..2, -t*64 for plane 3), each masked word a dp4a against
// the matching activation word.  Per tile and activation row: 16 logic ops shared by all rows + 16 dp4a.  When a
// warp leaves a column block it folds its planes (>> 2i), sums the four k-lanes with
// shuffles and parks 16 sums per row in its own slot of shared memory; at the end the CTA
// adds the 16 warps' slots, subtracts the row sum of the activations that met planes 0..2
// (whose codes are stored as t+1) and applies (float(acc) * sx) * scale + bias.
//
// Chained layers (bt_gemv_tiled_chained): when this kernel's output rows are the next layer's activations, the
// epilogue also publishes each row's max |y| (of the values as stored, i.e. after rounding to the output type, over
// the columns the next layer reads): one atomicMax on the float's bit pattern per CTA and row into one of
// AMAX_SLOTS words.  The next layer then takes its quantization scale from those words instead of reducing the row
// itself, so its threads quantize their share of the row as soon as it arrives: no row-maximum pass and no CTA
// barrier between the activation load and the quantizer.  Bit-identical by construction: the maximum is taken over
// exactly the values the consumer would have reduced.
//
// Algorithmic HBM bytes per call: ceil(K/4)*N + 4N (+4N bias) + x + y.
#pragma once

#include "act_quant.cuh"
#include "common.cuh"
#include "float_planes.cuh"
#include "retile.cuh"

namespace bt {

constexpr int GT_CONSUMER_WARPS = 16;
constexpr int GT_NCONS = GT_CONSUMER_WARPS * 32;
constexpr int GT_THREADS = GT_NCONS + 32;              // + one producer warp
constexpr int GT_TPW = 4;                              // consecutive tiles per consumer warp and stage
constexpr int GT_STAGE_TILES = GT_CONSUMER_WARPS * GT_TPW;
constexpr int GT_STAGE_BYTES = GT_STAGE_TILES * TILE_BYTES;   // 32 KB
constexpr int GT_MAX_STAGES = 3;                       // up to 96 KB of weights in flight per CTA
constexpr int GT_MAX_ROWS = 8;                         // activation rows per launch (accumulators live in registers)
constexpr int GT_X_PAD = 16;                           // bytes of padding per activation row in shared memory
constexpr int GT_SLOT_BUDGET = 32;                     // column blocks per CTA x padded rows, bounds the partial-sum slots
constexpr int AMAX_SLOTS = BT_AMAX_SLOTS;              // words per row that share the row-maximum atomics of a launch

struct GemvTiledParams {
    const void* X;         // FUSED: floating-point activations [M,K], row stride ldx
    const int8_t* Xq;      // else: int8 activations [M,K] contiguous
    const float* sx;       //       and their per-row scales
    const uint8_t* W;      // tiled weights
    const float* scale;
    const float* bias;
    void* Y;
    int8_t* xq_out;        // FUSED, optional: the int8 activations the kernel computed
    float* sx_out;         // FUSED, optional: their scales
    int32_t* acc_out;      // optional: int32 accumulators [M,N]
    int64_t ldx, ldy;
    int M, K, N;
    int KT;                // 128-wide k tiles per column block
    int NB;                // 16-column blocks
    int nbl_max;           // column blocks per CTA (upper bound)
    int stages;            // ring depth
    int x_dtype, y_dtype;
    int x_vec;             // activation rows can be read with vector loads
    int serialized;        // host only: launch without programmatic dependent launch (weights were just written)
    int planes;            // host only: floating-point activations as four digit planes (M = activation rows, <= 2)
    const uint32_t* amax_in;   // FUSED, optional: [M][AMAX_SLOTS] bit patterns whose maximum is the row's max |x|
    uint32_t* amax_out;        // optional: [M][AMAX_SLOTS], receives max |y as stored| over columns < amax_cols
    int amax_cols;
};

// Loads 4 consecutive activations of runtime dtype as float.
__device__ __forceinline__ void load_x4(const void* X, int dtype, int64_t idx, bool vec, int valid, float (&out)[4]) {
    if (dtype == BT_BF16) load4<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(X) + idx, vec, valid, out);
    else if (dtype == BT_F16) load4<__half>(static_cast<const __half*>(X) + idx, vec, valid, out);
    else load4<float>(static_cast<const float*>(X) + idx, vec, valid, out);
}

// The value a consumer reads back after `y` was stored as `dtype`.
__device__ __forceinline__ float rounded_as_stored(float y, int dtype) {
    if (dtype == BT_BF16) return round_through<__nv_bfloat16>(y);
    if (dtype == BT_F16) return round_through<__half>(y);
    return y;
}

// Two CTAs per SM (<= 56 registers) for the small row counts, so that the next layer's CTAs
// can move in and prefetch their weights while this layer finishes.
// MODE: how the int8 rows in shared memory come about
constexpr int GT_ROWS_INT8 = 0;    // the caller's int8 activations + scales (bt_gemv_tiled_i8)
constexpr int GT_ROWS_FUSED = 1;   // per-token int8 quantizer inside the kernel (bt_gemv_tiled, bt_gemv_tiled_chained)
constexpr int GT_ROWS_PLANES = 2;  // floating-point activations as four byte planes of a 32-bit fixed-point row
                                   // (bt_gemv_tiled_float): MR / 4 activation rows

template <int MR, int MODE>   // MR = int8 rows padded to a power of two: 1, 2, 4 or 8
__global__ void __launch_bounds__(GT_THREADS, (MR <= 2) ? 2 : 1)
gemv_tiled_kernel(const GemvTiledParams p) {
    constexpr bool FUSED = MODE == GT_ROWS_FUSED;
    BT_DYNAMIC_SMEM(smem, 128);
    const int k_pad = p.KT * TILE_K;
    const int xstride = k_pad + GT_X_PAD;
    uint8_t* s_ring = smem;
    int8_t* s_x = reinterpret_cast<int8_t*>(smem + p.stages * GT_STAGE_BYTES);             // [MR][xstride]
    int* s_part = reinterpret_cast<int*>(s_x + MR * xstride);                                // [16 warps][nbl_max][16][MR]
    int* s_rowsum = s_part + GT_CONSUMER_WARPS * p.nbl_max * TILE_N * MR;                    // [MR]
    int* s_wsum = s_rowsum + MR;                                                             // [16 warps][MR]
    float* s_wmax = reinterpret_cast<float*>(s_wsum + GT_CONSUMER_WARPS * MR);               // [16 warps][MR]
    float* s_sx = s_wmax + GT_CONSUMER_WARPS * MR;                                           // [MR]
    float* s_scale = s_sx + MR;                                                              // [nbl_max*16] weight scales
    float* s_bias = s_scale + p.nbl_max * TILE_N;                                            // [nbl_max*16]
    uint64_t* s_full = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(s_bias + p.nbl_max * TILE_N) + 7) & ~uintptr_t(7));
    uint64_t* s_empty = s_full + p.stages;
    __shared__ int s_abort;
    __shared__ uint32_t s_amax[GT_MAX_ROWS];               // this CTA's max |y| per row (bit patterns), amax_out only
    __shared__ int s_bad[GT_MAX_ROWS / 4];                 // planes mode: the activation row holds an infinity or a NaN

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int stages = p.stages;
    // this CTA's run of column blocks and tiles
    const int nb0 = static_cast<int>((static_cast<int64_t>(blockIdx.x) * p.NB) / gridDim.x);
    const int nb1 = static_cast<int>((static_cast<int64_t>(blockIdx.x + 1) * p.NB) / gridDim.x);
    const int nbl = nb1 - nb0;
    const int nt = nbl * p.KT;
    const int n_iters = (nt + GT_STAGE_TILES - 1) / GT_STAGE_TILES;
    const uint8_t* src = p.W + static_cast<int64_t>(nb0) * p.KT * TILE_BYTES;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_empty[s], GT_CONSUMER_WARPS);
        }
        s_abort = 0;
        mbar_fence_init();
    }
    if (tid < GT_MAX_ROWS) s_amax[tid] = 0u;
    if (tid < GT_MAX_ROWS / 4) s_bad[tid] = 0;
    for (int i = tid; i < GT_CONSUMER_WARPS * p.nbl_max * TILE_N * MR + MR + 2 * GT_CONSUMER_WARPS * MR; i += GT_THREADS)
        s_part[i] = 0;                                  // s_part, s_rowsum, s_wsum, s_wmax (0.0f)
    for (int c = tid; c < nbl * TILE_N; c += GT_THREADS) {   // epilogue constants: never written by a preceding kernel
        const int n = nb0 * TILE_N + c;
        s_scale[c] = (n < p.N) ? p.scale[n] : 0.0f;
        s_bias[c] = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.0f;
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == GT_CONSUMER_WARPS) {
        // ---- producer: one lane streams this CTA's contiguous byte range --------------------
        if (lane == 0) {
            int s = 0;
            uint32_t wrap_parity = 1;                        // parity of the "previous use" phase of the slot
            for (int it = 0; it < n_iters; ++it) {
                if (it >= stages) {
                    if (!mbar_wait_bounded(&s_empty[s], wrap_parity)) {
                        report_wait_timeout();
                        atomicExch(&s_abort, 1);
                        break;
                    }
                }
                const uint32_t bytes = static_cast<uint32_t>(min(GT_STAGE_TILES, nt - it * GT_STAGE_TILES)) * TILE_BYTES;
                mbar_expect_tx(&s_full[s], bytes);
                bulk_g2s(s_ring + s * GT_STAGE_BYTES, src + static_cast<int64_t>(it) * GT_STAGE_BYTES, bytes, &s_full[s]);
                if (++s == stages) { s = 0; wrap_parity ^= 1; }
            }
        }
    } else {
        // ---- consumers --------------------------------------------------------------------------
        pdl_wait();   // activations come from the preceding kernel
        if constexpr (MODE == GT_ROWS_PLANES) {
            // Floating-point activations, exact: with 2^e the smallest power of two above the row's max |x|,
            //     v[k] = rint(x[k] * 2^(30-e))          (|v| < 2^30; scaling by a power of two is exact)
            //     v    = b3 2^24 + b2 2^16 + b1 2^8 + b0  with balanced digits b in [-128, 127]
            // and digit plane p of row m becomes int8 row 4m+p of the integer pipeline.  The epilogue recombines the
            // four exact int32 accumulators in 64-bit arithmetic, so the output is the correctly rounded EXACT dot
            // product of the row as represented (elements within 2^6 of the row maximum are represented exactly,
            // the rest to 2^-30 of it) - tighter than any order of fp32 additions.
            constexpr int ROWS = MR / 4;
            const int tpr = GT_NCONS / ROWS;               // threads per activation row: whole warps
            const int m = tid / tpr, j = tid % tpr;
            const int nvec = (p.K + 3) / 4;
            const bool row_ok = m < p.M;
            const int64_t row_off = static_cast<int64_t>(m) * p.ldx;
            float x[4][4];
            float mx = 0.0f;
            int bad = 0;                                    // an infinity or a NaN in the row
            if (row_ok) {
                for (int v0 = j; v0 < nvec; v0 += 4 * tpr) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int v = v0 + u * tpr;
                        const int valid = (v < nvec) ? min(4, p.K - 4 * v) : 0;
                        if (valid > 0) load_x4(p.X, p.x_dtype, row_off + 4 * v, p.x_vec, valid, x[u]);
                        else x[u][0] = x[u][1] = x[u][2] = x[u][3] = 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float a = fabsf(x[u][i]);
                            mx = fmaxf(mx, a);
                            bad |= !(a <= 3.402823466e38f);
                        }
                }
            }
            mx = warp_max(mx);
            bad = warp_or(bad);
            if (lane == 0 && row_ok) {
                s_wmax[warp * MR + m] = mx;
                if (bad) s_bad[m] = 1;
            }
            named_barrier_sync<1>(GT_NCONS);
            float amax = 0.0f;
#pragma unroll
            for (int w = 0; w < GT_CONSUMER_WARPS; ++w) amax = fmaxf(amax, s_wmax[w * MR + (row_ok ? m : 0)]);
            const int e = planes_exponent(amax);            // amax < 2^e
            const float mult = ldexpf(1.0f, 30 - e);
            if (row_ok && j == 0) s_sx[4 * m] = ldexpf(1.0f, e - 30);
            // zero what the planes below will not write: padding rows and the tail past K
            {
                const int vecs = xstride / 16;
                const int first_tail = p.K / 16;
                for (int mm = 0; mm < MR; ++mm)
                    for (int vv = (mm >= 4 * p.M ? 0 : first_tail) + tid; vv < vecs; vv += GT_NCONS)
                        *reinterpret_cast<uint4*>(s_x + mm * xstride + vv * 16) = make_uint4(0, 0, 0, 0);
            }
            if (p.K % 16 != 0) named_barrier_sync<1>(GT_NCONS);
            int qsum[4] = {0, 0, 0, 0};
            if (row_ok) {
                const bool single = nvec <= 4 * tpr;        // the row stayed in registers
                for (int v0 = j; v0 < nvec; v0 += 4 * tpr) {
                    if (!single) {
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int v = v0 + u * tpr;
                            const int valid = (v < nvec) ? min(4, p.K - 4 * v) : 0;
                            if (valid > 0) load_x4(p.X, p.x_dtype, row_off + 4 * v, p.x_vec, valid, x[u]);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int v = v0 + u * tpr;
                        const int valid = (v < nvec) ? min(4, p.K - 4 * v) : 0;
                        if (valid <= 0) continue;
                        uint32_t w[4] = {0u, 0u, 0u, 0u};   // one word of four k per digit plane
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (i >= valid) continue;
                            int b[4];
                            balanced_digits(planes_fixed_point(x[u][i], mult), b);     // NaN -> 0; the row is flagged
#pragma unroll
                            for (int d = 0; d < 4; ++d) w[d] |= static_cast<uint32_t>(b[d] & 0xff) << (8 * i);
                        }
                        const bool counted = ((v >> 1) & 3) != 3;      // meets weight planes 0..2 (codes t+1)
#pragma unroll
                        for (int d = 0; d < 4; ++d) {
                            if (counted) qsum[d] = __dp4a(static_cast<int>(w[d]), 0x01010101, qsum[d]);
                            int8_t* dst = s_x + (4 * m + d) * xstride + 4 * v;
                            if (valid == 4) {
                                *reinterpret_cast<uint32_t*>(dst) = w[d];
                            } else {
                                for (int i = 0; i < valid; ++i) dst[i] = static_cast<int8_t>(w[d] >> (8 * i));
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                const int sum = warp_sum(qsum[d]);
                if (lane == 0 && row_ok) s_wsum[warp * MR + 4 * m + d] = sum;
            }
        } else if constexpr (FUSED) {
            // thread -> (row, 4-element vector): the 512 consumer threads are split evenly over
            // the next power of two >= M rows; thread j of a row takes vectors j, j+tpr, ...
            const int tpr = GT_NCONS / MR;                  // threads per row: 512 .. 64 (whole warps)
            const int m = tid / tpr, j = tid % tpr;
            const int nvec = (p.K + 3) / 4;
            const bool row_ok = m < p.M;
            const int64_t row_off = static_cast<int64_t>(m) * p.ldx;
            // a row that fits four vectors per thread stays in registers between the two passes
            const bool single = nvec <= 4 * tpr;
            // the producing kernel published the row maxima: no reduction pass, no barrier before the quantizer
            const bool published = p.amax_in != nullptr;
            uint32_t pub = 0u;
            if (published && row_ok) {
                const uint4* words = reinterpret_cast<const uint4*>(p.amax_in + static_cast<int64_t>(m) * AMAX_SLOTS);
#pragma unroll
                for (int q = 0; q < AMAX_SLOTS / 4; ++q) {
                    const uint4 w = __ldcg(words + q);
                    pub = max(max(pub, max(w.x, w.y)), max(w.z, w.w));
                }
            }
            float x[4][4];
            float mx = 0.0f;
            if (row_ok && (single || !published)) {
                for (int v0 = j; v0 < nvec; v0 += 4 * tpr) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {           // four independent loads in flight
                        const int v = v0 + u * tpr;
                        const int valid = (v < nvec) ? min(4, p.K - 4 * v) : 0;
                        if (valid > 0) load_x4(p.X, p.x_dtype, row_off + 4 * v, p.x_vec, valid, x[u]);
                        else x[u][0] = x[u][1] = x[u][2] = x[u][3] = 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        mx = fmaxf(fmaxf(fmaxf(mx, fabsf(x[u][0])), fmaxf(fabsf(x[u][1]), fabsf(x[u][2]))), fabsf(x[u][3]));
                }
            }
            float amax = 0.0f;
            if (published) {                                // the same condition in every thread of the CTA
                amax = __uint_as_float(pub);
            } else {
                mx = warp_max(mx);                          // a warp never straddles two rows (tpr >= 64)
                if (lane == 0 && row_ok) s_wmax[warp * MR + m] = mx;
                named_barrier_sync<1>(GT_NCONS);
#pragma unroll
                for (int w = 0; w < GT_CONSUMER_WARPS; ++w) amax = fmaxf(amax, s_wmax[w * MR + (row_ok ? m : 0)]);
            }
            // csrc/kernels/ternary_gemm_tensor_core.cu:438-440 (scale rule) and :456 (reciprocal)
            const float sxm = (amax > 1e-6f) ? __fdiv_rn(amax, 127.0f) : 1.0f;
            const float inv = __fdiv_rn(1.0f, sxm);
            if (row_ok && j == 0) {
                s_sx[m] = sxm;
                if (p.sx_out != nullptr && blockIdx.x == 0) p.sx_out[m] = sxm;
            }
            // zero what the quantizer will not write: padding rows and the tail past K
            {
                const int vecs = xstride / 16;
                const int first_tail = p.K / 16;            // first 16-byte vector that is not entirely real data
                for (int mm = 0; mm < MR; ++mm)
                    for (int vv = (mm >= p.M ? 0 : first_tail) + tid; vv < vecs; vv += GT_NCONS)
                        *reinterpret_cast<uint4*>(s_x + mm * xstride + vv * 16) = make_uint4(0, 0, 0, 0);
            }
            if (p.K % 16 != 0) named_barrier_sync<1>(GT_NCONS);   // tail bytes are rewritten below
            int qsum = 0;
            if (row_ok) {
                const bool emit = (p.xq_out != nullptr) && blockIdx.x == 0;
                for (int v0 = j; v0 < nvec; v0 += 4 * tpr) {
                    if (!single) {
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int v = v0 + u * tpr;
                            const int valid = (v < nvec) ? min(4, p.K - 4 * v) : 0;
                            if (valid > 0) load_x4(p.X, p.x_dtype, row_off + 4 * v, p.x_vec, valid, x[u]);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int v = v0 + u * tpr;
                        const int valid = (v < nvec) ? min(4, p.K - 4 * v) : 0;
                        if (valid <= 0) continue;
                        uint32_t w = 0;
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (i < valid) w |= static_cast<uint32_t>(quantize_i8(x[u][i], inv) & 0xff) << (8 * i);
                        if (((v >> 1) & 3) != 3) qsum = __dp4a(static_cast<int>(w), 0x01010101, qsum);   // planes 0..2 only
                        if (valid == 4) {
                            *reinterpret_cast<uint32_t*>(s_x + m * xstride + 4 * v) = w;
                        } else {
                            for (int i = 0; i < valid; ++i) s_x[m * xstride + 4 * v + i] = static_cast<int8_t>(w >> (8 * i));
                        }
                        if (emit)
                            for (int i = 0; i < valid; ++i)
                                p.xq_out[static_cast<int64_t>(m) * p.K + 4 * v + i] = static_cast<int8_t>(w >> (8 * i));
                    }
                }
            }
            qsum = warp_sum(qsum);
            if (lane == 0 && row_ok) s_wsum[warp * MR + m] = qsum;
        } else {
            // pre-quantized activations: copy the rows (padding rows and the tail are zero)
            const int vecs = xstride / 16;
            if (p.x_vec) {                                   // K % 16 == 0 and Xq 16-byte aligned
                for (int mm = 0; mm < MR; ++mm)
                    for (int vv = tid; vv < vecs; vv += GT_NCONS) {
                        uint4 val = make_uint4(0, 0, 0, 0);
                        if (mm < p.M && vv * 16 < p.K)
                            val = *reinterpret_cast<const uint4*>(p.Xq + static_cast<int64_t>(mm) * p.K + vv * 16);
                        *reinterpret_cast<uint4*>(s_x + mm * xstride + vv * 16) = val;
                    }
            } else {
                for (int mm = 0; mm < MR; ++mm)
                    for (int b = tid; b < xstride; b += GT_NCONS)
                        s_x[mm * xstride + b] = (mm < p.M && b < p.K) ? p.Xq[static_cast<int64_t>(mm) * p.K + b] : int8_t(0);
            }
            if (tid < MR) s_sx[tid] = (tid < p.M) ? p.sx[tid] : 0.0f;
            named_barrier_sync<1>(GT_NCONS);
            // row sums: warp w sums its share of every row
            for (int mm = 0; mm < MR; ++mm) {
                int sum = 0;
                for (int w = tid; w < k_pad / 4; w += GT_NCONS)
                    if (((w >> 1) & 3) != 3)                 // planes 0..2 only (plane 3 is stored sign-exact)
                        sum = __dp4a(*reinterpret_cast<const int*>(s_x + mm * xstride + w * 4), 0x01010101, sum);
                sum = warp_sum(sum);
                if (lane == 0) s_wsum[warp * MR + mm] = sum;
            }
        }
        named_barrier_sync<1>(GT_NCONS);      // int8 rows complete in shared memory
        if (tid < MR) {
            int sum = 0;
#pragma unroll
            for (int w = 0; w < GT_CONSUMER_WARPS; ++w) sum += s_wsum[w * MR + tid];
            s_rowsum[tid] = sum;                             // read after the final CTA barrier
        }

        // Lane (g,t), per tile: plane i / word q = four consecutive k of column g + 8(q&1),
        // k = 32t + 8i + 4(q>>1).  acc[m][i][h]: plane i of column g + 8h.
        int acc[MR][4][2];
#pragma unroll
        for (int a = 0; a < MR; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b][0] = acc[a][b][1] = 0;
        const int g = lane >> 2, t = lane & 3;
        int cur_nb = -1;                                    // column block (local) the accumulators belong to

        // folds the planes, sums the four k-lanes and parks the 16 column sums of each row
        auto flush = [&](int nb_local) {
#pragma unroll
            for (int m = 0; m < MR; ++m) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    int v = acc[m][0][h] + (acc[m][1][h] >> 2) + (acc[m][2][h] >> 4) - (acc[m][3][h] >> 6);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (t == 0) s_part[((warp * p.nbl_max + nb_local) * TILE_N + g + 8 * h) * MR + m] = v;
                    acc[m][0][h] = acc[m][1][h] = acc[m][2][h] = acc[m][3][h] = 0;
                }
            }
        };

        // Warp w takes the GT_TPW consecutive tiles GT_TPW*w .. of every stage.  No divisions in
        // the loop: slot / parity and (column block, k tile) advance incrementally.
        int s = 0;
        uint32_t parity = 0;
        int nb_local = 0, kt = GT_TPW * warp;
        while (kt >= p.KT) { kt -= p.KT; ++nb_local; }
        const uint8_t* lane_ring = s_ring + warp * (GT_TPW * TILE_BYTES) + lane * 16;
        const int8_t* lane_x = s_x + 32 * t;
        for (int it = 0; it < n_iters; ++it) {
            if (!mbar_wait_bounded(&s_full[s], parity)) {
                report_wait_timeout();
                atomicExch(&s_abort, 1);
                break;
            }
            const uint8_t* tp = lane_ring + s * GT_STAGE_BYTES;
            // one tile: mask the planes, dp4a against the lane's 32 activations of every row
            auto tile = [&](const uint4 wv, const int8_t* xk) {
                // planes 0..2: bytes (t+1)*4^i, at most 32, valid as signed; plane 3 owns the top
                // two bits, where {0x00,0x40,0x80} ^ 0x40 = {+64, 0, -64} = -t*64 as signed bytes
                int wm[4][4];
#pragma unroll
                for (int i = 0; i < 3; ++i) {
                    const uint32_t mask = 0x03030303u << (2 * i);
                    wm[i][0] = wv.x & mask; wm[i][1] = wv.y & mask; wm[i][2] = wv.z & mask; wm[i][3] = wv.w & mask;
                }
                wm[3][0] = (wv.x & 0xC0C0C0C0u) ^ 0x40404040u; wm[3][1] = (wv.y & 0xC0C0C0C0u) ^ 0x40404040u;
                wm[3][2] = (wv.z & 0xC0C0C0C0u) ^ 0x40404040u; wm[3][3] = (wv.w & 0xC0C0C0C0u) ^ 0x40404040u;
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const int4 xa = *reinterpret_cast<const int4*>(xk + m * xstride);        // words 2i + (q>>1)
                    const int4 xb = *reinterpret_cast<const int4*>(xk + m * xstride + 16);
                    const int xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc[m][i][0] = __dp4a(wm[i][0], xw[2 * i], acc[m][i][0]);
                        acc[m][i][1] = __dp4a(wm[i][1], xw[2 * i], acc[m][i][1]);
                        acc[m][i][0] = __dp4a(wm[i][2], xw[2 * i + 1], acc[m][i][0]);
                        acc[m][i][1] = __dp4a(wm[i][3], xw[2 * i + 1], acc[m][i][1]);
                    }
                }
            };
            if (nb_local < nbl && kt + GT_TPW <= p.KT) {
                // fast path: the warp's four tiles belong to one column block — straight-line code
                if (nb_local != cur_nb) {
                    if (cur_nb >= 0) flush(cur_nb);
                    cur_nb = nb_local;
                }
                uint4 wv[GT_TPW];
#pragma unroll
                for (int u = 0; u < GT_TPW; ++u) wv[u] = *reinterpret_cast<const uint4*>(tp + u * TILE_BYTES);
                const int8_t* xk = lane_x + kt * TILE_K;
#pragma unroll
                for (int u = 0; u < GT_TPW; ++u) tile(wv[u], xk + u * TILE_K);
                kt += GT_TPW;
                if (kt == p.KT) { kt = 0; ++nb_local; }
            } else {
#pragma unroll 1
                for (int u = 0; u < GT_TPW; ++u) {
                    if (nb_local < nbl) {                    // a real tile (the last stage may be short)
                        if (nb_local != cur_nb) {
                            if (cur_nb >= 0) flush(cur_nb);
                            cur_nb = nb_local;
                        }
                        tile(*reinterpret_cast<const uint4*>(tp + u * TILE_BYTES), lane_x + kt * TILE_K);
                    }
                    if (++kt == p.KT) { kt = 0; ++nb_local; }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[s]);
            if (++s == stages) { s = 0; parity ^= 1; }
            kt += GT_STAGE_TILES - GT_TPW;                   // on to this warp's tiles of the next stage
            while (kt >= p.KT) { kt -= p.KT; ++nb_local; }
        }
        if (cur_nb >= 0) flush(cur_nb);
    }
    __syncthreads();
    if (s_abort) {
        if (tid == 0) {
            // Give copies that may still be in flight a bounded chance to land before the
            // shared memory is released.
            for (int s = 0; s < stages && s < n_iters; ++s) {
                const int last_it = ((n_iters - 1 - s) / stages) * stages + s;
                mbar_wait_bounded(&s_full[s], (last_it / stages) & 1, 1u << 16);
            }
        }
        return;
    }
    // epilogue: one thread per (row, column) of this CTA's column blocks, columns fastest
    const int cols = nbl * TILE_N;
    if constexpr (MODE == GT_ROWS_PLANES) {
        // recombine the four digit planes exactly; one rounding to float, an exact power of two, then the usual
        // scale and bias.  A row that held an infinity or a NaN gives NaN (the reference's float kernel would
        // propagate them through its sum).
        for (int m = 0; m < p.M; ++m)
            for (int c = tid; c < cols; c += GT_THREADS) {
                const int n = nb0 * TILE_N + c;
                if (n >= p.N) continue;
                long long total = 0;
#pragma unroll
                for (int d = 3; d >= 0; --d) {
                    int acc = -s_rowsum[4 * m + d];
#pragma unroll
                    for (int w = 0; w < GT_CONSUMER_WARPS; ++w) acc += s_part[(w * p.nbl_max * TILE_N + c) * MR + 4 * m + d];
                    total = total * 256 + acc;
                }
                float y = __fmul_rn(__fmul_rn(__ll2float_rn(total), s_sx[4 * m]), s_scale[c]);
                if (p.bias != nullptr) y = __fadd_rn(y, s_bias[c]);
                if (s_bad[m]) y = __int_as_float(0x7fc00000);
                store_out_dt(p.Y, p.y_dtype, static_cast<int64_t>(m) * p.ldy + n, y);
            }
        return;
    }
    const bool publish = p.amax_out != nullptr;
    for (int m = 0; m < p.M; ++m) {
        float ymax = 0.0f;
        for (int c = tid; c < cols; c += GT_THREADS) {
            const int n = nb0 * TILE_N + c;
            if (n >= p.N) continue;
            int acc = -s_rowsum[m];
#pragma unroll
            for (int w = 0; w < GT_CONSUMER_WARPS; ++w) acc += s_part[(w * p.nbl_max * TILE_N + c) * MR + m];
            if (p.acc_out != nullptr) p.acc_out[static_cast<int64_t>(m) * p.N + n] = acc;
            const float y = dequant(acc, s_sx[m], s_scale[c], s_bias[c], p.bias != nullptr);
            store_out_dt(p.Y, p.y_dtype, static_cast<int64_t>(m) * p.ldy + n, y);
            // fmaxf drops a NaN operand, as the consumer's own reduction does
            if (publish && n < p.amax_cols) ymax = fmaxf(ymax, fabsf(rounded_as_stored(y, p.y_dtype)));
        }
        if (publish) {                                      // the same condition in every thread: whole warps get here
            ymax = warp_max(ymax);
            if (lane == 0 && ymax > 0.0f) atomicMax(&s_amax[m], __float_as_uint(ymax));
        }
    }
    if (publish) {
        __syncthreads();
        // non-negative floats order like their bit patterns; CTAs spread over AMAX_SLOTS words per row
        if (tid < p.M && s_amax[tid] != 0u)
            atomicMax(p.amax_out + static_cast<int64_t>(tid) * AMAX_SLOTS + (blockIdx.x % AMAX_SLOTS), s_amax[tid]);
    }
}

// ---- host side ------------------------------------------------------------------------------

static size_t gemv_tiled_smem(int mr, int k_pad, int nbl_max, int stages) {
    return static_cast<size_t>(stages) * GT_STAGE_BYTES + static_cast<size_t>(mr) * (k_pad + GT_X_PAD) +
           sizeof(int) * (static_cast<size_t>(GT_CONSUMER_WARPS) * nbl_max * TILE_N * mr + mr + 2 * GT_CONSUMER_WARPS * mr + mr +
                          2 * static_cast<size_t>(nbl_max) * TILE_N) +
           sizeof(uint64_t) * (2 * stages + 1);
}

// Rows of activations one launch can hold as int8 in shared memory next to the ring.
static int gemv_tiled_rows_per_launch(int64_t K) {
    const int64_t k_pad = ceil_div<int64_t>(K, TILE_K) * TILE_K + GT_X_PAD;
    int rows = GT_MAX_ROWS;
    while (rows > 1 && rows * k_pad > 96 * 1024) rows >>= 1;
    return rows;
}

template <int MR, int MODE>
static int launch_gemv_tiled_kernel(const GemvTiledParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = gemv_tiled_kernel<MR, MODE>;
#ifdef BT_SIMT_HOST
    (void)st;
    const int rc = ::simt::launch(kern, dim3(grid), dim3(GT_THREADS), smem, p);
    if (rc != BT_OK) set_error("gemv_tiled_kernel: %s", ::simt::error_text());
    return rc;
#else
    static std::atomic<size_t> granted[BT_MAX_DEVICES];
    if (const int rc = ensure_dynamic_smem(kern, smem, granted)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    // Programmatic dependent launch lets the kernel start (and stream its weights, read scale / bias) while its
    // predecessor drains; that is only right when the predecessor did not write them.  `serialized` launches
    // without the attribute: griddepcontrol.* are then no-ops and the kernel is ordinarily stream-ordered.
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = p.serialized ? 0 : 1;
    BT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
    return BT_OK;
#endif
}

// One launch over `p.M` <= GT_MAX_ROWS rows (planes: <= 2 activation rows = 8 int8 rows).
static int launch_gemv_tiled_rows(GemvTiledParams p, cudaStream_t st) {
    p.KT = ceil_div(p.K, TILE_K);
    p.NB = ceil_div(p.N, TILE_N);
    const int rows8 = p.planes ? 4 * p.M : p.M;               // int8 rows held in shared memory
    const int mr = (rows8 <= 1) ? 1 : (rows8 <= 2) ? 2 : (rows8 <= 4) ? 4 : 8;
    // one CTA per SM; more CTAs only when a CTA's partial-sum slots would outgrow their budget
    const int nbl_cap = std::max(1, GT_SLOT_BUDGET / mr);
    const int grid = std::max(std::min(p.NB, sm_count()), ceil_div(p.NB, nbl_cap));
    p.nbl_max = ceil_div(p.NB, grid);
    const int max_tiles = p.nbl_max * p.KT;
    p.stages = std::max(1, std::min(GT_MAX_STAGES, ceil_div(max_tiles, GT_STAGE_TILES)));
    // 227 KB per CTA, static and dynamic together: leave room for the kernel's few static words
    constexpr size_t SMEM_LIMIT = 227 * 1024 - 256;
    size_t smem = gemv_tiled_smem(mr, p.KT * TILE_K, p.nbl_max, p.stages);
    while (smem > SMEM_LIMIT && p.stages > 1) {               // long rows: a shallower weight ring makes room
        --p.stages;
        smem = gemv_tiled_smem(mr, p.KT * TILE_K, p.nbl_max, p.stages);
    }
    BT_UNSUPPORTED_IF(smem > SMEM_LIMIT, "gemv_tiled: needs %zu bytes of shared memory (K too large)", smem);
    if (p.planes) {
        if (mr == 4) return launch_gemv_tiled_kernel<4, GT_ROWS_PLANES>(p, grid, smem, st);
        return launch_gemv_tiled_kernel<8, GT_ROWS_PLANES>(p, grid, smem, st);
    }
    const bool fused = p.X != nullptr;
#define BT_GEMV_CASE(MRV)                                                                       \
    if (mr == MRV)                                                                              \
        return fused ? launch_gemv_tiled_kernel<MRV, GT_ROWS_FUSED>(p, grid, smem, st)          \
                     : launch_gemv_tiled_kernel<MRV, GT_ROWS_INT8>(p, grid, smem, st);
    BT_GEMV_CASE(1)
    BT_GEMV_CASE(2)
    BT_GEMV_CASE(4)
    BT_GEMV_CASE(8)
#undef BT_GEMV_CASE
    return BT_ERR_INVALID;
}

// Splits M rows into launches of at most gemv_tiled_rows_per_launch(K) rows over the same weights.
static int launch_gemv_tiled(const GemvTiledParams& p, cudaStream_t st) {
    // planes: two activation rows (eight int8 rows) per launch where they fit next to the partial sums, else one
    const int rows = p.planes ? ((8 * (ceil_div<int64_t>(p.K, TILE_K) * TILE_K + GT_X_PAD) <= 96 * 1024) ? 2 : 1)
                              : gemv_tiled_rows_per_launch(p.K);
    for (int m0 = 0; m0 < p.M; m0 += rows) {
        GemvTiledParams q = p;
        q.M = std::min(rows, p.M - m0);
        if (p.X != nullptr) q.X = static_cast<const char*>(p.X) + static_cast<size_t>(m0) * p.ldx * dtype_size(p.x_dtype);
        if (p.Xq != nullptr) q.Xq = p.Xq + static_cast<int64_t>(m0) * p.K;
        if (p.sx != nullptr) q.sx = p.sx + m0;
        if (p.xq_out != nullptr) q.xq_out = p.xq_out + static_cast<int64_t>(m0) * p.K;
        if (p.sx_out != nullptr) q.sx_out = p.sx_out + m0;
        if (p.acc_out != nullptr) q.acc_out = p.acc_out + static_cast<int64_t>(m0) * p.N;
        if (p.amax_in != nullptr) q.amax_in = p.amax_in + static_cast<int64_t>(m0) * AMAX_SLOTS;
        if (p.amax_out != nullptr) q.amax_out = p.amax_out + static_cast<int64_t>(m0) * AMAX_SLOTS;
        q.Y = static_cast<char*>(p.Y) + static_cast<size_t>(m0) * p.ldy * dtype_size(p.y_dtype);
        const int rc = launch_gemv_tiled_rows(q, st);
        if (rc != BT_OK) return rc;
    }
    return BT_OK;
}

static int check_gemv_tiled_args(const char* who, int64_t M, int64_t K, const uint8_t* tiled, int64_t N, const float* scale,
                                 void* Y, int y_dtype, int64_t ldy) {
    BT_REQUIRE(tiled && scale && Y, "%s: NULL pointer", who);
    BT_REQUIRE(M > 0 && K > 0 && N > 0, "%s: X is empty or weight is empty", who);
    BT_REQUIRE(valid_dtype(y_dtype), "%s: unknown output dtype %d", who, y_dtype);
    BT_REQUIRE(ldy >= N, "%s: output row stride %lld < N %lld", who, (long long)ldy, (long long)N);
    BT_REQUIRE(aligned(tiled, 16), "%s: tiled weights must be 16-byte aligned", who);
    BT_UNSUPPORTED_IF(M > BT_GEMV_MAX_M, "%s: M=%lld exceeds %d", who, (long long)M, BT_GEMV_MAX_M);
    BT_UNSUPPORTED_IF(K > BT_MAX_K, "%s: K=%lld exceeds %d", who, (long long)K, BT_MAX_K);
    BT_UNSUPPORTED_IF(N > (int64_t{1} << 30), "%s: N too large", who);
    return BT_OK;
}

static GemvTiledParams base_tiled_params(int64_t M, int64_t K, const uint8_t* tiled, int64_t N, const float* scale,
                                         const float* bias, void* Y, int y_dtype, int64_t ldy, int32_t* acc_out, int flags) {
    GemvTiledParams p = {};
    p.serialized = (flags & BT_LAUNCH_WEIGHTS_JUST_WRITTEN) != 0;
    p.W = tiled; p.scale = scale; p.bias = bias; p.Y = Y; p.acc_out = acc_out; p.ldy = ldy;
    p.M = static_cast<int>(M); p.K = static_cast<int>(K); p.N = static_cast<int>(N);
    p.y_dtype = y_dtype; p.x_dtype = BT_F32;
    return p;
}

}  // namespace bt

extern "C" int bt_gemv_tiled_i8(const int8_t* Xq, const float* sx, int64_t M, int64_t K, const uint8_t* tiled,
                                int64_t N, const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                                int32_t* acc_out, int flags, void* stream) {
    using namespace bt;
    BT_REQUIRE(Xq != nullptr && sx != nullptr, "bt_gemv_tiled_i8: NULL pointer");
    BT_REQUIRE((flags & ~BT_LAUNCH_WEIGHTS_JUST_WRITTEN) == 0, "bt_gemv_tiled_i8: unknown flags %d", flags);
    int rc = check_gemv_tiled_args("bt_gemv_tiled_i8", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc != BT_OK) return rc;
    GemvTiledParams p = base_tiled_params(M, K, tiled, N, scale, bias, Y, y_dtype, ldy, acc_out, flags);
    p.Xq = Xq; p.sx = sx;
    p.x_vec = (K % 16 == 0) && aligned(Xq, 16);
    return launch_gemv_tiled(p, static_cast<cudaStream_t>(stream));
}

extern "C" int bt_gemv_tiled(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, const uint8_t* tiled,
                             int64_t N, const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                             int8_t* xq_out, float* sx_out, int32_t* acc_out, int flags, void* stream) {
    using namespace bt;
    BT_REQUIRE(X != nullptr, "bt_gemv_tiled: NULL pointer");
    BT_REQUIRE((flags & ~BT_LAUNCH_WEIGHTS_JUST_WRITTEN) == 0, "bt_gemv_tiled: unknown flags %d", flags);
    BT_REQUIRE(valid_dtype(x_dtype), "bt_gemv_tiled: unknown activation dtype %d", x_dtype);
    BT_REQUIRE(ldx >= K, "bt_gemv_tiled: row stride %lld < K %lld", (long long)ldx, (long long)K);
    int rc = check_gemv_tiled_args("bt_gemv_tiled", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc != BT_OK) return rc;
    GemvTiledParams p = base_tiled_params(M, K, tiled, N, scale, bias, Y, y_dtype, ldy, acc_out, flags);
    p.X = X; p.x_dtype = x_dtype; p.ldx = ldx; p.xq_out = xq_out; p.sx_out = sx_out;
    p.x_vec = (K % 4 == 0) && (ldx % 4 == 0) && aligned(X, 4 * dtype_size(x_dtype));
    return launch_gemv_tiled(p, static_cast<cudaStream_t>(stream));
}

extern "C" int bt_gemv_tiled_chained(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, const uint8_t* tiled,
                                     int64_t N, const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                                     const uint32_t* amax_in, uint32_t* amax_out, int64_t amax_cols, int flags,
                                     void* stream) {
    using namespace bt;
    BT_REQUIRE(X != nullptr, "bt_gemv_tiled_chained: NULL pointer");
    BT_REQUIRE((flags & ~BT_LAUNCH_WEIGHTS_JUST_WRITTEN) == 0, "bt_gemv_tiled_chained: unknown flags %d", flags);
    BT_REQUIRE(valid_dtype(x_dtype), "bt_gemv_tiled_chained: unknown activation dtype %d", x_dtype);
    BT_REQUIRE(ldx >= K, "bt_gemv_tiled_chained: row stride %lld < K %lld", (long long)ldx, (long long)K);
    BT_REQUIRE(amax_in == nullptr || aligned(amax_in, 16), "bt_gemv_tiled_chained: amax_in must be 16-byte aligned");
    BT_REQUIRE(amax_out == nullptr || (amax_cols > 0 && amax_cols <= N),
               "bt_gemv_tiled_chained: amax_cols %lld outside 1..N", (long long)amax_cols);
    int rc = check_gemv_tiled_args("bt_gemv_tiled_chained", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc != BT_OK) return rc;
    GemvTiledParams p = base_tiled_params(M, K, tiled, N, scale, bias, Y, y_dtype, ldy, nullptr, flags);
    p.X = X; p.x_dtype = x_dtype; p.ldx = ldx;
    p.x_vec = (K % 4 == 0) && (ldx % 4 == 0) && aligned(X, 4 * dtype_size(x_dtype));
    p.amax_in = amax_in; p.amax_out = amax_out; p.amax_cols = static_cast<int>(amax_cols);
    return launch_gemv_tiled(p, static_cast<cudaStream_t>(stream));
}

extern "C" int bt_gemv_tiled_float(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, const uint8_t* tiled,
                                   int64_t N, const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                                   int flags, void* stream) {
    using namespace bt;
    BT_REQUIRE(X != nullptr, "bt_gemv_tiled_float: NULL pointer");
    BT_REQUIRE((flags & ~BT_LAUNCH_WEIGHTS_JUST_WRITTEN) == 0, "bt_gemv_tiled_float: unknown flags %d", flags);
    BT_REQUIRE(valid_dtype(x_dtype), "bt_gemv_tiled_float: unknown activation dtype %d", x_dtype);
    BT_REQUIRE(ldx >= K, "bt_gemv_tiled_float: row stride %lld < K %lld", (long long)ldx, (long long)K);
    int rc = check_gemv_tiled_args("bt_gemv_tiled_float", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc != BT_OK) return rc;
    // digits reach -128: half the K of the int8 kernels keeps every 32-bit partial sum exact
    BT_UNSUPPORTED_IF(K > BT_MAX_K / 2, "bt_gemv_tiled_float: K=%lld exceeds %d", (long long)K, BT_MAX_K / 2);
    GemvTiledParams p = base_tiled_params(M, K, tiled, N, scale, bias, Y, y_dtype, ldy, nullptr, flags);
    p.X = X; p.x_dtype = x_dtype; p.ldx = ldx; p.planes = 1;
    p.x_vec = (K % 4 == 0) && (ldx % 4 == 0) && aligned(X, 4 * dtype_size(x_dtype));
    return launch_gemv_tiled(p, static_cast<cudaStream_t>(stream));
}
