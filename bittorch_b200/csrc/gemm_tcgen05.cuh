// Prefill-size packed ternary linear on int8 activations: tcgen05 (5th-gen tensor core)
// GEMM with accumulators in tensor memory.
//
// Persistent kernel, one CTA per SM, output tile 128 (rows of X) x BN (output columns, 256 / 128 / 64),
// K consumed in blocks of 128.  Warp roles:
//   warp 0       producer: two TMA tensor loads per K block: the int8 activation tile (up to 128 rows x 128 B,
//                128-byte swizzle) and the block's 2-bit weight tiles (the tiled buffer seen as [column block][K])
//   warp 1       MMA issuer: the whole warp runs the loop, one elected lane issues each K block as one
//                instruction burst (4 x tcgen05.mma.kind::i8 128xBNx32, polls of the next block's barriers,
//                commits that free the stage / publish the accumulator)
//   warps 2-5    epilogue: tcgen05.ld of the int32 accumulators, un-scale, dequantise, store
//   warps 6-13   unpack: 2-bit tiles -> unsigned bytes t+1 in the K-major 128-byte-swizzled B tile
// Weights enter the MMA as u8 codes t+1 (one shift and one mask per four weights, four
// 16-byte shared-memory stores per lane and tile); the epilogue subtracts the row sum of the
// int8 activations, which the activation quantizer provides.
// Accumulators are double-buffered in the 512 TMEM columns so the epilogue of one tile
// overlaps the main loop of the next.
// A second instantiation (SPLIT) serves batches of up to 32 rows: one 128 x 256 tile per thread-block
// cluster, K split over the cluster's CTAs, partial accumulators exchanged through distributed shared memory.
// The CTA-pair kernel (cta_group::2) for large batches is in gemm_tcgen05_2cta.cuh.
// Algorithmic work per call: 2*M*N*K integer ops.
#pragma once

#include <cuda.h>   // CUtensorMap types only; the encoder is looked up at run time

#include <mutex>

#include "common.cuh"
#include "retile.cuh"

namespace bt {

constexpr int GM_BM = 128;
constexpr int GM_BK = 128;                       // bytes = int8 elements per K block
constexpr int GM_A_BYTES = GM_BM * GM_BK;        // 16 KB activation tile
constexpr int GM_UNPACK_WARPS = 8;
constexpr int GM_UNPACK_GROUPS = 2;              // groups of unpack warps that work on alternate K blocks
constexpr int GM_GROUP_WARPS = GM_UNPACK_WARPS / GM_UNPACK_GROUPS;
constexpr int GM_EPI_WARPS = 4;
constexpr int GM_THREADS = (2 + GM_EPI_WARPS + GM_UNPACK_WARPS) * 32;          // 448

// Per output-tile width BN: the load ring (activation tile + 2-bit weight tiles, filled by
// TMA) is deep because its latency is a global-memory round trip, the ring of unpacked
// weight tiles is shallow because it is filled from shared memory.
// Powers of two: the MMA issuer derives slot and phase from one block counter with masks and shifts.
// NL is the depth of the load ring when the activation tile has all 128 rows; with fewer rows
// (M <= 120) only those rows are copied and the ring gets deeper (gemm_ring_depth).
template <int BN> struct GemmCfg;
template <> struct GemmCfg<256> { static constexpr int NL = 4, NB = 4; };
template <> struct GemmCfg<128> { static constexpr int NL = 8, NB = 4; };
template <> struct GemmCfg<64> { static constexpr int NL = 8, NB = 4; };
constexpr int GM_MAX_NL = 32;
constexpr size_t GM_SMEM_LIMIT = 227 * 1024;

template <int BN> __host__ __device__ constexpr int gm_p_tiles() { return BN / TILE_N; }                 // packed tiles per stage
template <int BN> __host__ __device__ constexpr int gm_p_bytes() { return gm_p_tiles<BN>() * TILE_BYTES; }
template <int BN> __host__ __device__ constexpr int gm_b_bytes() { return BN * GM_BK; }
template <int BN> constexpr size_t gm_smem_bytes(int nl, int a_rows) {
    return 1024 /*alignment slack*/ + static_cast<size_t>(nl) * (static_cast<size_t>(a_rows) * GM_BK + gm_p_bytes<BN>()) +
           static_cast<size_t>(GemmCfg<BN>::NB) * gm_b_bytes<BN>() + 1024 /*barriers*/;
}

// Position in a ring of mbarrier-guarded stages (no divisions in the loops).
struct RingPos {
    int s = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance(int n) {
        if (++s == n) { s = 0; phase ^= 1; }
    }
    __device__ __forceinline__ void advance_by(int n, int step) {
        for (int i = 0; i < step; ++i) advance(n);
    }
};

struct GemmParams {
    const uint8_t* tiled;
    const float* sx;
    const int32_t* xsum;   // per-row sums of the int8 activations
    const float* scale;
    const float* bias;
    void* Y;
    int32_t* acc_out;
    int64_t ldy;
    int M, K, N;
    int KT;        // 128-wide k tiles in the tiled layout
    int NB;        // 16-column blocks in the tiled layout
    int y_dtype;
    int a_rows;    // rows of the activation tile that are copied (a multiple of 8; 128 unless M is small)
    int nl_log2;   // log2 of the load ring's depth
};

// ---- tcgen05 / TMA PTX wrappers ----------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One K block (128 inputs = four K=32 MMAs) issued as a single instruction sequence:
//   MMA, MMA, poll(next block's two "full" barriers), MMA, MMA, commit(c0), commit(c1)
// and only then the two poll predicates are read.  The issuing thread has about one MMA time (128 cycles) of
// slack between bursts; with one asm statement per instruction (a setp per MMA, a selp right behind every poll) the
// bookkeeping of a K block alone cost 200-300 cycles and the tensor pipe ran at 60 % of its rate.
// Returns non-zero when both polled barriers had already completed their phase.
// PAIR: cta_group::2 MMAs, commits multicast to both CTAs of the pair.
template <bool PAIR>
__device__ __forceinline__ uint32_t umma_i8_burst4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate_first, uint64_t* poll0, uint32_t parity0, uint64_t* poll1,
                                                   uint32_t parity1, uint64_t* commit0, uint64_t* commit1) {
    uint32_t ok0, ok1;
#define BT_MMA1_AT(off) "add.s64 ta, %3, " #off ";\n\tadd.s64 tb, %4, " #off ";\n\ttcgen05.mma.cta_group::1.kind::i8 [%2], ta, tb, %5, pt;\n\t"
#define BT_MMA2_AT(off) "add.s64 ta, %3, " #off ";\n\tadd.s64 tb, %4, " #off ";\n\ttcgen05.mma.cta_group::2.kind::i8 [%2], ta, tb, %5, pt;\n\t"
#define BT_POLLS "mbarrier.test_wait.parity.shared::cta.b64 p0, [%7], %8;\n\tmbarrier.test_wait.parity.shared::cta.b64 p1, [%9], %10;\n\t"
    if (PAIR) {
        asm volatile(
            "{\n\t.reg .pred pa, pt, p0, p1;\n\t.reg .b64 ta, tb;\n\t"
            "setp.ne.b32 pa, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%2], %3, %4, %5, pa;\n\t"
            BT_MMA2_AT(2) BT_POLLS BT_MMA2_AT(4) BT_MMA2_AT(6)
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%11], %13;\n\t"
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%12], %13;\n\t"
            "selp.u32 %0, 1, 0, p0;\n\tselp.u32 %1, 1, 0, p1;\n\t}"
            : "=r"(ok0), "=r"(ok1)
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(smem_u32(poll0)), "r"(parity0),
              "r"(smem_u32(poll1)), "r"(parity1), "r"(smem_u32(commit0)), "r"(smem_u32(commit1)), "h"(static_cast<uint16_t>(3))
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred pa, pt, p0, p1;\n\t.reg .b64 ta, tb;\n\t"
            "setp.ne.b32 pa, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%2], %3, %4, %5, pa;\n\t"
            BT_MMA1_AT(2) BT_POLLS BT_MMA1_AT(4) BT_MMA1_AT(6)
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%11];\n\t"
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%12];\n\t"
            "selp.u32 %0, 1, 0, p0;\n\tselp.u32 %1, 1, 0, p1;\n\t}"
            : "=r"(ok0), "=r"(ok1)
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(smem_u32(poll0)), "r"(parity0),
              "r"(smem_u32(poll1)), "r"(parity1), "r"(smem_u32(commit0)), "r"(smem_u32(commit1))
            : "memory");
    }
#undef BT_MMA1_AT
#undef BT_MMA2_AT
#undef BT_POLLS
    return ok0 & ok1;
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 B apart,
// 8-row groups 1024 B apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);       // start address
    d |= static_cast<uint64_t>(1) << 16;                            // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                    // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                            // version
    d |= static_cast<uint64_t>(2) << 61;                            // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D = s32, A = s8 (activations), B = u8 (weight codes), both K-major,
// M = 128, N = BN.
template <int BN> __host__ __device__ constexpr uint32_t gm_idesc() {
    return (2u << 4) | (1u << 7) | (0u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(GM_BM >> 4) << 24);
}

// Stores up to 32 consecutive outputs of one row (16-byte stores when the row segment is
// complete and aligned).
__device__ __forceinline__ void store_row32(void* Y, int y_dtype, int64_t base, const float (&y)[32], int valid) {
    const bool full = valid >= 32;
    if (y_dtype == BT_F32) {
        float* out = reinterpret_cast<float*>(Y) + base;
        if (full && aligned(out, 16)) {
#pragma unroll
            for (int c = 0; c < 32; c += 4)
                *reinterpret_cast<float4*>(out + c) = make_float4(y[c], y[c + 1], y[c + 2], y[c + 3]);
        } else {
#pragma unroll
            for (int c = 0; c < 32; ++c)
                if (c < valid) out[c] = y[c];
        }
    } else {
        uint16_t* out = reinterpret_cast<uint16_t*>(Y) + base;
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
            if (y_dtype == BT_F16) {
                __half2 h = __floats2half2_rn(y[c], y[c + 1]);
                pk[c / 2] = *reinterpret_cast<uint32_t*>(&h);
            } else {
                __nv_bfloat162 h = __floats2bfloat162_rn(y[c], y[c + 1]);
                pk[c / 2] = *reinterpret_cast<uint32_t*>(&h);
            }
        }
        if (full && aligned(out, 16)) {
#pragma unroll
            for (int c = 0; c < 16; c += 4)
                *reinterpret_cast<uint4*>(out + 2 * c) = make_uint4(pk[c], pk[c + 1], pk[c + 2], pk[c + 3]);
        } else {
#pragma unroll
            for (int c = 0; c < 32; ++c)
                if (c < valid) out[c] = static_cast<uint16_t>(pk[c / 2] >> (16 * (c & 1)));
        }
    }
}

// Bounded mbarrier wait that also gives up when another role has already failed.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_BUDGET_NS) break;
        }
    }
    report_wait_timeout();
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ uint32_t map_to_cta(const void* local_smem_ptr, uint32_t cta_rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_smem_ptr)), "r"(cta_rank));
    return remote;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, int a, int b, int c, int d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_cluster_s32(uint32_t cluster_addr, int v) {
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// The same wait run by all 32 lanes of a converged warp, with a warp-uniform result.
__device__ __forceinline__ bool wait_or_abort_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, wait_or_abort(bar, parity, abort_flag));
}
__device__ __forceinline__ bool elect_one_lane() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// SPLIT (M <= 32 rows): one output tile per thread-block cluster, CTA r of the cluster contracts the r-th slice of
// K, and the partial accumulators meet in distributed shared memory: CTA r finishes BN / cluster-size columns of the
// tile, so every CTA sends each owner its rows x columns block, adds what it received and stores.  The issue of a
// tcgen05.mma costs about as much as a 128 x 256 x 32 MMA runs, whatever its width, so a narrow batch is spread
// over the SMs by splitting K under full-width tiles, not by narrowing the tiles.
template <int BN, bool SPLIT>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
    constexpr int NB = GemmCfg<BN>::NB;
    // With few activation rows only those rows are copied per K block and the ring's stages are that much closer
    // together (and there are more of them).  The MMA still reads 128 rows from a stage's base: the rows past
    // a_rows are whatever follows in shared memory, and the accumulator rows they produce are never stored.
    const int NL = 1 << p.nl_log2;
    const int a_stride = p.a_rows * GM_BK;
    constexpr int P_TILES = gm_p_tiles<BN>(), P_BYTES = gm_p_bytes<BN>(), B_BYTES = gm_b_bytes<BN>();
    constexpr uint32_t TMEM_COLS = 2 * BN;               // double-buffered accumulator (power of two >= 128)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_a = smem;                                 // [NL] activation tiles, 128-byte swizzle
    uint8_t* s_b = s_a + NL * a_stride;                  // [NB] unpacked weight tiles, 128-byte swizzle
    uint8_t* s_p = s_b + NB * B_BYTES;                   // [NL] packed 2-bit tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + NL * P_BYTES);
    uint64_t* full_load = bars;                          // [NL] producer -> unpack, MMA
    uint64_t* empty_load = full_load + NL;               // [NL] MMA -> producer
    uint64_t* full_b = empty_load + NL;                  // [NB] unpack -> MMA
    uint64_t* empty_b = full_b + NB;                     // [NB] MMA -> unpack
    uint64_t* tmem_full = empty_b + NB;                  // [2] MMA -> epilogue
    uint64_t* tmem_empty = tmem_full + 2;                // [2] epilogue -> MMA
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    int* s_stage = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 1024);   // SPLIT: [cluster size][a_rows][BN / cluster size]
    __shared__ int s_abort_storage;
    volatile int* s_abort = &s_abort_storage;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (p.M + GM_BM - 1) / GM_BM;
    const int n_tiles = (p.N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const int k_blocks_all = (p.K + GM_BK - 1) / GM_BK;
    // SPLIT: this CTA's tile and K slice; otherwise a persistent loop over tiles and all of K
    const int csize = SPLIT ? static_cast<int>(cluster_nctarank()) : 1;
    const int crank = SPLIT ? static_cast<int>(cluster_ctarank()) : 0;
    const int kb_lo = SPLIT ? crank * k_blocks_all / csize : 0;
    const int k_blocks = SPLIT ? (crank + 1) * k_blocks_all / csize - kb_lo : k_blocks_all;
    const int tile_first = SPLIT ? static_cast<int>(blockIdx.x) / csize : static_cast<int>(blockIdx.x);
    const int tile_step = SPLIT ? total_tiles : static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NL; ++s) {
            mbar_init(&full_load[s], 1);
            mbar_init(&empty_load[s], 1);
        }
        for (int s = 0; s < NB; ++s) {
            mbar_init(&full_b[s], GM_GROUP_WARPS);
            mbar_init(&empty_b[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], GM_EPI_WARPS);
        }
        s_abort_storage = 0;
        mbar_fence_init();
    }
    if (warp == 2) tmem_alloc(s_tmem, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    if (SPLIT) cluster_sync_all();   // every CTA of the cluster has started: its shared memory may be written
    pdl_launch_dependents();
    pdl_wait();   // activations (and their scales) come from the preceding kernel

    if (warp == 0) {
        // ================= producer =================
        if (lane == 0) {
            RingPos ld;
            for (int tile = tile_first; tile < total_tiles && !*s_abort; tile += tile_step) {
                const int mt = tile % m_tiles, nt = tile / m_tiles;
                const int nb0 = nt * P_TILES;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!wait_or_abort(&empty_load[ld.s], ld.phase ^ 1, s_abort)) { ok = false; break; }
                    // two tensor copies per stage: issuing one bulk copy per 512-byte tile from this single
                    // thread cost more than the MMAs of the stage.  Column blocks past the end arrive as zeros
                    // (and count their bytes); their outputs are never stored.
                    mbar_expect_tx(&full_load[ld.s], a_stride + P_BYTES);
                    tma_load_2d(s_a + ld.s * a_stride, &map_x, (kb_lo + kb) * GM_BK, mt * GM_BM, &full_load[ld.s]);
                    tma_load_2d(s_p + ld.s * P_BYTES, &map_w, (kb_lo + kb) * (TILE_BYTES / 4), nb0, &full_load[ld.s]);
                    ld.advance(NL);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        // The whole warp runs the loop and one elected lane issues.  With warp-uniform control flow the compiler keeps
        // the block counter, descriptors and barrier addresses in uniform registers, which is what the tcgen05
        // instructions take; computed by a single diverged lane they had to be moved there for every K block, and
        // everything this warp does between two bursts delays the next one (the slack is about one MMA, 128 cycles).
        // For the same reason slot and phase of both rings come from one block counter with masks and shifts.
        {
            static_assert((NB & (NB - 1)) == 0, "ring depths must be powers of two");
            static_assert(GM_BK == 128, "umma_i8_burst4 issues four K=32 MMAs");
            const uint64_t desc_a0 = umma_desc_sw128(smem_u32(s_a)), desc_b0 = umma_desc_sw128(smem_u32(s_b));
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);   // the same value, provably warp-uniform
            const uint32_t nl_mask = NL - 1, nl_log2 = p.nl_log2, a_step = a_stride >> 4;
            uint32_t cnt = 0, tcount = 0;      // K blocks / tiles issued so far
            bool ready = false;
            for (int tile = tile_first; tile < total_tiles; tile += tile_step, ++tcount) {
                if (__any_sync(0xffffffffu, *s_abort != 0)) break;
                const uint32_t a = tcount & 1;
                if (!wait_or_abort_warp(&tmem_empty[a], ((tcount >> 1) & 1) ^ 1, s_abort)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_u + a * BN;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    const uint32_t sl = cnt & nl_mask, sb = cnt & (NB - 1), nx = cnt + 1, nsl = nx & nl_mask, nsb = nx & (NB - 1);
                    if (!ready && (!wait_or_abort_warp(&full_load[sl], (cnt >> nl_log2) & 1, s_abort) || !wait_or_abort_warp(&full_b[sb], (cnt / NB) & 1, s_abort))) { ok = false; break; }
                    tc_fence_after();
                    uint32_t polled = 0;
                    if (elect_one_lane())   // the commits free the activation + packed tiles of this K block and its unpacked weight tile
                        polled = umma_i8_burst4<false>(d_tmem, desc_a0 + sl * a_step, desc_b0 + sb * (B_BYTES >> 4), gm_idesc<BN>(),
                                                       kb > 0 ? 1u : 0u, &full_load[nsl], (nx >> nl_log2) & 1, &full_b[nsb], (nx / NB) & 1,
                                                       &empty_load[sl], &empty_b[sb]);
                    ready = __any_sync(0xffffffffu, polled != 0);
                    cnt = nx;
                }
                if (!ok) break;
                if (elect_one_lane()) umma_commit(&tmem_full[a]);
                __syncwarp();
            }
        }
    } else if (warp < 2 + GM_EPI_WARPS) {
        // ================= epilogue =================
        const int lq = warp & 3;                       // TMEM lane quarter this warp may access
        uint32_t tcount = 0;
        for (int tile = tile_first; tile < total_tiles && !*s_abort; tile += tile_step, ++tcount) {
            const int mt = tile % m_tiles, nt = tile / m_tiles;
            const uint32_t a = tcount & 1;
            if (!wait_or_abort(&tmem_full[a], (tcount >> 1) & 1, s_abort)) break;
            tc_fence_after();
            const int m = mt * GM_BM + lq * 32 + lane;
            const float sxm = (m < p.M) ? p.sx[m] : 0.0f;
            const int xs = (m < p.M) ? p.xsum[m] : 0;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lq * 32) << 16) + a * BN;
            if (SPLIT) {
                // rows of this lane quarter that exist: send each 32-column chunk to the CTA that finishes it
                const int cols_own = BN / csize;
                const int row = lq * 32 + lane;
                if (lq * 32 < p.a_rows) {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32) {
                        int v[32];
                        if (k_blocks > 0) {
                            tmem_ld_32x32b_x32(taddr + c0, v);
                            tmem_ld_wait();
                        } else {
#pragma unroll
                            for (int c = 0; c < 32; ++c) v[c] = 0;
                        }
                        if (row < p.a_rows) {
                            const uint32_t dst = map_to_cta(&s_stage[(crank * p.a_rows + row) * cols_own + (c0 % cols_own)], static_cast<uint32_t>(c0 / cols_own));
#pragma unroll
                            for (int c = 0; c < 32; c += 4) st_cluster_v4(dst + c * 4, v[c], v[c + 1], v[c + 2], v[c + 3]);
                        }
                    }
                }
                tc_fence_before();
            }
#pragma unroll 1
            for (int c0 = 0; !SPLIT && c0 < BN; c0 += 32) {
                int v[32];
                tmem_ld_32x32b_x32(taddr + c0, v);
                tmem_ld_wait();
                if (c0 + 32 == BN) {
                    // accumulator fully read: hand the TMEM buffer back before the stores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[a]);
                }
                const int n0 = nt * BN + c0;
                if (m < p.M && n0 < p.N) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] -= xs;      // weights were multiplied as t+1
                    if (p.acc_out != nullptr) {
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (n0 + c < p.N) p.acc_out[static_cast<int64_t>(m) * p.N + n0 + c] = v[c];
                    }
                    float y[32];
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int n = min(n0 + c, p.N - 1);
                        y[c] = dequant(v[c], sxm, __ldg(p.scale + n), p.bias ? __ldg(p.bias + n) : 0.0f, p.bias != nullptr);
                    }
                    store_row32(p.Y, p.y_dtype, static_cast<int64_t>(m) * p.ldy + n0, y, min(32, p.N - n0));
                }
            }
        }
    } else {
        // ================= unpack: 2-bit tiles -> u8 codes, K-major, 128-byte swizzle =================
        const int utid = threadIdx.x - (2 + GM_EPI_WARPS) * 32;   // 0..255
        const int uwarp = utid >> 5;
        const int g = lane >> 2, t = lane & 3;
        // Group `grp` unpacks the K blocks whose running index is congruent to grp: the latency
        // chain of one block (barrier, loads, stores, proxy fence, arrive) overlaps the next block's.
        const int grp = uwarp / GM_GROUP_WARPS, gwarp = uwarp % GM_GROUP_WARPS;
        RingPos ld, bb;
        ld.advance_by(NL, grp);
        bb.advance_by(NB, grp);
        uint32_t kcount = grp;                               // running K-block index of this group's next block
        uint32_t kseen = 0;                                  // running index of the current tile's first block
        for (int tile = tile_first; tile < total_tiles && !*s_abort; tile += tile_step, kseen += k_blocks) {
            bool ok = true;
            for (; kcount < kseen + k_blocks; kcount += GM_UNPACK_GROUPS) {
                // the packed tiles have landed and the MMAs that read this B slot have finished
                if (!wait_or_abort(&full_load[ld.s], ld.phase, s_abort) || !wait_or_abort(&empty_b[bb.s], bb.phase ^ 1, s_abort)) { ok = false; break; }
                const uint8_t* pk = s_p + ld.s * P_BYTES;
                uint8_t* bt = s_b + bb.s * B_BYTES;
                // P_TILES packed tiles (16-column blocks) per stage, spread over the group's warps.  Lane (g,t)
                // holds, for column g + 8h, the 32 consecutive k = 32t .. 32t+31: two 16-byte chunks per column.
#pragma unroll
                for (int tix = gwarp; tix < P_TILES; tix += GM_GROUP_WARPS) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(pk + tix * TILE_BYTES + lane * 16);
                    const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};     // word q = h | (h2 << 1)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = TILE_N * tix + g + 8 * h;
                        uint8_t* rowp = bt + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
                        for (int c = 0; c < 2; ++c) {                   // chunk 2t + c holds planes 2c, 2c+1
                            uint4 v;
                            v.x = (w[h] >> (4 * c)) & 0x03030303u;            // plane 2c,   k half 0
                            v.y = (w[h + 2] >> (4 * c)) & 0x03030303u;        // plane 2c,   k half 1
                            v.z = (w[h] >> (4 * c + 2)) & 0x03030303u;        // plane 2c+1, k half 0
                            v.w = (w[h + 2] >> (4 * c + 2)) & 0x03030303u;    // plane 2c+1, k half 1
                            *reinterpret_cast<uint4*>(rowp + (((2 * t + c) ^ (row & 7)) << 4)) = v;
                        }
                    }
                }
                fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor core (async proxy)
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_b[bb.s]);
                ld.advance_by(NL, GM_UNPACK_GROUPS);
                bb.advance_by(NB, GM_UNPACK_GROUPS);
            }
            if (!ok) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (SPLIT) {
        // A CTA that gave up on a wait sent nothing (or not everything): tell every CTA of the cluster, so that none
        // adds a slice that never arrived.  The flag travels with the same barrier as the partial accumulators.
        if (threadIdx.x == 0 && *s_abort)
            for (int r = 0; r < csize; ++r) st_cluster_s32(map_to_cta(&s_abort_storage, static_cast<uint32_t>(r)), 1);
        cluster_sync_all();   // the partial accumulators of this CTA's columns have arrived from every K slice
        const int cols_own = BN / csize;
        const int nt = tile_first;                       // one M tile: the tile index is the column tile
        for (int idx = threadIdx.x; idx < p.M * cols_own; idx += GM_THREADS) {
            const int c = idx % cols_own, m = idx / cols_own;
            const int n = nt * BN + crank * cols_own + c;
            if (n < p.N && !*s_abort) {
                int acc = -p.xsum[m];                    // weights were multiplied as t+1
                for (int r = 0; r < csize; ++r) acc += s_stage[(r * p.a_rows + m) * cols_own + c];
                if (p.acc_out != nullptr) p.acc_out[static_cast<int64_t>(m) * p.N + n] = acc;
                const float y = dequant(acc, p.sx[m], __ldg(p.scale + n), p.bias ? __ldg(p.bias + n) : 0.0f, p.bias != nullptr);
                store_out_dt(p.Y, p.y_dtype, static_cast<int64_t>(m) * p.ldy + n, y);
            }
        }
    }
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side ------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Tensor map over the tiled weights seen as [column blocks][KT * 128 words]: one box is the `block_rows`
// 512-byte tiles that one K block of an output tile needs.
static int encode_weight_map(EncodeTiledFn encode, const GemmParams& p, int block_rows, CUtensorMap* map) {
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(p.KT) * (TILE_BYTES / 4), static_cast<cuuint64_t>(p.NB)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(p.KT) * TILE_BYTES};
    const cuuint32_t box[2] = {TILE_BYTES / 4, static_cast<cuuint32_t>(block_rows)};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult cr = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(p.tiled), gdim, gstride, box, estride,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        set_error("bt_gemm_tiled_i8: cuTensorMapEncodeTiled (weights) failed with code %d", static_cast<int>(cr));
        return BT_ERR_CUDA;
    }
    return BT_OK;
}

// Depth of the load ring for an activation tile of a_rows rows: the configured depth for full tiles, otherwise
// the largest power of two (at most GM_MAX_NL, and no more than the K blocks there are) that fits shared memory.
template <int BN>
static int gemm_ring_depth_log2(int a_rows, int k_blocks, size_t extra_bytes = 0) {
    int lg = 0;
    while ((1 << lg) < GemmCfg<BN>::NL) ++lg;
    if (a_rows == GM_BM) return lg;
    while ((1 << (lg + 1)) <= GM_MAX_NL && (1 << lg) < k_blocks &&
           gm_smem_bytes<BN>(1 << (lg + 1), a_rows) + extra_bytes + 1024 <= GM_SMEM_LIMIT)
        ++lg;
    return lg;
}

// Clusters of `split` CTAs of the split-K kernel that can be resident at once (they need `split` free SMs inside one
// GPC each, so this is less than SMs / split); 0 on error.  Cached per cluster size for the largest footprint.
static int gemm_split_max_clusters(int split);

// split > 1: one tile per cluster of `split` CTAs, K divided among them (BN = 256, M <= 32)
template <int BN, bool SPLIT>
static int launch_gemm(EncodeTiledFn encode, const CUtensorMap& map, GemmParams p, cudaStream_t st, int split = 1) {
    CUtensorMap map_w;
    if (const int rc = encode_weight_map(encode, p, gm_p_tiles<BN>(), &map_w)) return rc;
    const int k_blocks = static_cast<int>(ceil_div<int64_t>(p.K, GM_BK));
    const size_t stage_bytes = SPLIT ? static_cast<size_t>(p.a_rows) * BN * 4 : 0;     // received partial accumulators
    p.nl_log2 = gemm_ring_depth_log2<BN>(p.a_rows, ceil_div(k_blocks, split), stage_bytes);
    const size_t smem = gm_smem_bytes<BN>(1 << p.nl_log2, p.a_rows) + stage_bytes;
    const int64_t tiles = ceil_div<int64_t>(p.M, GM_BM) * ceil_div<int64_t>(p.N, BN);
    const unsigned grid = SPLIT ? static_cast<unsigned>(tiles * split) : static_cast<unsigned>(std::min<int64_t>(tiles, sm_count()));
    auto kern = gemm_tcgen05_kernel<BN, SPLIT>;
    static std::atomic<size_t> granted[BT_MAX_DEVICES];
    if (const int rc = ensure_dynamic_smem(kern, smem, granted)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = static_cast<unsigned>(split);
    attrs[1].val.clusterDim.y = 1;
    attrs[1].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = SPLIT ? 2 : 1;
    BT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, map, map_w, p));
    return BT_OK;
}

static int gemm_split_max_clusters(int split) {
    static int cache[9] = {0};
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (split < 2 || split > 8) return 0;
    if (cache[split] == 0) {
        auto kern = gemm_tcgen05_kernel<256, true>;
        const size_t smem = GM_SMEM_LIMIT - 1024;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) return 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(split) * 64);
        cfg.blockDim = dim3(GM_THREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = static_cast<unsigned>(split);
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
        cache[split] = n > 0 ? n : -1;
    }
    return cache[split] > 0 ? cache[split] : 0;
}

static int launch_gemm_pair(EncodeTiledFn encode, const CUtensorMap& map, const GemmParams& p, cudaStream_t st);   // gemm_tcgen05_2cta.cuh

}  // namespace bt

extern "C" int bt_gemm_tiled_i8(const int8_t* Xq, const float* sx, const int32_t* xsum, int64_t M, int64_t K,
                                const uint8_t* tiled, int64_t N, const float* scale, const float* bias, void* Y,
                                int y_dtype, int64_t ldy, int32_t* acc_out, void* stream) {
    using namespace bt;
    BT_REQUIRE(Xq && sx && xsum && tiled && scale && Y, "bt_gemm_tiled_i8: NULL pointer");
    BT_REQUIRE(M > 0 && K > 0 && N > 0, "bt_gemm_tiled_i8: X is empty or weight is empty");
    BT_REQUIRE(valid_dtype(y_dtype), "bt_gemm_tiled_i8: unknown output dtype %d", y_dtype);
    BT_REQUIRE(ldy >= N, "bt_gemm_tiled_i8: output row stride %lld < N %lld", (long long)ldy, (long long)N);
    BT_REQUIRE(aligned(tiled, 16) && aligned(Xq, 16), "bt_gemm_tiled_i8: Xq and tiled weights must be 16-byte aligned");
    BT_UNSUPPORTED_IF(K % 16 != 0, "bt_gemm_tiled_i8: K=%lld must be a multiple of 16 (TMA row pitch)", (long long)K);
    BT_UNSUPPORTED_IF(K > BT_MAX_K || N > (int64_t{1} << 30) || M > (int64_t{1} << 30), "bt_gemm_tiled_i8: shape too large");

    EncodeTiledFn encode = get_encode_tiled();
    if (encode == nullptr) {
        set_error("bt_gemm_tiled_i8: cuTensorMapEncodeTiled is not available from the driver");
        return BT_ERR_CUDA;
    }
    // CTA pairs (cta_group::2, 256 x 256 tiles) once there are enough 256-row tiles to fill the GPU
    const int sms = sm_count();
    bool pair = M > GM_BM && ceil_div<int64_t>(M, 256) * ceil_div<int64_t>(N, 256) >= (sms / 2) * 55 / 100;
    if (const int v = tuning(BT_TUNE_GEMM_PAIR); v >= 0) pair = v != 0;      // testing / tuning override
    // rows of the activation tile that are copied: all 128, or M rounded up to the 8-row swizzle atom when M is small
    const int a_rows = (pair || M > GM_BM - 8) ? GM_BM : static_cast<int>(ceil_div<int64_t>(M, 8) * 8);
    CUtensorMap map;
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(K)};
    const cuuint32_t box[2] = {GM_BK, static_cast<cuuint32_t>(a_rows)};
    const cuuint32_t estride[2] = {1, 1};
    CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(Xq), gdim, gstride, box, estride,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        set_error("bt_gemm_tiled_i8: cuTensorMapEncodeTiled failed with code %d", static_cast<int>(cr));
        return BT_ERR_CUDA;
    }

    GemmParams p;
    p.tiled = tiled; p.sx = sx; p.xsum = xsum; p.scale = scale; p.bias = bias; p.Y = Y; p.acc_out = acc_out; p.ldy = ldy;
    p.M = static_cast<int>(M); p.K = static_cast<int>(K); p.N = static_cast<int>(N);
    p.KT = static_cast<int>(ceil_div<int64_t>(K, TILE_K));
    p.NB = static_cast<int>(ceil_div<int64_t>(N, TILE_N));
    p.y_dtype = y_dtype;
    p.a_rows = a_rows;
    p.nl_log2 = 0;

    // the widest output tile that still gives every SM a tile; narrow tiles for small problems
    const int64_t m_tiles = ceil_div<int64_t>(M, GM_BM);
    int bn = 64;
    if (m_tiles * ceil_div<int64_t>(N, 256) >= sms) bn = 256;
    else if (m_tiles * ceil_div<int64_t>(N, 128) >= sms) bn = 128;
    {      // testing / tuning override
        const int v = tuning(BT_TUNE_GEMM_BN);
        if (v == 64 || v == 128 || v == 256) bn = v;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (pair) return launch_gemm_pair(encode, map, p, st);
    // a narrow batch: full-width tiles, K split over a cluster so that the tiles still cover the SMs
    if (M <= 32) {
        const int64_t tiles = ceil_div<int64_t>(N, 256);
        const int k_blocks = static_cast<int>(ceil_div<int64_t>(K, GM_BK));
        int split = 8;      // the widest split whose clusters are all resident at once
        while (split > 1 && (tiles > gemm_split_max_clusters(split) || split > k_blocks)) split >>= 1;
        {   // testing / tuning override: 1 disables
            const int v = tuning(BT_TUNE_GEMM_SPLIT);
            if ((v == 1 || v == 2 || v == 4 || v == 8) && v <= std::max(1, k_blocks)) split = v;
        }
        if (split > 1) return launch_gemm<256, true>(encode, map, p, st, split);
    }
    if (bn == 256) return launch_gemm<256, false>(encode, map, p, st);
    if (bn == 128) return launch_gemm<128, false>(encode, map, p, st);
    return launch_gemm<64, false>(encode, map, p, st);
}
