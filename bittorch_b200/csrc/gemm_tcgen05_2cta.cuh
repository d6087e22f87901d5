// Prefill-size packed ternary linear, CTA-pair version: tcgen05.mma.cta_group::2.
//
// Two CTAs of a (2,1,1) cluster share one 256 x 256 output tile.  Each CTA loads its own
// 128 activation rows (TMA, 128-byte swizzle), unpacks its own HALF of the weight tile
// (128 columns) into shared memory, and owns the 128 x 256 slice of the accumulator that
// lives in its tensor memory; one elected lane of the even ("leader") CTA issues the MMAs for
// the pair.  Compared with the one-CTA kernel, every CTA unpacks and stores half as many weight
// bytes per MMA, and the pair fetches every activation tile once for 256 columns.
//
// Synchronisation (all mbarriers; waits are bounded):
//   full_a[NL]    leader only   <- TMA bytes of BOTH CTAs' activation tiles
//   full_p[NL]    per CTA       <- TMA bytes of the CTA's 2-bit tiles
//   empty_load[NL] per CTA      <- tcgen05.commit, multicast to both CTAs
//   full_b[NB]    leader only   <- unpack warps of both CTAs (the peer arrives remotely)
//   empty_b[NB]   per CTA       <- tcgen05.commit, multicast
//   tmem_full[2]  per CTA       <- tcgen05.commit, multicast
//   tmem_empty[2] leader only   <- epilogue warps of both CTAs
#pragma once

#include "gemm_tcgen05.cuh"

namespace bt {

constexpr int G2_BN = 256;                      // columns of the pair's tile
constexpr int G2_HALF = G2_BN / 2;              // columns unpacked by each CTA
constexpr int G2_NL = 8, G2_NB = 4;       // powers of two (see the MMA issuer)
constexpr int G2_P_TILES = G2_HALF / TILE_N;    // 8 packed tiles per CTA and K block
constexpr int G2_P_BYTES = G2_P_TILES * TILE_BYTES;      // 4 KB
constexpr int G2_B_BYTES = G2_HALF * GM_BK;              // 16 KB
constexpr size_t G2_SMEM_BYTES = 1024 + static_cast<size_t>(G2_NL) * (GM_A_BYTES + G2_P_BYTES) +
                                 static_cast<size_t>(G2_NB) * G2_B_BYTES + 512;
// D = s32, A = s8, B = u8, K-major, M = 256 (the pair), N = 256
constexpr uint32_t G2_IDESC = (2u << 4) | (1u << 7) | (0u << 10) | (static_cast<uint32_t>(G2_BN >> 3) << 17) |
                              (static_cast<uint32_t>(256 >> 4) << 24);
constexpr uint32_t G2_PEER_BIT_MASK = 0xFEFFFFFFu;   // clears the CTA-in-pair bit of a shared-window address

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
    // executed by both CTAs; the transaction bytes are counted on the leader's barrier
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
        : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs once every MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(static_cast<uint16_t>(3)) : "memory");
}
// Arrive on a barrier of another CTA of the cluster.  The default (CTA-scope release) form: a cluster-scope
// release costs about 1400 cycles per arrive here, and the data it would order is either read through the
// async proxy (after fence.proxy.async) or through tensor memory (after tcgen05.fence), not by generic loads.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
    constexpr int NL = G2_NL, NB = G2_NB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_a = smem;                                 // [NL] this CTA's 128 activation rows
    uint8_t* s_b = s_a + NL * GM_A_BYTES;                // [NB] this CTA's 128 unpacked weight columns
    uint8_t* s_p = s_b + NB * G2_B_BYTES;                // [NL] this CTA's packed tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + NL * G2_P_BYTES);
    uint64_t* full_a = bars;
    uint64_t* full_p = full_a + NL;
    uint64_t* empty_load = full_p + NL;
    uint64_t* full_b = empty_load + NL;
    uint64_t* empty_b = full_b + NB;
    uint64_t* tmem_full = empty_b + NB;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    __shared__ int s_abort_storage;
    volatile int* s_abort = &s_abort_storage;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();             // 0 = leader, 1 = peer
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int m_tiles = (p.M + 255) / 256;
    const int n_tiles = (p.N + G2_BN - 1) / G2_BN;
    const int total_tiles = m_tiles * n_tiles;
    const int k_blocks = (p.K + GM_BK - 1) / GM_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NL; ++s) {
            mbar_init(&full_a[s], 1);
            mbar_init(&full_p[s], 1);
            mbar_init(&empty_load[s], 1);
        }
        for (int s = 0; s < NB; ++s) {
            mbar_init(&full_b[s], 2 * GM_GROUP_WARPS);   // the group's warps of both CTAs
            mbar_init(&empty_b[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], 2 * GM_EPI_WARPS);
        }
        s_abort_storage = 0;
        mbar_fence_init();
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    // both CTAs' barriers exist before anyone signals across the pair
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ================= producer (both CTAs) =================
        if (lane == 0) {
            RingPos ld;
            for (int tile = pair; tile < total_tiles && !*s_abort; tile += n_pairs) {
                const int mt = tile % m_tiles, nt = tile / m_tiles;
                const int nb0 = nt * (G2_BN / TILE_N) + static_cast<int>(rank) * G2_P_TILES;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!wait_or_abort(&empty_load[ld.s], ld.phase ^ 1, s_abort)) { ok = false; break; }
                    if (leader) mbar_expect_tx(&full_a[ld.s], 2 * GM_A_BYTES);
                    tma_load_2d_pair(s_a + ld.s * GM_A_BYTES, &map_x, kb * GM_BK, mt * 256 + static_cast<int>(rank) * GM_BM,
                                     smem_u32(&full_a[ld.s]) & G2_PEER_BIT_MASK);
                    mbar_expect_tx(&full_p[ld.s], G2_P_BYTES);      // column blocks past the end arrive as zeros
                    tma_load_2d(s_p + ld.s * G2_P_BYTES, &map_w, kb * (TILE_BYTES / 4), nb0, &full_p[ld.s]);
                    ld.advance(NL);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer (leader CTA only) =================
        // warp-uniform loop, one elected lane issues (see the one-CTA kernel)
        if (leader) {
            static_assert((NL & (NL - 1)) == 0 && (NB & (NB - 1)) == 0, "ring depths must be powers of two");
            const uint64_t desc_a0 = umma_desc_sw128(smem_u32(s_a)), desc_b0 = umma_desc_sw128(smem_u32(s_b));
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);   // the same value, provably warp-uniform
            uint32_t cnt = 0, tcount = 0;      // K blocks / tiles issued so far
            bool ready = false;
            for (int tile = pair; tile < total_tiles; tile += n_pairs, ++tcount) {
                if (__any_sync(0xffffffffu, *s_abort != 0)) break;
                const uint32_t a = tcount & 1;
                if (!wait_or_abort_warp(&tmem_empty[a], ((tcount >> 1) & 1) ^ 1, s_abort)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_u + a * G2_BN;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    const uint32_t sl = cnt & (NL - 1), sb = cnt & (NB - 1), nx = cnt + 1, nsl = nx & (NL - 1), nsb = nx & (NB - 1);
                    if (!ready && (!wait_or_abort_warp(&full_a[sl], (cnt / NL) & 1, s_abort) || !wait_or_abort_warp(&full_b[sb], (cnt / NB) & 1, s_abort))) { ok = false; break; }
                    tc_fence_after();
                    uint32_t polled = 0;
                    if (elect_one_lane())
                        polled = umma_i8_burst4<true>(d_tmem, desc_a0 + sl * (GM_A_BYTES >> 4), desc_b0 + sb * (G2_B_BYTES >> 4), G2_IDESC,
                                                      kb > 0 ? 1u : 0u, &full_a[nsl], (nx / NL) & 1, &full_b[nsb], (nx / NB) & 1,
                                                      &empty_load[sl], &empty_b[sb]);
                    ready = __any_sync(0xffffffffu, polled != 0);
                    cnt = nx;
                }
                if (!ok) break;
                if (elect_one_lane()) umma_commit_pair(&tmem_full[a]);
                __syncwarp();
            }
        }
    } else if (warp < 2 + GM_EPI_WARPS) {
        // ================= epilogue (both CTAs, own 128 rows) =================
        const int lq = warp & 3;
        uint32_t tcount = 0;
        for (int tile = pair; tile < total_tiles && !*s_abort; tile += n_pairs, ++tcount) {
            const int mt = tile % m_tiles, nt = tile / m_tiles;
            const uint32_t a = tcount & 1;
            if (!wait_or_abort(&tmem_full[a], (tcount >> 1) & 1, s_abort)) break;
            tc_fence_after();
            const int m = mt * 256 + static_cast<int>(rank) * GM_BM + lq * 32 + lane;
            const float sxm = (m < p.M) ? p.sx[m] : 0.0f;
            const int xs = (m < p.M) ? p.xsum[m] : 0;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lq * 32) << 16) + a * G2_BN;
#pragma unroll 1
            for (int c0 = 0; c0 < G2_BN; c0 += 32) {
                int v[32];
                {
                tmem_ld_32x32b_x32(taddr + c0, v);
                tmem_ld_wait();
                }
                if (c0 + 32 == G2_BN) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(map_to_cta(&tmem_empty[a], 0));
                }
                const int n0 = nt * G2_BN + c0;
                if (m < p.M && n0 < p.N) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] -= xs;
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
        // ================= unpack (both CTAs, own 128 columns) =================
        const int utid = threadIdx.x - (2 + GM_EPI_WARPS) * 32;
        const int uwarp = utid >> 5;
        const int g = lane >> 2, t = lane & 3;
        const int grp = uwarp / GM_GROUP_WARPS, gwarp = uwarp % GM_GROUP_WARPS;
        RingPos ld, bb;
        ld.advance_by(NL, grp);
        bb.advance_by(NB, grp);
        uint32_t kcount = grp, kseen = 0;
        for (int tile = pair; tile < total_tiles && !*s_abort; tile += n_pairs, kseen += k_blocks) {
            bool ok = true;
            for (; kcount < kseen + k_blocks; kcount += GM_UNPACK_GROUPS) {
                if (!wait_or_abort(&full_p[ld.s], ld.phase, s_abort) || !wait_or_abort(&empty_b[bb.s], bb.phase ^ 1, s_abort)) { ok = false; break; }
                const uint8_t* pk = s_p + ld.s * G2_P_BYTES;
                uint8_t* bt = s_b + bb.s * G2_B_BYTES;
#pragma unroll
                for (int tix = gwarp; tix < G2_P_TILES; tix += GM_GROUP_WARPS) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(pk + tix * TILE_BYTES + lane * 16);
                    const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int row = TILE_N * tix + g + 8 * h;
                        uint8_t* rowp = bt + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            uint4 v;
                            v.x = (w[h] >> (4 * c)) & 0x03030303u;
                            v.y = (w[h + 2] >> (4 * c)) & 0x03030303u;
                            v.z = (w[h] >> (4 * c + 2)) & 0x03030303u;
                            v.w = (w[h + 2] >> (4 * c + 2)) & 0x03030303u;
                            *reinterpret_cast<uint4*>(rowp + (((2 * t + c) ^ (row & 7)) << 4)) = v;
                        }
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(map_to_cta(&full_b[bb.s], 0));
                ld.advance_by(NL, GM_UNPACK_GROUPS);
                bb.advance_by(NB, GM_UNPACK_GROUPS);
            }
            if (!ok) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    // neither CTA may leave (or free tensor memory) while the other can still signal it or read its operands
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

static int launch_gemm_pair(EncodeTiledFn encode, const CUtensorMap& map, const GemmParams& p, cudaStream_t st) {
    CUtensorMap map_w;
    if (const int rc = encode_weight_map(encode, p, G2_P_TILES, &map_w)) return rc;
    const int64_t tiles = ceil_div<int64_t>(p.M, 256) * ceil_div<int64_t>(p.N, G2_BN);
    const unsigned pairs = static_cast<unsigned>(std::min<int64_t>(tiles, sm_count() / 2));
    auto kern = gemm_tcgen05_pair_kernel;
    static std::atomic<size_t> granted[BT_MAX_DEVICES];
    if (const int rc = ensure_dynamic_smem(kern, G2_SMEM_BYTES, granted)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(GM_THREADS);
    cfg.dynamicSmemBytes = G2_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 2;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    BT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, map, map_w, p));
    return BT_OK;
}

}  // namespace bt
