// Runs the library's CUDA kernels on the CPU, one OS thread per CUDA thread.  TEST INFRASTRUCTURE ONLY.
//
// The kernel sources (bittorch_b200/csrc/*.cuh) are compiled as plain C++ by g++ with BT_SIMT_HOST defined: this
// header supplies what the device would - threadIdx / blockIdx, __syncthreads, named barriers, warp shuffles,
// mbarriers with transaction counts, the 1-D bulk copy, atomics and the arithmetic intrinsics - so that the SAME
// kernel code executes with real concurrency between the threads of a CTA (CTAs run one after the other).  What this
// checks: index arithmetic, barrier and mbarrier protocols (phases, arrival counts, byte counts), data flow and the
// integer / float arithmetic of the kernels, bit for bit against the oracle, plus the alignment rules of the bulk
// copy and overruns of dynamic shared memory.  What it cannot check: anything about timing, memory ordering weaker
// than sequential consistency, programmatic dependent launch, or the tensor-core kernels (not built here).
#pragma once
#define BT_SIMT_HOST 1

#include <pthread.h>
#include <sched.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include <cuda_runtime.h>   // vector types, dim3, launch-config structs (types only: nothing of the runtime is called)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#undef __shared__
#define __shared__ static   // one copy for all threads; CTAs run one after the other
#ifndef __launch_bounds__
#define __launch_bounds__(...)
#endif

using std::max;
using std::min;

namespace simt {

struct Mbar {
    int init_count = 0, pending = 0;
    long long tx = 0;
    unsigned phase = 0;
};

struct Warp {
    pthread_barrier_t bar;
    uint32_t xchg[32];
};

struct Block {
    dim3 grid, block, index;
    int nthreads = 0;
    pthread_barrier_t cta_bar;
    std::vector<std::unique_ptr<Warp>> warps;
    std::mutex mu;                                            // guards named barriers, mbarriers, atomics
    std::map<std::pair<int, int>, std::unique_ptr<pthread_barrier_t>> named;
    std::map<const void*, Mbar> mbars;
    uint8_t* dyn_smem = nullptr;
};

struct Thread {
    Block* blk = nullptr;
    uint3 tid = {0, 0, 0};
    int linear = 0;
};

inline Thread& tl() {
    static thread_local Thread t;
    return t;
}

inline std::atomic<int>& error_count() {
    static std::atomic<int> n{0};
    return n;
}
inline std::mutex& error_mutex() {
    static std::mutex m;
    return m;
}
inline char* error_text() {
    static char text[512] = "";
    return text;
}
inline void fail(const char* what) {
    std::lock_guard<std::mutex> lock(error_mutex());
    if (error_count().fetch_add(1) == 0) snprintf(error_text(), 512, "%s", what);
}

constexpr size_t GUARD = 256;
constexpr uint8_t POISON = 0xCD;

// Runs kern(args...) for every thread of every block of the grid.  Returns 0, or 2 (BT_ERR_CUDA) if a rule of the
// emulated hardware was broken (misaligned bulk copy, write past the dynamic shared memory, ...).
template <typename Kern, typename... Args>
int launch(Kern kern, dim3 grid, dim3 block, size_t smem_bytes, Args... args) {
    const int nthreads = static_cast<int>(block.x * block.y * block.z);
    if (nthreads <= 0 || nthreads > 1024 || nthreads % 32 != 0 || smem_bytes > 227 * 1024) {
        fail("launch: bad block size or shared-memory size");
        return 2;
    }
    const int before = error_count().load();
    std::vector<uint8_t> smem(smem_bytes + 2 * GUARD + 1024);
    for (unsigned bz = 0; bz < grid.z; ++bz)
        for (unsigned by = 0; by < grid.y; ++by)
            for (unsigned bx = 0; bx < grid.x; ++bx) {
                Block blk;
                blk.grid = grid;
                blk.block = block;
                blk.index = dim3(bx, by, bz);
                blk.nthreads = nthreads;
                pthread_barrier_init(&blk.cta_bar, nullptr, nthreads);
                for (int w = 0; w < nthreads / 32; ++w) {
                    blk.warps.emplace_back(new Warp);
                    pthread_barrier_init(&blk.warps.back()->bar, nullptr, 32);
                }
                std::fill(smem.begin(), smem.end(), POISON);   // shared memory starts as garbage
                uint8_t* base = smem.data() + GUARD;
                base += (1024 - reinterpret_cast<uintptr_t>(base) % 1024) % 1024;
                blk.dyn_smem = base;
                std::vector<std::thread> threads;
                threads.reserve(nthreads);
                for (int t = 0; t < nthreads; ++t)
                    threads.emplace_back([&, t] {
                        Thread& me = tl();
                        me.blk = &blk;
                        me.linear = t;
                        me.tid.x = t % block.x;
                        me.tid.y = (t / block.x) % block.y;
                        me.tid.z = t / (block.x * block.y);
                        kern(args...);
                        me.blk = nullptr;
                    });
                for (auto& th : threads) th.join();
                for (size_t i = 0; i < GUARD; ++i)
                    if (base[smem_bytes + i] != POISON || *(base - 1 - i) != POISON) {
                        fail("a kernel wrote outside its dynamic shared memory");
                        break;
                    }
                pthread_barrier_destroy(&blk.cta_bar);
                for (auto& w : blk.warps) pthread_barrier_destroy(&w->bar);
                for (auto& nb : blk.named) pthread_barrier_destroy(nb.second.get());
            }
    return error_count().load() == before ? 0 : 2;
}

inline Warp& my_warp() { return *tl().blk->warps[tl().linear / 32]; }
inline int my_lane() { return tl().linear % 32; }

template <typename T>
inline T shfl(T v, int src_lane) {
    static_assert(sizeof(T) == 4, "32-bit shuffles only");
    Warp& w = my_warp();
    uint32_t bits;
    memcpy(&bits, &v, 4);
    w.xchg[my_lane()] = bits;
    pthread_barrier_wait(&w.bar);
    bits = w.xchg[src_lane & 31];
    pthread_barrier_wait(&w.bar);
    T r;
    memcpy(&r, &bits, 4);
    return r;
}

}  // namespace simt

// ---- built-in variables -------------------------------------------------------------------------
#define threadIdx (::simt::tl().tid)
#define blockIdx (::simt::tl().blk->index)
#define blockDim (::simt::tl().blk->block)
#define gridDim (::simt::tl().blk->grid)

// ---- synchronisation and warp primitives --------------------------------------------------------
inline void __syncthreads() { pthread_barrier_wait(&::simt::tl().blk->cta_bar); }
inline void __syncwarp(unsigned = 0xffffffffu) { pthread_barrier_wait(&::simt::my_warp().bar); }
inline int __shfl_xor_sync(unsigned, int v, int lane_mask) { return ::simt::shfl(v, ::simt::my_lane() ^ lane_mask); }
inline unsigned __shfl_xor_sync(unsigned, unsigned v, int lane_mask) { return ::simt::shfl(v, ::simt::my_lane() ^ lane_mask); }
inline float __shfl_xor_sync(unsigned, float v, int lane_mask) { return ::simt::shfl(v, ::simt::my_lane() ^ lane_mask); }

// ---- atomics (sequentially consistent) ------------------------------------------------------------
inline int atomicExch(int* p, int v) {
    std::lock_guard<std::mutex> lock(::simt::tl().blk->mu);
    const int old = *p;
    *p = v;
    return old;
}
inline unsigned atomicMax(unsigned* p, unsigned v) {
    static std::mutex global_mu;                              // global memory: shared by all blocks (sequential anyway)
    std::lock_guard<std::mutex> lock(global_mu);
    const unsigned old = *p;
    if (v > old) *p = v;
    return old;
}

// ---- arithmetic intrinsics ----------------------------------------------------------------------------
inline int __dp4a(int a, int b, int c) {
    for (int i = 0; i < 4; ++i) c += static_cast<int>(static_cast<int8_t>(a >> (8 * i))) * static_cast<int>(static_cast<int8_t>(b >> (8 * i)));
    return c;
}
inline uint4 __ldcg(const uint4* p) { return *p; }
inline float __ldg(const float* p) { return *p; }
inline unsigned __float_as_uint(float f) { unsigned u; memcpy(&u, &f, 4); return u; }
inline float __uint_as_float(unsigned u) { float f; memcpy(&f, &u, 4); return f; }
inline float __int_as_float(int i) { float f; memcpy(&f, &i, 4); return f; }
inline float __fdiv_rn(float a, float b) { return a / b; }
inline float __fmul_rn(float a, float b) { return a * b; }            // build with -ffp-contract=off
inline float __fadd_rn(float a, float b) { return a + b; }
inline long long __double_as_longlong(double d) { long long v; memcpy(&v, &d, 8); return v; }
inline double __longlong_as_double(long long v) { double d; memcpy(&d, &v, 8); return d; }
inline float __int2float_rn(int v) { return static_cast<float>(v); }
inline float __ll2float_rn(long long v) { return static_cast<float>(v); }
inline int __float2int_rn(float v) {                                     // round to nearest even, saturating; NaN -> 0
    if (v != v) return 0;
    if (v >= 2147483648.0f) return 2147483647;
    if (v <= -2147483648.0f) return -2147483647 - 1;
    return static_cast<int>(std::nearbyintf(v));
}

// ---- what common.cuh leaves to the device build ----------------------------------------------------------
#define BT_LAUNCH(kernel, grid, block, smem, stream, ...) \
    ((void)(stream), ::simt::launch(kernel, dim3(grid), dim3(block), (smem), __VA_ARGS__))
#define BT_DYNAMIC_SMEM(name, alignment) uint8_t* name = ::simt::tl().blk->dyn_smem

namespace bt {

constexpr unsigned long long WAIT_BUDGET_NS = 60000000000ull;   // emulated threads are slow: a minute

inline unsigned long long global_timer_ns() {
    return static_cast<unsigned long long>(std::chrono::duration_cast<std::chrono::nanoseconds>(
                                               std::chrono::steady_clock::now().time_since_epoch()).count());
}

inline ::simt::Mbar& mbar_of(const void* bar) { return ::simt::tl().blk->mbars[bar]; }

inline void mbar_complete_if_done(::simt::Mbar& m) {
    if (m.pending == 0 && m.tx == 0) {
        m.phase ^= 1u;
        m.pending = m.init_count;
    }
}
inline void mbar_init(uint64_t* bar, uint32_t count) {
    std::lock_guard<std::mutex> lock(::simt::tl().blk->mu);
    ::simt::Mbar& m = mbar_of(bar);
    m.init_count = m.pending = static_cast<int>(count);
    m.tx = 0;
    m.phase = 0;
}
inline void mbar_fence_init() {}
inline void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {              // arrive + expect
    std::lock_guard<std::mutex> lock(::simt::tl().blk->mu);
    ::simt::Mbar& m = mbar_of(bar);
    if (m.init_count == 0) ::simt::fail("mbarrier used before it was initialised");
    m.tx += bytes;
    if (--m.pending < 0) ::simt::fail("more arrivals on an mbarrier than its count");
    mbar_complete_if_done(m);
}
inline void mbar_arrive(uint64_t* bar) {
    std::lock_guard<std::mutex> lock(::simt::tl().blk->mu);
    ::simt::Mbar& m = mbar_of(bar);
    if (m.init_count == 0) ::simt::fail("mbarrier used before it was initialised");
    if (--m.pending < 0) ::simt::fail("more arrivals on an mbarrier than its count");
    mbar_complete_if_done(m);
}
inline bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    bool done;
    {
        std::lock_guard<std::mutex> lock(::simt::tl().blk->mu);
        done = (mbar_of(bar).phase & 1u) != (parity & 1u);
    }
    if (!done) usleep(20);
    return done;
}
inline bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > WAIT_BUDGET_NS) return false;
    }
    return false;
}
// 1-D bulk copy global -> shared with its hardware rules: both addresses 16-byte aligned, size a multiple of 16.
inline void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    if (reinterpret_cast<uintptr_t>(dst_smem) % 16 != 0 || reinterpret_cast<uintptr_t>(src_gmem) % 16 != 0 || bytes % 16 != 0 ||
        bytes == 0)
        ::simt::fail("bulk copy: addresses must be 16-byte aligned and the size a non-zero multiple of 16");
    memcpy(dst_smem, src_gmem, bytes);
    std::lock_guard<std::mutex> lock(::simt::tl().blk->mu);
    ::simt::Mbar& m = mbar_of(bar);
    m.tx -= bytes;
    if (m.tx < 0) ::simt::fail("bulk copy completed more bytes than the mbarrier expected");
    mbar_complete_if_done(m);
}
inline void pdl_launch_dependents() {}
inline void pdl_wait() {}

template <int ID>
inline void named_barrier_sync(int nthreads) {
    ::simt::Block& blk = *::simt::tl().blk;
    pthread_barrier_t* bar;
    {
        std::lock_guard<std::mutex> lock(blk.mu);
        auto& slot = blk.named[{ID, nthreads}];
        if (!slot) {
            slot.reset(new pthread_barrier_t);
            pthread_barrier_init(slot.get(), nullptr, nthreads);
        }
        bar = slot.get();
    }
    pthread_barrier_wait(bar);
}

}  // namespace bt
