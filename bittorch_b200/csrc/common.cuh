// Shared host/device helpers of the sm_100a ternary linear kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/bittorch_b200.h"

namespace bt {

constexpr int BT_MAX_DEVICES = 64;

// ---- host-side error plumbing --------------------------------------------------

void set_error(const char* fmt, ...);   // stores a thread-local message (lib.cu)

#define BT_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            ::bt::set_error(__VA_ARGS__);     \
            return BT_ERR_INVALID;            \
        }                                     \
    } while (0)

#define BT_UNSUPPORTED_IF(cond, ...)          \
    do {                                      \
        if (cond) {                           \
            ::bt::set_error(__VA_ARGS__);     \
            return BT_ERR_UNSUPPORTED;        \
        }                                     \
    } while (0)

#ifndef BT_SIMT_HOST
#define BT_CUDA_OK(expr)                                                              \
    do {                                                                              \
        cudaError_t e__ = (expr);                                                     \
        if (e__ != cudaSuccess) {                                                     \
            ::bt::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));         \
            return BT_ERR_CUDA;                                                       \
        }                                                                             \
    } while (0)

// Kernel launch with the triple-chevron syntax.  (A host build that runs the kernels as threads on the CPU, for tests,
// defines BT_SIMT_HOST and supplies its own BT_LAUNCH, BT_LAUNCH_OK and the primitives marked below.)
#define BT_LAUNCH(kernel, grid, block, smem, stream, ...) kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__)
// The CTA's dynamic shared memory as a byte array called `name`.
#define BT_DYNAMIC_SMEM(name, alignment) extern __shared__ __align__(alignment) uint8_t name[]

// Checks the launch that was just enqueued.
#define BT_LAUNCH_OK(name)                                                            \
    do {                                                                              \
        cudaError_t e__ = cudaGetLastError();                                         \
        if (e__ != cudaSuccess) {                                                     \
            ::bt::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__)); \
            return BT_ERR_CUDA;                                                       \
        }                                                                             \
    } while (0)
#else
#define BT_LAUNCH_OK(name)                                                            \
    do {                                                                              \
        if (::simt::error_count().load() != 0) {                                      \
            ::bt::set_error("%s: %s", name, ::simt::error_text());                    \
            return BT_ERR_CUDA;                                                       \
        }                                                                             \
    } while (0)
#endif

inline bool valid_dtype(int d) { return d == BT_F32 || d == BT_F16 || d == BT_BF16; }
inline size_t dtype_size(int d) { return d == BT_F32 ? 4 : 2; }
__host__ __device__ inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
template <typename T>
inline T ceil_div(T a, T b) { return (a + b - 1) / b; }

int sm_count();   // SMs of the current device, cached (lib.cu)

// Kernel-selection overrides for tests and tuning (lib.cu): -1 = automatic.  Set with bt_set_tuning(); the
// environment variable of the same meaning is read once, the first time a knob is looked at.
int tuning(int knob);

// Raises a kernel's dynamic shared-memory limit once per device and size instead of on every launch.
// `granted` is a zero-initialised per-kernel array (one slot per device ordinal).
template <typename Kern>
inline int ensure_dynamic_smem(Kern kern, size_t smem, std::atomic<size_t>* granted) {
    if (smem <= 48 * 1024) return BT_OK;
#ifdef BT_SIMT_HOST
    (void)kern; (void)granted;
    return BT_OK;
#else
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= BT_MAX_DEVICES) dev = -1;
    if (dev >= 0 && granted[dev].load(std::memory_order_acquire) >= smem) return BT_OK;
    BT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    if (dev >= 0) {
        size_t seen = granted[dev].load(std::memory_order_relaxed);
        while (seen < smem && !granted[dev].compare_exchange_weak(seen, smem, std::memory_order_release)) {}
    }
    return BT_OK;
#endif
}

// Sticky per-device status word written by kernels whose bounded waits ran out.
// The library is one translation unit (lib.cu includes every kernel file), so a
// plain definition here is the only copy.
__device__ int g_device_status = 0;
__device__ __forceinline__ void report_wait_timeout() { atomicExch(&g_device_status, BT_ERR_DEVICE_WAIT); }

// ---- device helpers --------------------------------------------------------------

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<double>(double v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ double from_float<double>(float v) { return static_cast<double>(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Rounds an fp32 value to the storage type T and widens it back.
template <typename T> __device__ __forceinline__ float round_through(float v) { return to_float<T>(from_float<T>(v)); }

// Loads 4 consecutive elements (vectorised when `vec` says the address is aligned).
template <typename T>
__device__ __forceinline__ void load4(const T* p, bool vec, int valid, float (&out)[4]);

template <>
__device__ __forceinline__ void load4<float>(const float* p, bool vec, int valid, float (&out)[4]) {
    if (vec && valid == 4) {
        float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = (i < valid) ? p[i] : 0.0f;
    }
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, bool vec, int valid, float (&out)[4]) {
    if (vec && valid == 4) {
        uint2 raw = *reinterpret_cast<const uint2*>(p);
        __half2 a = *reinterpret_cast<__half2*>(&raw.x), b = *reinterpret_cast<__half2*>(&raw.y);
        out[0] = __low2float(a); out[1] = __high2float(a); out[2] = __low2float(b); out[3] = __high2float(b);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = (i < valid) ? __half2float(p[i]) : 0.0f;
    }
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, bool vec, int valid, float (&out)[4]) {
    if (vec && valid == 4) {
        uint2 raw = *reinterpret_cast<const uint2*>(p);
        out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
        out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = (i < valid) ? __bfloat162float(p[i]) : 0.0f;
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_or(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v |= __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Shared epilogue of the integer kernels: (float(acc) * sx) * scale + bias, no FMA
// contraction, matching csrc/kernels/ternary_gemm_tensor_core.cu:652 with the
// factor 127 cancelled.
__device__ __forceinline__ float dequant(int acc, float sx, float scale, float bias, bool has_bias) {
    float r = __fmul_rn(__fmul_rn(__int2float_rn(acc), sx), scale);
    return has_bias ? __fadd_rn(r, bias) : r;
}

template <typename T>
__device__ __forceinline__ void store_out(void* Y, int64_t idx, float v) {
    reinterpret_cast<T*>(Y)[idx] = from_float<T>(v);
}
__device__ __forceinline__ void store_out_dt(void* Y, int dt, int64_t idx, float v) {
    if (dt == BT_F32) store_out<float>(Y, idx, v);
    else if (dt == BT_F16) store_out<__half>(Y, idx, v);
    else store_out<__nv_bfloat16>(Y, idx, v);
}

#ifndef BT_SIMT_HOST
// ---- PTX wrappers (sm_90+/sm_100a features) ---------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
constexpr unsigned long long WAIT_BUDGET_NS = 2000000000ull;   // a device-side wait gives up after 2 s

// Bounded wait: polls the barrier (each poll may itself suspend for a hardware-defined
// short time) and gives up after `limit` polls or WAIT_BUDGET_NS of wall time, whichever
// comes first.  Returns false on timeout; the caller records it.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_BUDGET_NS) return false;
        }
    }
    return false;
}

// 1-D bulk copy global -> shared (TMA engine), completion counted on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start early /
// wait for the previous kernel's memory to be visible.  No-ops when the launch
// did not request the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Thread-block cluster helpers.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ int ld_dsmem_s32(const void* local_smem_ptr, uint32_t cta_rank) {
    uint32_t remote;
    int v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_smem_ptr)), "r"(cta_rank));
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
}

// Named barrier ID over the `nthreads` threads that call it (whole warps).
template <int ID>
__device__ __forceinline__ void named_barrier_sync(int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "r"(nthreads) : "memory");
}
#endif   // BT_SIMT_HOST

}  // namespace bt
