// libbittorch_b200.so — single translation unit of the sm_100a ternary linear backend.
// Every kernel file is a header included here, so device globals have one definition
// and no relocatable device code is needed.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace bt {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static std::atomic<int> cached[BT_MAX_DEVICES];            // zero-initialised; a race only repeats the query
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= BT_MAX_DEVICES) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// ---- kernel-selection overrides (tests, tuning) ------------------------------------------------
static std::atomic<int> g_tuning[BT_TUNE_COUNT];
static std::once_flag g_tuning_once;

static void tuning_init() {
    static const char* const env_names[BT_TUNE_COUNT] = {"BITTORCH_B200_GEMM_PAIR", "BITTORCH_B200_GEMM_BN",
                                                         "BITTORCH_B200_GEMM_SPLIT", "BITTORCH_B200_GEMV_SPLIT"};
    for (int k = 0; k < BT_TUNE_COUNT; ++k) {
        const char* e = std::getenv(env_names[k]);
        g_tuning[k].store(e != nullptr ? std::atoi(e) : -1, std::memory_order_relaxed);
    }
}

int tuning(int knob) {
    std::call_once(g_tuning_once, tuning_init);
    return (knob >= 0 && knob < BT_TUNE_COUNT) ? g_tuning[knob].load(std::memory_order_relaxed) : -1;
}

// A wait that nothing will ever satisfy, with a small poll limit: exercises the give-up path of the bounded
// waits (status word, normal return) without any kernel of the library having to fail.
__global__ void wait_timeout_selftest_kernel(int polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait_bounded(&bar, 0, static_cast<uint32_t>(polls))) report_wait_timeout();
    __syncthreads();
}

}  // namespace bt

#include "act_quant.cuh"
#include "float_planes.cuh"
#include "fused_elementwise.cuh"
#include "gemm_tcgen05.cuh"
#include "gemm_tcgen05_2cta.cuh"
#include "gemv.cuh"
#include "gemv_tiled.cuh"
#include "linear_float.cuh"
#include "quantize_pack.cuh"
#include "retile.cuh"

extern "C" int bt_version(void) { return 100; }   // 0.1.0

extern "C" const char* bt_last_error(void) { return bt::g_error; }

extern "C" int bt_device_status(int* status_host, void* stream) {
    using namespace bt;
    BT_REQUIRE(status_host != nullptr, "bt_device_status: NULL pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    BT_CUDA_OK(cudaStreamSynchronize(st));
    int v = 0;
    BT_CUDA_OK(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        BT_CUDA_OK(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    }
    *status_host = v;
    return BT_OK;
}

extern "C" int bt_dummy(const void* src, void* dst, size_t bytes, void* stream) {
    using namespace bt;
    if (bytes == 0) return BT_OK;
    BT_REQUIRE(src != nullptr && dst != nullptr, "bt_dummy: NULL pointer");
    BT_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return BT_OK;
}

extern "C" int bt_set_tuning(int knob, int value) {
    using namespace bt;
    BT_REQUIRE(knob >= 0 && knob < BT_TUNE_COUNT, "bt_set_tuning: unknown knob %d", knob);
    tuning(knob);                                              // the environment is read before the first override
    g_tuning[knob].store(value, std::memory_order_relaxed);
    return BT_OK;
}

extern "C" int bt_selftest_wait_timeout(void* stream) {
    using namespace bt;
    BT_LAUNCH(wait_timeout_selftest_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), 2048);
    BT_LAUNCH_OK("wait_timeout_selftest_kernel");
    return BT_OK;
}
