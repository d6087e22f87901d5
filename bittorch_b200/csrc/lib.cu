// libbittorch_b200.so — single translation unit of the sm_100a ternary linear backend.
// Every kernel file is a header included here, so device globals have one definition
// and no relocatable device code is needed.
#include <algorithm>
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
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace bt

#include "act_quant.cuh"
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

#ifdef BT_TRACE
// Bring-up aid (only in -DBT_TRACE builds): copies the kernel timeline stamps to the host.
extern "C" int bt_trace_read(unsigned long long* out64) {
    using namespace bt;
    BT_CUDA_OK(cudaDeviceSynchronize());
    BT_CUDA_OK(cudaMemcpyFromSymbol(out64, g_trace, sizeof(unsigned long long) * 128));
    return BT_OK;
}
extern "C" int bt_trace_read_cta(unsigned long long* out64, unsigned int* sm) {
    using namespace bt;
    BT_CUDA_OK(cudaDeviceSynchronize());
    BT_CUDA_OK(cudaMemcpyFromSymbol(out64, g_trace_cta, sizeof(unsigned long long) * 4096 * 4));
    BT_CUDA_OK(cudaMemcpyFromSymbol(sm, g_trace_sm, sizeof(unsigned int) * 4096));
    return BT_OK;
}
#endif
