// libbt_simt.so: the library's kernels compiled for the CPU (see simt_host.h).  TEST INFRASTRUCTURE ONLY.
//
// Includes the real kernel files, so every extern "C" entry point they define (bt_quantize_pack, bt_pack_codes[_rows],
// bt_unpack_codes[_rows], bt_act_quant_i8, bt_retile_packed, bt_untile_packed, bt_gemv_tiled, bt_gemv_tiled_i8,
// bt_gemv_tiled_chained, bt_gemv_tiled_float, bt_linear_unpacked, bt_linear_packed_float, bt_silu_mul_quant,
// bt_add_rmsnorm_quant) is exported with its
// usual signature and takes HOST pointers.  Not built here: the tensor-core GEMMs (tcgen05, TMEM) and the
// cluster kernel of the public layout (distributed shared memory).
#include "simt_host.h"

#include <cstdarg>

#include "../../bittorch_b200/csrc/common.cuh"

namespace bt {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

static int g_sm_count = 6;                                    // few "SMs": several column blocks per CTA in small cases
int sm_count() { return g_sm_count; }
int tuning(int) { return -1; }

}  // namespace bt

#include "../../bittorch_b200/csrc/act_quant.cuh"
#include "../../bittorch_b200/csrc/float_planes.cuh"
#include "../../bittorch_b200/csrc/fused_elementwise.cuh"
#include "../../bittorch_b200/csrc/gemv_tiled.cuh"
#include "../../bittorch_b200/csrc/linear_float.cuh"
#include "../../bittorch_b200/csrc/quantize_pack.cuh"
#include "../../bittorch_b200/csrc/retile.cuh"

extern "C" int bt_version(void) { return 100; }
extern "C" const char* bt_last_error(void) { return bt::g_error; }
extern "C" int bt_device_status(int* status_host, void*) {
    *status_host = bt::g_device_status;
    bt::g_device_status = 0;
    return BT_OK;
}
extern "C" void simt_set_sm_count(int n) { bt::g_sm_count = n > 0 ? n : 1; }
// Rule violations of the emulated hardware since the last call (misaligned bulk copy, shared-memory overrun, ...).
extern "C" int simt_take_errors(char* text, size_t size) {
    std::lock_guard<std::mutex> lock(simt::error_mutex());
    const int n = simt::error_count().exchange(0);
    if (text != nullptr && size > 0) snprintf(text, size, "%s", simt::error_text());
    simt::error_text()[0] = 0;
    return n;
}
