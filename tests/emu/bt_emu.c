/*
 * Host emulation of the C ABI declared in include/bittorch_b200.h.  TEST INFRASTRUCTURE ONLY.
 *
 * Every entry point has the signature of the CUDA library's, takes HOST pointers and
 * computes with the CPU oracle's arithmetic (oracle/bt_oracle.c, included below).  It
 * exists so that the host-side code that drives the library (the ctypes binding, the
 * modules, the decoder harness, bench.py) can be exercised end to end on a machine
 * without a GPU: tests/emu/runtime.py loads this file in place of the CUDA library in
 * a child process.  The shipped package never loads it.
 *
 * The private tiled layout is the real one (bittorch_b200/csrc/retile.cuh), written
 * here a second time from its definition, so that the emulated decode and GEMM entry
 * points read the same bytes as the kernels.
 */
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../oracle/bt_oracle.c"

#include "../../include/bittorch_b200.h"

static __thread char g_error[512] = "";

static int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

#define REQUIRE(cond, ...) do { if (!(cond)) return fail(BT_ERR_INVALID, __VA_ARGS__); } while (0)

/* ---- element types --------------------------------------------------------------- */

static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            float f = (float)man / 16777216.0f;               /* man * 2^-24 */
            memcpy(&u, &f, 4);
            u |= sign;
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 112u) << 23) | (man << 13);
    float r;
    memcpy(&r, &u, 4);
    return r;
}

static uint16_t float_to_half(float v) {
    float r = round_to_f16(v);                                 /* exactly representable now */
    uint32_t u;
    memcpy(&u, &r, 4);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    float a = fabsf(r);
    if (isnan(r)) return (uint16_t)(sign | 0x7e00u);
    if (isinf(a)) return (uint16_t)(sign | 0x7c00u);
    if (a == 0.0f) return sign;
    if (a < 6.103515625e-05f) return (uint16_t)(sign | (uint16_t)(a * 16777216.0f));
    int e;
    float m = frexpf(a, &e);                                   /* a = m 2^e, m in [0.5,1) */
    uint32_t man = (uint32_t)((m * 2.0f - 1.0f) * 1024.0f);
    return (uint16_t)(sign | ((uint32_t)(e - 1 + 15) << 10) | man);
}

static float load_elem(const void* p, int dtype, int64_t i) {
    if (dtype == BT_F32) return ((const float*)p)[i];
    if (dtype == BT_F64) return (float)((const double*)p)[i];
    if (dtype == BT_F16) return half_to_float(((const uint16_t*)p)[i]);
    uint32_t u = (uint32_t)((const uint16_t*)p)[i] << 16;
    float r;
    memcpy(&r, &u, 4);
    return r;
}

static void store_elem(void* p, int dtype, int64_t i, float v) {
    if (dtype == BT_F32) ((float*)p)[i] = v;
    else if (dtype == BT_F64) ((double*)p)[i] = (double)v;
    else if (dtype == BT_F16) ((uint16_t*)p)[i] = float_to_half(v);
    else {
        float r = round_to_bf16(v);
        uint32_t u;
        memcpy(&u, &r, 4);
        if (isnan(v)) u = 0x7fc00000u;
        ((uint16_t*)p)[i] = (uint16_t)(u >> 16);
    }
}

static int valid_dtype(int d) { return d == BT_F32 || d == BT_F16 || d == BT_BF16; }

static float* widen(const void* X, int dtype, int64_t M, int64_t K, int64_t ld) {
    float* out = (float*)malloc(sizeof(float) * (size_t)(M * K > 0 ? M * K : 1));
    for (int64_t m = 0; m < M; ++m)
        for (int64_t k = 0; k < K; ++k) out[m * K + k] = load_elem(X, dtype, m * ld + k);
    return out;
}

/* ---- tiled layout (bittorch_b200/csrc/retile.cuh) ---------------------------------- */

static void tile_slot(int n_local, int k_local, int* word, int* shift) {
    int g = n_local & 7, qlo = n_local >> 3;
    int t = k_local >> 5, r = k_local & 31;
    int i = r >> 3, qhi = (r >> 2) & 1, j = r & 3;
    *word = (4 * g + t) * 4 + (qlo | (qhi << 1));
    *shift = 8 * j + 2 * i;
}

static int8_t tiled_weight(const uint8_t* tiled, int64_t KT, int64_t n, int64_t k) {
    int word, shift;
    tile_slot((int)(n % 16), (int)(k % 128), &word, &shift);
    const uint32_t* words = (const uint32_t*)(tiled + ((n / 16) * KT + k / 128) * 512);
    return (int8_t)((int)((words[word] >> shift) & 3u) - 1);
}

static int8_t* codes_from_tiled(const uint8_t* tiled, int64_t K, int64_t N) {
    int64_t KT = (K + 127) / 128;
    int8_t* codes = (int8_t*)malloc((size_t)(N * K));
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) codes[n * K + k] = tiled_weight(tiled, KT, n, k);
    return codes;
}

/* ---- entry points -------------------------------------------------------------------- */

int bt_version(void) { return 100; }
const char* bt_last_error(void) { return g_error; }

static int g_status = 0;
static int g_tuning[BT_TUNE_COUNT] = {-1, -1, -1, -1};

int bt_device_status(int* status_host, void* stream) {
    (void)stream;
    REQUIRE(status_host != NULL, "bt_device_status: NULL pointer");
    *status_host = g_status;
    g_status = 0;
    return BT_OK;
}

int bt_set_tuning(int knob, int value) {
    REQUIRE(knob >= 0 && knob < BT_TUNE_COUNT, "bt_set_tuning: unknown knob %d", knob);
    g_tuning[knob] = value;                                    /* recorded; the emulation has one code path */
    return BT_OK;
}

int bt_selftest_wait_timeout(void* stream) {
    (void)stream;
    g_status = BT_ERR_DEVICE_WAIT;
    return BT_OK;
}

int bt_dummy(const void* src, void* dst, size_t bytes, void* stream) {
    (void)stream;
    if (bytes == 0) return BT_OK;
    REQUIRE(src && dst, "bt_dummy: NULL pointer");
    memcpy(dst, src, bytes);
    return BT_OK;
}

int bt_quantize_pack(const void* W, int w_dtype, int64_t N, int64_t K, int64_t ldw, float threshold_factor,
                     uint8_t* packed_T, float* scale, int8_t* codes, void* tern, void* stream) {
    (void)stream;
    REQUIRE(W && scale, "bt_quantize_pack: NULL pointer");
    REQUIRE(valid_dtype(w_dtype), "bt_quantize_pack: unknown dtype %d", w_dtype);
    REQUIRE(N > 0 && K > 0, "bt_quantize_pack: weight is empty");
    REQUIRE(ldw >= K, "bt_quantize_pack: row stride < K");
    float* w = widen(W, w_dtype, N, K, ldw);
    int8_t* c = codes ? codes : (int8_t*)malloc((size_t)(N * K));
    bto_ternarize(w, N, K, K, threshold_factor, w_dtype, c, scale);
    if (packed_T) bto_pack_transposed(c, N, K, packed_T);
    if (tern)
        for (int64_t i = 0; i < N * K; ++i) store_elem(tern, w_dtype, i, (float)c[i]);
    if (!codes) free(c);
    free(w);
    return BT_OK;
}

int bt_pack_codes(const int8_t* codes, int64_t N, int64_t K, uint8_t* packed_T, void* stream) {
    (void)stream;
    REQUIRE(codes && packed_T, "bt_pack_codes: NULL pointer");
    REQUIRE(N > 0 && K > 0, "bt_pack_codes: empty");
    bto_pack_transposed(codes, N, K, packed_T);
    return BT_OK;
}

int bt_pack_codes_rows(const int8_t* codes, int64_t N, int64_t K, uint8_t* packed, void* stream) {
    (void)stream;
    REQUIRE(codes && packed, "bt_pack_codes_rows: NULL pointer");
    REQUIRE(N > 0 && K > 0, "bt_pack_codes_rows: empty");
    bto_pack(codes, N, K, packed);
    return BT_OK;
}

int bt_unpack_codes(const uint8_t* packed_T, int64_t N, int64_t K, int8_t* codes, void* stream) {
    (void)stream;
    REQUIRE(codes && packed_T, "bt_unpack_codes: NULL pointer");
    REQUIRE(N > 0 && K > 0, "bt_unpack_codes: empty");
    bto_unpack_transposed(packed_T, N, K, codes);
    return BT_OK;
}

int bt_unpack_codes_rows(const uint8_t* packed, int64_t N, int64_t K, int8_t* codes, void* stream) {
    (void)stream;
    REQUIRE(codes && packed, "bt_unpack_codes_rows: NULL pointer");
    REQUIRE(N > 0 && K > 0, "bt_unpack_codes_rows: empty");
    bto_unpack(packed, N, K, codes);
    return BT_OK;
}

static void act_quant_rows(const float* x, int64_t M, int64_t K, int8_t* Xq, float* sx, int32_t* xsum) {
    bto_act_quant(x, M, K, K, Xq, sx);
    if (xsum)
        for (int64_t m = 0; m < M; ++m) {
            int32_t s = 0;
            for (int64_t k = 0; k < K; ++k) s += Xq[m * K + k];
            xsum[m] = s;
        }
}

int bt_act_quant_i8(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* Xq, float* sx,
                    int32_t* xsum, void* stream) {
    (void)stream;
    REQUIRE(X && Xq && sx, "bt_act_quant_i8: NULL pointer");
    REQUIRE(valid_dtype(x_dtype), "bt_act_quant_i8: unknown dtype %d", x_dtype);
    REQUIRE(M > 0 && K > 0, "bt_act_quant_i8: X is empty");
    REQUIRE(ldx >= K, "bt_act_quant_i8: row stride < K");
    float* x = widen(X, x_dtype, M, K, ldx);
    act_quant_rows(x, M, K, Xq, sx, xsum);
    free(x);
    return BT_OK;
}

size_t bt_tiled_bytes(int64_t K, int64_t N) {
    if (K <= 0 || N <= 0) return 0;
    return (size_t)((N + 15) / 16) * (size_t)((K + 127) / 128) * 512;
}

int bt_retile_packed(const uint8_t* packed_T, int64_t K, int64_t N, uint8_t* tiled, void* stream) {
    (void)stream;
    REQUIRE(packed_T && tiled, "bt_retile_packed: NULL pointer");
    REQUIRE(K > 0 && N > 0, "bt_retile_packed: empty weight");
    int64_t KT = (K + 127) / 128, NB = (N + 15) / 16;
    uint32_t* words = (uint32_t*)tiled;
    /* padding outside N x K is the code of a zero weight (1) */
    for (int64_t i = 0; i < NB * KT * 128; ++i) words[i] = 0x55555555u;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) {
            uint8_t c = (packed_T[(k / 4) * N + n] >> (2 * (k % 4))) & 3u;
            int t = (c == 1) - (c == 2);
            int word, shift;
            tile_slot((int)(n % 16), (int)(k % 128), &word, &shift);
            uint32_t* w = words + ((n / 16) * KT + k / 128) * 128 + word;
            *w = (*w & ~(3u << shift)) | ((uint32_t)(t + 1) << shift);
        }
    return BT_OK;
}

int bt_untile_packed(const uint8_t* tiled, int64_t K, int64_t N, uint8_t* packed_T, void* stream) {
    (void)stream;
    REQUIRE(packed_T && tiled, "bt_untile_packed: NULL pointer");
    REQUIRE(K > 0 && N > 0, "bt_untile_packed: empty weight");
    int8_t* codes = codes_from_tiled(tiled, K, N);
    bto_pack_transposed(codes, N, K, packed_T);
    free(codes);
    return BT_OK;
}

static int int_linear(const int8_t* Xq, const float* sx, int64_t M, int64_t K, const int8_t* codes, int64_t N,
                      const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy, int32_t* acc_out) {
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)(M * N));
    float* y = (float*)malloc(sizeof(float) * (size_t)(M * N));
    bto_gemm_i32(Xq, M, K, codes, N, acc);
    bto_epilogue(acc, M, N, sx, scale, bias, y);
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) store_elem(Y, y_dtype, m * ldy + n, y[m * N + n]);
    if (acc_out) memcpy(acc_out, acc, sizeof(int32_t) * (size_t)(M * N));
    free(acc);
    free(y);
    return BT_OK;
}

static int check_linear(const char* who, int64_t M, int64_t K, const void* w, int64_t N, const float* scale, void* Y,
                        int y_dtype, int64_t ldy) {
    REQUIRE(w && scale && Y, "%s: NULL pointer", who);
    REQUIRE(M > 0 && K > 0 && N > 0, "%s: X is empty or weight is empty", who);
    REQUIRE(valid_dtype(y_dtype), "%s: unknown output dtype %d", who, y_dtype);
    REQUIRE(ldy >= N, "%s: output row stride < N", who);
    return BT_OK;
}

int bt_gemv_packed_i8(const int8_t* Xq, const float* sx, int64_t M, int64_t K, const uint8_t* packed_T, int64_t N,
                      const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy, int32_t* acc_out,
                      void* stream) {
    (void)stream;
    REQUIRE(Xq && sx, "bt_gemv_packed_i8: NULL pointer");
    int rc = check_linear("bt_gemv_packed_i8", M, K, packed_T, N, scale, Y, y_dtype, ldy);
    if (rc) return rc;
    if (M > BT_GEMV_MAX_M) return fail(BT_ERR_UNSUPPORTED, "bt_gemv_packed_i8: M=%lld exceeds %d", (long long)M, BT_GEMV_MAX_M);
    int8_t* codes = (int8_t*)malloc((size_t)(N * K));
    bto_unpack_transposed(packed_T, N, K, codes);
    rc = int_linear(Xq, sx, M, K, codes, N, scale, bias, Y, y_dtype, ldy, acc_out);
    free(codes);
    return rc;
}

int bt_gemv_tiled_i8(const int8_t* Xq, const float* sx, int64_t M, int64_t K, const uint8_t* tiled, int64_t N,
                     const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy, int32_t* acc_out,
                     int flags, void* stream) {
    (void)stream;
    REQUIRE((flags & ~BT_LAUNCH_WEIGHTS_JUST_WRITTEN) == 0, "bt_gemv_tiled_i8: unknown flags %d", flags);
    REQUIRE(Xq && sx, "bt_gemv_tiled_i8: NULL pointer");
    int rc = check_linear("bt_gemv_tiled_i8", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc) return rc;
    if (M > BT_GEMV_MAX_M) return fail(BT_ERR_UNSUPPORTED, "bt_gemv_tiled_i8: M=%lld exceeds %d", (long long)M, BT_GEMV_MAX_M);
    int8_t* codes = codes_from_tiled(tiled, K, N);
    rc = int_linear(Xq, sx, M, K, codes, N, scale, bias, Y, y_dtype, ldy, acc_out);
    free(codes);
    return rc;
}

int bt_gemv_tiled(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, const uint8_t* tiled, int64_t N,
                  const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy, int8_t* xq_out,
                  float* sx_out, int32_t* acc_out, int flags, void* stream) {
    REQUIRE(X != NULL, "bt_gemv_tiled: NULL pointer");
    REQUIRE(valid_dtype(x_dtype), "bt_gemv_tiled: unknown activation dtype %d", x_dtype);
    REQUIRE(ldx >= K, "bt_gemv_tiled: row stride < K");
    int rc = check_linear("bt_gemv_tiled", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc) return rc;
    if (M > BT_GEMV_MAX_M) return fail(BT_ERR_UNSUPPORTED, "bt_gemv_tiled: M=%lld exceeds %d", (long long)M, BT_GEMV_MAX_M);
    float* x = widen(X, x_dtype, M, K, ldx);
    int8_t* xq = (int8_t*)malloc((size_t)(M * K));
    float* sx = (float*)malloc(sizeof(float) * (size_t)M);
    act_quant_rows(x, M, K, xq, sx, NULL);
    rc = bt_gemv_tiled_i8(xq, sx, M, K, tiled, N, scale, bias, Y, y_dtype, ldy, acc_out, flags, stream);
    if (xq_out) memcpy(xq_out, xq, (size_t)(M * K));
    if (sx_out) memcpy(sx_out, sx, sizeof(float) * (size_t)M);
    free(x);
    free(xq);
    free(sx);
    return rc;
}

/* Quantizer of bto_act_quant with the row maximum supplied from outside. */
static void quantize_row_with_max(const float* row, int64_t K, float mx, int8_t* q, float* sx) {
    float s = (mx > 1e-6f) ? (mx / 127.0f) : 1.0f;
    float inv = 1.0f / s;
    *sx = s;
    for (int64_t k = 0; k < K; ++k) {
        float v = fmaxf(-127.0f, fminf(127.0f, roundf(row[k] * inv)));
        q[k] = (int8_t)v;
    }
}

int bt_gemv_tiled_chained(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, const uint8_t* tiled, int64_t N,
                          const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                          const uint32_t* amax_in, uint32_t* amax_out, int64_t amax_cols, int flags, void* stream) {
    REQUIRE(X != NULL, "bt_gemv_tiled_chained: NULL pointer");
    REQUIRE((flags & ~BT_LAUNCH_WEIGHTS_JUST_WRITTEN) == 0, "bt_gemv_tiled_chained: unknown flags %d", flags);
    REQUIRE(valid_dtype(x_dtype), "bt_gemv_tiled_chained: unknown activation dtype %d", x_dtype);
    REQUIRE(ldx >= K, "bt_gemv_tiled_chained: row stride < K");
    REQUIRE(amax_in == NULL || ((uintptr_t)amax_in % 16) == 0, "bt_gemv_tiled_chained: amax_in must be 16-byte aligned");
    REQUIRE(amax_out == NULL || (amax_cols > 0 && amax_cols <= N), "bt_gemv_tiled_chained: amax_cols outside 1..N");
    int rc = check_linear("bt_gemv_tiled_chained", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc) return rc;
    if (M > BT_GEMV_MAX_M) return fail(BT_ERR_UNSUPPORTED, "bt_gemv_tiled_chained: M=%lld exceeds %d", (long long)M, BT_GEMV_MAX_M);
    float* x = widen(X, x_dtype, M, K, ldx);
    int8_t* xq = (int8_t*)malloc((size_t)(M * K));
    float* sx = (float*)malloc(sizeof(float) * (size_t)M);
    if (amax_in) {
        for (int64_t m = 0; m < M; ++m) {
            uint32_t best = 0;
            for (int s = 0; s < BT_AMAX_SLOTS; ++s)
                if (amax_in[m * BT_AMAX_SLOTS + s] > best) best = amax_in[m * BT_AMAX_SLOTS + s];
            float mx;
            memcpy(&mx, &best, 4);
            quantize_row_with_max(x + m * K, K, mx, xq + m * K, sx + m);
        }
    } else {
        act_quant_rows(x, M, K, xq, sx, NULL);
    }
    rc = bt_gemv_tiled_i8(xq, sx, M, K, tiled, N, scale, bias, Y, y_dtype, ldy, NULL, flags, stream);
    if (rc == BT_OK && amax_out) {
        for (int64_t m = 0; m < M; ++m) {
            float mx = 0.0f;
            for (int64_t n = 0; n < amax_cols; ++n) mx = fmaxf(mx, fabsf(load_elem(Y, y_dtype, m * ldy + n)));
            uint32_t bits;
            memcpy(&bits, &mx, 4);
            uint32_t* slot = amax_out + m * BT_AMAX_SLOTS + (3 * m + 5) % BT_AMAX_SLOTS;     /* any slot of the row */
            if (bits > *slot) *slot = bits;
        }
    }
    free(x);
    free(xq);
    free(sx);
    return rc;
}

/* bt_gemv_tiled_float by its definition: 32-bit fixed point from the row maximum's power of two, exact contraction. */
int bt_gemv_tiled_float(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, const uint8_t* tiled, int64_t N,
                        const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy, int flags, void* stream) {
    (void)stream;
    REQUIRE(X != NULL, "bt_gemv_tiled_float: NULL pointer");
    REQUIRE((flags & ~BT_LAUNCH_WEIGHTS_JUST_WRITTEN) == 0, "bt_gemv_tiled_float: unknown flags %d", flags);
    REQUIRE(valid_dtype(x_dtype), "bt_gemv_tiled_float: unknown activation dtype %d", x_dtype);
    REQUIRE(ldx >= K, "bt_gemv_tiled_float: row stride < K");
    int rc = check_linear("bt_gemv_tiled_float", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc) return rc;
    if (M > BT_GEMV_MAX_M) return fail(BT_ERR_UNSUPPORTED, "bt_gemv_tiled_float: M=%lld exceeds %d", (long long)M, BT_GEMV_MAX_M);
    if (K > BT_MAX_K / 2) return fail(BT_ERR_UNSUPPORTED, "bt_gemv_tiled_float: K=%lld exceeds %d", (long long)K, BT_MAX_K / 2);
    float* x = widen(X, x_dtype, M, K, ldx);
    int8_t* codes = codes_from_tiled(tiled, K, N);
    int64_t* v = (int64_t*)malloc(sizeof(int64_t) * (size_t)K);
    for (int64_t m = 0; m < M; ++m) {
        const float* row = x + m * K;
        float amax = 0.0f;
        int bad = 0;
        for (int64_t k = 0; k < K; ++k) {
            float a = fabsf(row[k]);
            amax = fmaxf(amax, a);
            if (!(a <= 3.402823466e38f)) bad = 1;
        }
        int e = 0;
        frexpf(amax, &e);
        if (e < -96) e = -96;
        if (e > 127) e = 127;
        float mult = ldexpf(1.0f, 30 - e), back = ldexpf(1.0f, e - 30);
        for (int64_t k = 0; k < K; ++k) {
            float p = row[k] * mult;
            int64_t q = (p != p) ? 0 : (int64_t)nearbyintf(p);
            if (q > (1 << 30)) q = 1 << 30;
            if (q < -(1 << 30)) q = -(1 << 30);
            v[k] = q;
        }
        for (int64_t n = 0; n < N; ++n) {
            int64_t total = 0;
            for (int64_t k = 0; k < K; ++k) total += v[k] * codes[n * K + k];
            float y = ((float)total * back) * scale[n];
            if (bias) y = y + bias[n];
            if (bad) y = NAN;
            store_elem(Y, y_dtype, m * ldy + n, y);
        }
    }
    free(v);
    free(codes);
    free(x);
    return BT_OK;
}

int bt_float_planes_quant(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* planes, float* pw,
                          int32_t* xsum, int32_t* bad, void* stream) {
    (void)stream;
    REQUIRE(X && planes && pw && xsum && bad, "bt_float_planes_quant: NULL pointer");
    REQUIRE(valid_dtype(x_dtype), "bt_float_planes_quant: unknown dtype %d", x_dtype);
    REQUIRE(M > 0 && K > 0, "bt_float_planes_quant: X is empty");
    REQUIRE(ldx >= K, "bt_float_planes_quant: row stride < K");
    if (K > BT_MAX_K / 2) return fail(BT_ERR_UNSUPPORTED, "bt_float_planes_quant: K=%lld exceeds %d", (long long)K, BT_MAX_K / 2);
    float* x = widen(X, x_dtype, M, K, ldx);
    for (int64_t m = 0; m < M; ++m) {
        const float* row = x + m * K;
        float amax = 0.0f;
        int nonfinite = 0;
        for (int64_t k = 0; k < K; ++k) {
            float a = fabsf(row[k]);
            amax = fmaxf(amax, a);
            if (!(a <= 3.402823466e38f)) nonfinite = 1;
        }
        int e = 0;
        frexpf(amax, &e);
        if (e < -96) e = -96;
        if (e > 127) e = 127;
        float mult = ldexpf(1.0f, 30 - e);
        int32_t sums[4] = {0, 0, 0, 0};
        for (int64_t k = 0; k < K; ++k) {
            float p = row[k] * mult;
            int64_t v = (p != p) ? 0 : (int64_t)nearbyintf(p);
            if (v > (1 << 30)) v = 1 << 30;
            if (v < -(1 << 30)) v = -(1 << 30);
            for (int d = 0; d < 4; ++d) {
                int b = (d < 3) ? (int)(int8_t)(v & 0xff) : (int)v;
                planes[(4 * m + d) * K + k] = (int8_t)b;
                sums[d] += b;
                v = (v - b) >> 8;
            }
        }
        for (int d = 0; d < 4; ++d) xsum[4 * m + d] = sums[d];
        pw[m] = ldexpf(1.0f, e - 30);
        bad[m] = nonfinite;
    }
    free(x);
    return BT_OK;
}

int bt_float_planes_combine(const int32_t* acc, int64_t M, int64_t N, const float* pw, const int32_t* bad, const float* scale,
                            const float* bias, void* Y, int y_dtype, int64_t ldy, void* stream) {
    (void)stream;
    REQUIRE(acc && pw && bad && scale && Y, "bt_float_planes_combine: NULL pointer");
    REQUIRE(valid_dtype(y_dtype), "bt_float_planes_combine: unknown output dtype %d", y_dtype);
    REQUIRE(M > 0 && N > 0, "bt_float_planes_combine: empty output");
    REQUIRE(ldy >= N, "bt_float_planes_combine: output row stride < N");
    if (M > 65535) return fail(BT_ERR_UNSUPPORTED, "bt_float_planes_combine: more than 65535 rows per call");
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            int64_t total = 0;
            for (int d = 3; d >= 0; --d) total = total * 256 + acc[(4 * m + d) * N + n];
            float y = ((float)total * pw[m]) * scale[n];
            if (bias) y = y + bias[n];
            if (bad[m]) y = NAN;
            store_elem(Y, y_dtype, m * ldy + n, y);
        }
    return BT_OK;
}

int bt_gemm_tiled_i8(const int8_t* Xq, const float* sx, const int32_t* xsum, int64_t M, int64_t K, const uint8_t* tiled,
                     int64_t N, const float* scale, const float* bias, void* Y, int y_dtype, int64_t ldy,
                     int32_t* acc_out, void* stream) {
    (void)stream;
    REQUIRE(Xq && sx && xsum, "bt_gemm_tiled_i8: NULL pointer");
    int rc = check_linear("bt_gemm_tiled_i8", M, K, tiled, N, scale, Y, y_dtype, ldy);
    if (rc) return rc;
    if (K % 16 != 0) return fail(BT_ERR_UNSUPPORTED, "bt_gemm_tiled_i8: K must be a multiple of 16");
    for (int64_t m = 0; m < M; ++m) {                          /* the kernel trusts xsum; the emulation checks it */
        int32_t s = 0;
        for (int64_t k = 0; k < K; ++k) s += Xq[m * K + k];
        REQUIRE(s == xsum[m], "bt_gemm_tiled_i8: xsum[%lld] is not the row sum of Xq", (long long)m);
    }
    int8_t* codes = codes_from_tiled(tiled, K, N);
    rc = int_linear(Xq, sx, M, K, codes, N, scale, bias, Y, y_dtype, ldy, acc_out);
    free(codes);
    return rc;
}

int bt_silu_mul_quant(const void* GU, int dtype, int64_t M, int64_t F, int64_t ld, int8_t* Hq, float* sx, int32_t* xsum,
                      void* H, void* stream) {
    (void)stream;
    REQUIRE(GU && Hq && sx, "bt_silu_mul_quant: NULL pointer");
    REQUIRE(valid_dtype(dtype), "bt_silu_mul_quant: unknown dtype %d", dtype);
    REQUIRE(M > 0 && F > 0, "bt_silu_mul_quant: input is empty");
    REQUIRE(ld >= 2 * F, "bt_silu_mul_quant: row stride < 2F");
    float* gu = widen(GU, dtype, M, 2 * F, ld);
    float* h = H ? (float*)malloc(sizeof(float) * (size_t)(M * F)) : NULL;
    bto_silu_mul_quant(gu, M, F, 2 * F, dtype, Hq, sx, xsum, h);
    if (H)
        for (int64_t i = 0; i < M * F; ++i) store_elem(H, dtype, i, h[i]);
    free(gu);
    free(h);
    return BT_OK;
}

int bt_add_rmsnorm_quant(void* X, const void* delta, int dtype, int64_t M, int64_t D, int64_t ldx, int64_t ldd,
                         const void* weight, float eps, int8_t* Yq, float* sx, int32_t* xsum, void* Y, void* stream) {
    (void)stream;
    REQUIRE(X && weight && Yq && sx, "bt_add_rmsnorm_quant: NULL pointer");
    REQUIRE(valid_dtype(dtype), "bt_add_rmsnorm_quant: unknown dtype %d", dtype);
    REQUIRE(M > 0 && D > 0, "bt_add_rmsnorm_quant: input is empty");
    REQUIRE(ldx >= D && (!delta || ldd >= D), "bt_add_rmsnorm_quant: row stride smaller than D");
    REQUIRE(eps >= 0.0f, "bt_add_rmsnorm_quant: eps must not be negative");
    float* x = widen(X, dtype, M, D, ldx);
    float* d = delta ? widen(delta, dtype, M, D, ldd) : NULL;
    float* w = widen(weight, dtype, 1, D, D);
    float* y = Y ? (float*)malloc(sizeof(float) * (size_t)(M * D)) : NULL;
    bto_add_rmsnorm_quant(x, d, M, D, D, D, w, eps, dtype, Yq, sx, xsum, y);
    if (delta)
        for (int64_t m = 0; m < M; ++m)
            for (int64_t k = 0; k < D; ++k) store_elem(X, dtype, m * ldx + k, x[m * D + k]);
    if (Y)
        for (int64_t i = 0; i < M * D; ++i) store_elem(Y, dtype, i, y[i]);
    free(x);
    free(d);
    free(w);
    free(y);
    return BT_OK;
}

static int float_linear(const void* X, int x_dtype, int64_t M, int64_t K, const int8_t* codes, int64_t N,
                        const float* scale, const float* bias, void* Y) {
    float* x = widen(X, x_dtype, M, K, K);
    float* y = (float*)malloc(sizeof(float) * (size_t)(M * N));
    bto_linear_float(x, M, K, codes, N, scale, bias, y);
    for (int64_t i = 0; i < M * N; ++i) store_elem(Y, x_dtype, i, y[i]);
    free(x);
    free(y);
    return BT_OK;
}

int bt_linear_unpacked(const void* X, int x_dtype, int64_t M, int64_t K, const int8_t* W, int64_t N, const float* scale,
                       const float* bias, void* Y, void* stream) {
    (void)stream;
    REQUIRE(X && W && scale && Y, "bt_linear_unpacked: NULL pointer");
    REQUIRE(valid_dtype(x_dtype) || x_dtype == BT_F64, "bt_linear_unpacked: unknown dtype %d", x_dtype);
    REQUIRE(M > 0 && K > 0 && N > 0, "bt_linear_unpacked: X is empty");
    return float_linear(X, x_dtype, M, K, W, N, scale, bias, Y);
}

int bt_linear_packed_float(const void* X, int x_dtype, int64_t M, int64_t K, const uint8_t* packed_T, int64_t N,
                           const float* scale, const float* bias, void* Y, void* stream) {
    (void)stream;
    REQUIRE(X && packed_T && scale && Y, "bt_linear_packed_float: NULL pointer");
    REQUIRE(valid_dtype(x_dtype) || x_dtype == BT_F64, "bt_linear_packed_float: unknown dtype %d", x_dtype);
    REQUIRE(M > 0 && K > 0 && N > 0, "bt_linear_packed_float: X is empty");
    int8_t* codes = (int8_t*)malloc((size_t)(N * K));
    bto_unpack_transposed(packed_T, N, K, codes);
    int rc = float_linear(X, x_dtype, M, K, codes, N, scale, bias, Y);
    free(codes);
    return rc;
}
