/*
 * bittorch_b200 — C ABI of the B200 (sm_100a) ternary linear backend.
 *
 * This header is the drop-in boundary: a torch-free shared library
 * (libbittorch_b200.so) whose entry points take raw device pointers, explicit
 * sizes and a CUDA stream.  It replaces the reference's pybind11 extension
 * `bittorch._C` (csrc/bindings/bittorch_bindings.cpp:34-88) and the host dispatch
 * behind it (csrc/core/dispatch.cpp).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless said otherwise;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *     all work is enqueued on it and nothing synchronises unless stated;
 *   - return value: BT_OK (0) or a BT_ERR_* code; bt_last_error() then returns a
 *     human-readable message for the calling thread;
 *   - no entry point allocates or frees device memory; outputs and workspaces
 *     are the caller's (sizes from the bt_*_bytes helpers);
 *   - nothing throws or aborts across this boundary, and no kernel traps: a
 *     device-side wait that runs out records a code readable with
 *     bt_device_status().
 *   - scale / bias vectors are always float32 on this side of the boundary; the
 *     Python layer converts the (tiny) [N] vectors when the reference API hands
 *     them over in fp16 / bf16.
 */
#ifndef BITTORCH_B200_H
#define BITTORCH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BT_OK 0
#define BT_ERR_INVALID 1      /* bad argument (shape, alignment, NULL, dtype) */
#define BT_ERR_CUDA 2         /* a CUDA runtime call or launch failed */
#define BT_ERR_UNSUPPORTED 3  /* valid request outside the kernel's limits */
#define BT_ERR_DEVICE_WAIT 4  /* a bounded device-side wait ran out */

/* Element types of activations / master weights / outputs. */
#define BT_F32 0
#define BT_F16 1
#define BT_BF16 2
/* float64: accepted by the two floating-point-activation entry points only
 * (bt_linear_unpacked, bt_linear_packed_float), as the reference dispatches them
 * (AT_DISPATCH_FLOATING_TYPES_AND_HALF, csrc/kernels/ternary_gemm.cu:248,
 * csrc/kernels/ternary_gemm_production.cu:331). */
#define BT_F64 3

/* Launch flags of the decode entry points (bt_gemv_tiled, bt_gemv_tiled_i8). */
#define BT_LAUNCH_DEFAULT 0
/* The weights, scales or bias of this call were written by work enqueued just before
 * it on the same stream (a fresh quantize / re-tile / copy): launch fully
 * stream-ordered.  Without the flag the decode kernel is launched with programmatic
 * dependent launch and reads scale / bias and starts streaming its WEIGHTS before the
 * preceding kernel has finished (only the activations are read after the dependency
 * wait), which is what lets consecutive layers overlap. */
#define BT_LAUNCH_WEIGHTS_JUST_WRITTEN 1

/* Kernel-selection overrides for tests and tuning, bt_set_tuning(knob, value); value -1
 * (the default) lets the library choose.  Each knob's initial value comes from the
 * environment variable named beside it, read once. */
#define BT_TUNE_GEMM_PAIR 0   /* BITTORCH_B200_GEMM_PAIR : 1 / 0 force the CTA-pair GEMM on / off */
#define BT_TUNE_GEMM_BN 1     /* BITTORCH_B200_GEMM_BN   : 64 / 128 / 256 output-tile width */
#define BT_TUNE_GEMM_SPLIT 2  /* BITTORCH_B200_GEMM_SPLIT: 1 / 2 / 4 / 8 K split of the narrow-batch GEMM */
#define BT_TUNE_GEMV_SPLIT 3  /* BITTORCH_B200_GEMV_SPLIT: 1 / 2 / 4 / 8 K split of bt_gemv_packed_i8 */
#define BT_TUNE_COUNT 4

/* Largest M handled by the decode (GEMV) kernels. */
#define BT_GEMV_MAX_M 16
/* Words per row of the row-maximum buffers of bt_gemv_tiled_chained. */
#define BT_AMAX_SLOTS 8
/* Largest K of the integer kernels: keeps 128*127*K inside int32. */
#define BT_MAX_K 131072

/* Library version, major*10000 + minor*100 + patch. */
int bt_version(void);

/* Message for the last non-zero return on the calling thread ("" if none). */
const char* bt_last_error(void);

/*
 * Reads (and clears) the sticky device-side status word of the current device:
 * 0, or BT_ERR_DEVICE_WAIT if some kernel gave up on a bounded wait since the
 * last call.  Synchronises `stream`.
 */
int bt_device_status(int* status_host, void* stream);

/* Process-wide; takes effect for later calls.  No counterpart in the reference. */
int bt_set_tuning(int knob, int value);

/*
 * Enqueues a one-warp kernel whose bounded wait can never be satisfied and gives up
 * after a few thousand polls (microseconds): afterwards bt_device_status() reads
 * BT_ERR_DEVICE_WAIT once and then 0 again.  Lets a caller check the give-up path of
 * the library's device-side waits - status word, normal kernel exit, usable context -
 * without any real kernel failing.  No counterpart in the reference.
 */
int bt_selftest_wait_timeout(void* stream);

/*
 * Device-to-device clone of `bytes` bytes.
 * Replaces `_C.dummy` (csrc/core/dispatch.cpp:7-9).
 */
int bt_dummy(const void* src, void* dst, size_t bytes, void* stream);

/*
 * Fused weight ternarizer + 2-bit packer.
 *   scale[n] = clamp(max_k |W[n,k]|, 1e-8);  thr = threshold_factor * scale[n];
 *   code     = |W| > thr ? sign(W) : 0;      byte[kb,n] = codes of W[n,4kb..4kb+3]
 * (0 -> 00, +1 -> 01, -1 -> 10, K padded with zeros), arithmetic in W's dtype.
 * Replaces bittorch.quant.ternary_quantize (bittorch/quant/ternary.py:100-150)
 * followed by pack_ternary_transposed (bittorch/quant/ternary_packed.py:174-206).
 *
 * W         [N,K] row-major with row stride ldw (elements), dtype w_dtype
 * packed_T  uint8 [ceil(K/4), N]            (may be NULL)
 * scale     float32 [N]                     (values are exact widenings of w_dtype)
 * codes     int8 [N,K] in {-1,0,+1}         (may be NULL)
 * tern      [N,K] contiguous, dtype w_dtype, values -1/0/+1 (may be NULL);
 *           this is what TernaryLinear.get_quantized_weight() returns
 *           (bittorch/nn/ternary_linear.py:227-242).
 */
int bt_quantize_pack(const void* W, int w_dtype, int64_t N, int64_t K, int64_t ldw,
                     float threshold_factor, uint8_t* packed_T, float* scale,
                     int8_t* codes, void* tern, void* stream);

/*
 * 2-bit packer / unpacker for already-ternary weights.
 * Replace pack_ternary_transposed / unpack_ternary_transposed
 * (bittorch/quant/ternary_packed.py:174-223).  codes: int8 [N,K].  The reserved
 * bit pattern 11 decodes to 0 (ternary_packed.py:112-115).
 */
int bt_pack_codes(const int8_t* codes, int64_t N, int64_t K, uint8_t* packed_T, void* stream);
int bt_unpack_codes(const uint8_t* packed_T, int64_t N, int64_t K, int8_t* codes, void* stream);

/*
 * The same bytes in the row layout uint8 [N, ceil(K/4)] (byte [n,kb] = codes of
 * W[n,4kb..4kb+3]): pack_ternary / unpack_ternary
 * (bittorch/quant/ternary_packed.py:22-75, 78-120) and the browser runtime's weight
 * format (js/src/core/types.ts:9).
 */
int bt_pack_codes_rows(const int8_t* codes, int64_t N, int64_t K, uint8_t* packed, void* stream);
int bt_unpack_codes_rows(const uint8_t* packed, int64_t N, int64_t K, int8_t* codes, void* stream);

/*
 * Per-token int8 activation quantizer (one scale per row of X):
 *   s = max|x| > 1e-6 ? max|x|/127 : 1;  q = clamp(roundf(x * (1/s)), -127, 127)
 * Replaces the in-kernel quantizer of the reference's integer kernel
 * (csrc/kernels/ternary_gemm_tensor_core.cu:343-347, 424-459), applied per row as
 * that file's header specifies (:16-18).
 * X [M,K] row stride ldx, dtype x_dtype; Xq int8 [M,K]; sx float32 [M];
 * xsum int32 [M] (optional): per-row sums of the int8 codes, an input of
 * bt_gemm_tiled_i8 (which multiplies weights stored as t+1).
 */
int bt_act_quant_i8(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                    int8_t* Xq, float* sx, int32_t* xsum, void* stream);

/*
 * Private streaming layout of the packed weights ("tiled"): still 2 bits per
 * weight, re-ordered into 512-byte tiles of 16 output columns x 128 inputs, the
 * tiles of a column block contiguous along K, so that a column block is one bulk
 * copy and one 16-byte load per lane yields ready-made dp4a operands.  It is a derived
 * cache of the public [ceil(K/4),N] buffer and round-trips to it bit for bit.
 * (No counterpart in the reference; the public buffer stays the wire format of
 * TernaryLinearInference.weight_packed, bittorch/nn/ternary_linear_infer.py:68-73.)
 */
size_t bt_tiled_bytes(int64_t K, int64_t N);
int bt_retile_packed(const uint8_t* packed_T, int64_t K, int64_t N, uint8_t* tiled, void* stream);
int bt_untile_packed(const uint8_t* tiled, int64_t K, int64_t N, uint8_t* packed_T, void* stream);

/*
 * Decode-size (M <= BT_GEMV_MAX_M) packed ternary linear on int8 activations:
 *   acc[m,n] = sum_k Xq[m,k] * T[n,k]            (int32, exact)
 *   Y[m,n]   = (float(acc) * sx[m]) * scale[n] + bias[n]
 * bt_gemv_packed_i8 reads the public [ceil(K/4),N] buffer, bt_gemv_tiled_i8 the
 * tiled one (the bandwidth-bound fast path).  Both replace
 * ternary_linear_packed_forward for small batches
 * (csrc/core/dispatch.cpp:105-142; csrc/kernels/ternary_gemm_production.cu:53-142)
 * with the integer arithmetic of csrc/kernels/ternary_gemm_tensor_core.cu:349-657.
 *
 * Xq int8 [M,K] contiguous; sx float32 [M]; scale float32 [N]; bias float32 [N] or NULL;
 * Y [M,N] row stride ldy, dtype y_dtype; acc_out int32 [M,N] or NULL (parity checks).
 * bt_gemv_tiled_i8 / bt_gemv_tiled: `flags` is BT_LAUNCH_DEFAULT, or
 * BT_LAUNCH_WEIGHTS_JUST_WRITTEN when tiled / scale / bias were produced by the work
 * enqueued just before this call (see the flag's comment): PRECONDITION of the default.
 */
int bt_gemv_packed_i8(const int8_t* Xq, const float* sx, int64_t M, int64_t K,
                      const uint8_t* packed_T, int64_t N, const float* scale, const float* bias,
                      void* Y, int y_dtype, int64_t ldy, int32_t* acc_out, void* stream);
int bt_gemv_tiled_i8(const int8_t* Xq, const float* sx, int64_t M, int64_t K,
                     const uint8_t* tiled, int64_t N, const float* scale, const float* bias,
                     void* Y, int y_dtype, int64_t ldy, int32_t* acc_out, int flags, void* stream);

/*
 * Decode-size packed ternary linear straight from floating-point activations: the
 * per-token int8 quantizer of bt_act_quant_i8 runs inside the GEMV kernel (every CTA
 * quantizes the few activation rows itself, into shared memory, while its weights stream in),
 * so a decode layer is ONE dependent kernel launch.  Results are bit-identical to
 * bt_act_quant_i8 followed by bt_gemv_tiled_i8.
 * Replaces the quantize-inside-the-GEMM structure of the reference's integer kernel
 * (csrc/kernels/ternary_gemm_tensor_core.cu:396-459) for small batches.
 *
 * X [M,K] row stride ldx, dtype x_dtype, M <= BT_GEMV_MAX_M; other arguments as
 * bt_gemv_tiled_i8.  xq_out int8 [M,K] and sx_out float32 [M] (both optional) receive
 * the quantized activations the kernel used (parity checks).
 */
int bt_gemv_tiled(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                  const uint8_t* tiled, int64_t N, const float* scale, const float* bias,
                  void* Y, int y_dtype, int64_t ldy, int8_t* xq_out, float* sx_out,
                  int32_t* acc_out, int flags, void* stream);

/*
 * bt_gemv_tiled for layers that feed one another: the kernel that WRITES a layer's
 * activations also publishes each row's max |y|, so the kernel that READS them takes its
 * per-token quantization scale from there instead of reducing the row first (no
 * row-maximum pass and no block-wide barrier in front of the quantizer).  Results are
 * bit-identical to bt_gemv_tiled: the maximum is taken over the values as stored in
 * y_dtype, which are the values the consumer would have reduced.
 * (No counterpart in the reference, whose integer kernel re-derives the scale inside
 * every tile: csrc/kernels/ternary_gemm_tensor_core.cu:424-444.)
 *
 * amax_out  uint32 [M][BT_AMAX_SLOTS] or NULL: receives, by atomic maximum on the float
 *           bit patterns, max |Y[m, 0..amax_cols)| spread over the BT_AMAX_SLOTS words of
 *           row m (their maximum is the row's value).  MUST BE ZERO before the launch
 *           (one memset for all layers of a step); amax_cols = the leading columns the
 *           consumer reads (its K).
 * amax_in   uint32 [M][BT_AMAX_SLOTS] or NULL, 16-byte aligned: what the producer of X
 *           published.  Preconditions: that producer stored exactly this call's
 *           X[0..M, 0..K) in x_dtype with amax_cols == K, and nothing modified X since.
 *           With NULL the kernel reduces the rows itself, like bt_gemv_tiled.
 * Other arguments and `flags` as bt_gemv_tiled (no debug outputs).
 */
int bt_gemv_tiled_chained(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                          const uint8_t* tiled, int64_t N, const float* scale, const float* bias,
                          void* Y, int y_dtype, int64_t ldy, const uint32_t* amax_in,
                          uint32_t* amax_out, int64_t amax_cols, int flags, void* stream);

/*
 * Decode-size packed ternary linear with FLOATING-POINT activations (no activation
 * quantization): Y[m,n] = (sum_k X[m,k] * T[n,k]) * scale[n] + bias[n], the arithmetic of
 * the reference's packed float kernel (csrc/kernels/ternary_gemm_production.cu:53-142,
 * decode (c==1)-(c==2) at :37-39) on the tiled layout at the decode kernel's streaming rate.
 * The sum is computed EXACTLY: each activation row is rescaled by a power of two into 32-bit
 * fixed point (elements within 2^6 of the row's largest magnitude exactly, the rest to 2^-30
 * of it), split into four signed-byte digit planes that go through the integer pipeline as
 * four int8 rows, and recombined in 64-bit arithmetic; one rounding to float follows, then
 * scale and bias.  The result is therefore independent of summation order and at least as
 * close to the real-number result as the reference's fp32 accumulation (whose own tests allow
 * 1e-4, tests/test_packed_kernel.py:50).  A row containing an infinity or a NaN yields NaN.
 * X [M,K] row stride ldx, dtype x_dtype, M <= BT_GEMV_MAX_M (two rows per launch), K <=
 * BT_MAX_K / 2; other arguments and `flags` as bt_gemv_tiled.
 */
int bt_gemv_tiled_float(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                        const uint8_t* tiled, int64_t N, const float* scale, const float* bias,
                        void* Y, int y_dtype, int64_t ldy, int flags, void* stream);

/*
 * The same construction around the tensor-core GEMM, for any batch size: the reference's
 * float-activation kernels for large batches (csrc/kernels/ternary_gemm_production.cu:158-250;
 * csrc/kernels/ternary_gemm_tensor_core.cu:120-271, "version 1") as three calls,
 *   bt_float_planes_quant   X [M,K] -> int8 digit planes [4M,K] (row 4m+p = digit p of row m),
 *                           their int32 row sums xsum [4M], pw float32 [M] (the power of two
 *                           that undoes the scaling), bad int32 [M] (row holds inf / NaN)
 *   bt_gemm_tiled_i8        on the planes as 4M int8 rows (sx: any values, e.g. ones), with
 *                           acc_out int32 [4M,N]
 *   bt_float_planes_combine acc, pw, bad, scale, bias -> Y [M,N]: the four accumulators of
 *                           an output recombined in 64 bits, one rounding to float, exact
 *                           power of two, scale, bias; NaN for flagged rows
 * giving the correctly rounded exact sum at a quarter of the int8 tensor-core rate.
 * K <= BT_MAX_K / 2 (and a multiple of 16 for the GEMM); at most 65535 rows per combine call.
 */
int bt_float_planes_quant(const void* X, int x_dtype, int64_t M, int64_t K, int64_t ldx,
                          int8_t* planes, float* pw, int32_t* xsum, int32_t* bad, void* stream);
int bt_float_planes_combine(const int32_t* acc, int64_t M, int64_t N, const float* pw,
                            const int32_t* bad, const float* scale, const float* bias,
                            void* Y, int y_dtype, int64_t ldy, void* stream);

/*
 * Prefill-size packed ternary linear on int8 activations (any M >= 1), same
 * arithmetic as above, contraction on the 5th-generation tensor cores
 * (tcgen05.mma kind::i8, accumulators in tensor memory).  Reads the tiled layout.
 * Replaces ternary_linear_packed_forward for large batches
 * (csrc/kernels/ternary_gemm_production.cu:158-250) and the experimental
 * mma.sync kernel (csrc/kernels/ternary_gemm_tensor_core.cu:349-657).
 * xsum int32 [M]: per-row sums of Xq, as written by bt_act_quant_i8 (required).
 * K must be a multiple of 16 (row pitch of the TMA descriptor over Xq).
 * Three kernels behind this entry, chosen by shape: CTA pairs (tcgen05.mma.cta_group::2, 256 x 256
 * tiles) when there are enough such tiles; one CTA per 128 x {256,128,64} tile otherwise; and, up to
 * 32 rows, full-width tiles with K split over a thread-block cluster whose partial accumulators meet
 * in distributed shared memory.  None uses global scratch memory; results do not depend on the choice.
 * All three wait for the preceding kernel before their first global read, so the call is
 * stream-ordered with respect to every operand (no precondition on freshly written weights).
 */
int bt_gemm_tiled_i8(const int8_t* Xq, const float* sx, const int32_t* xsum, int64_t M, int64_t K,
                     const uint8_t* tiled, int64_t N, const float* scale, const float* bias,
                     void* Y, int y_dtype, int64_t ldy, int32_t* acc_out, void* stream);

/*
 * Elementwise steps of a decoder block fused with the per-token int8 quantizer of
 * bt_act_quant_i8, so that the packed layer behind them starts from int8 rows + scales
 * (bt_gemv_tiled_i8 / bt_gemm_tiled_i8).  No counterpart in the reference's Python
 * package; the steps are those of its browser runtime (SwiGLU:
 * js/src/models/TernaryTransformer.ts:520-550; pre-norm residual block: :366-464; RMSNorm
 * with eps inside the root: js/src/core/RMSNorm.ts:10-38).  Values are rounded to the
 * activation type `dtype` wherever the unfused sequence of operations would have stored
 * them; the arithmetic is fixed operation by operation (see csrc/fused_elementwise.cuh), so
 * results do not depend on the launch.
 *
 * bt_silu_mul_quant:    h = silu(gate) * up.  GU [M, ld] holds gate in columns [0, F) and up
 *                       in [F, 2F) (the output of a fused gate/up layer).  Hq int8 [M, F],
 *                       sx float32 [M], xsum int32 [M] or NULL, H [M, F] in dtype or NULL
 *                       (the unquantized product).
 * bt_add_rmsnorm_quant: x += delta (delta NULL: no addition); y = x / sqrt(mean(x^2) + eps)
 *                       * weight.  X [M, ldx] is UPDATED IN PLACE (the residual stream),
 *                       delta [M, ldd], weight [D] in dtype.  Yq int8 [M, D], sx, xsum as
 *                       above, Y [M, D] in dtype or NULL (the unquantized normalised row).
 */
int bt_silu_mul_quant(const void* GU, int dtype, int64_t M, int64_t F, int64_t ld,
                      int8_t* Hq, float* sx, int32_t* xsum, void* H, void* stream);
int bt_add_rmsnorm_quant(void* X, const void* delta, int dtype, int64_t M, int64_t D,
                         int64_t ldx, int64_t ldd, const void* weight, float eps,
                         int8_t* Yq, float* sx, int32_t* xsum, void* Y, void* stream);

/*
 * Unpacked-weight linear with floating-point activations, fp32 accumulation:
 *   Y[b,n] = (sum_k X[b,k] * W[n,k]) * scale[n] + bias[n],   W int8 [N,K]
 * Replaces `_C.ternary_linear_forward` (csrc/core/dispatch.cpp:52-87;
 * csrc/kernels/ternary_gemm.cu:41-177).  x_dtype may be BT_F64: X and Y are float64
 * and the arithmetic is still float32, as in the reference (`static_cast<float>(X[...])`,
 * csrc/kernels/ternary_gemm.cu:56-61); scale / bias stay float32 on this side of the boundary.
 */
int bt_linear_unpacked(const void* X, int x_dtype, int64_t M, int64_t K,
                       const int8_t* W, int64_t N, const float* scale, const float* bias,
                       void* Y, void* stream);

/*
 * Packed-weight linear with floating-point activations, fp32 accumulation (the
 * reference's exact float semantics, for callers that need its 1e-4 agreement):
 *   Y[b,n] = (sum_k X[b,k] * T[n,k]) * scale[n] + bias[n]
 * Replaces the float arithmetic of `_C.ternary_linear_packed_forward`
 * (csrc/kernels/ternary_gemm_production.cu:53-250).  Reads the public layout.
 * x_dtype may be BT_F64.
 */
int bt_linear_packed_float(const void* X, int x_dtype, int64_t M, int64_t K,
                           const uint8_t* packed_T, int64_t N, const float* scale, const float* bias,
                           void* Y, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BITTORCH_B200_H */
