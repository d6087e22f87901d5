"""ctypes binding of ``libbittorch_b200.so`` (the C ABI declared in include/bittorch_b200.h).

This module stands where the reference has its pybind11 extension ``bittorch._C``
(csrc/bindings/bittorch_bindings.cpp:34-88): it exposes the same four callables
(``dummy``, ``ternary_linear_forward``, ``ternary_linear_packed_forward``,
``ternary_linear_tensor_core_forward``) with the argument checks of
csrc/core/dispatch.cpp:52-142 raised as ``RuntimeError``, plus thin wrappers of the
new entry points.  Importing it fails with ``ImportError`` when the library has not
been built; nothing here computes on the CPU.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _build

BT_F32, BT_F16, BT_BF16, BT_F64 = 0, 1, 2, 3
LAUNCH_DEFAULT, LAUNCH_WEIGHTS_JUST_WRITTEN = 0, 1
TUNE_GEMM_PAIR, TUNE_GEMM_BN, TUNE_GEMM_SPLIT, TUNE_GEMV_SPLIT = 0, 1, 2, 3
AMAX_SLOTS = 8           # words per row of the row-maximum buffers of gemv_tiled_chained
GEMV_MAX_M = 16          # largest batch the decode kernels accept
DECODE_MAX_M = 4         # batches up to here run the decode kernel; above it the tensor-core kernel is faster
_DT = {torch.float32: BT_F32, torch.float16: BT_F16, torch.bfloat16: BT_BF16}
_DT_FLOAT_PATH = dict(_DT)
_DT_FLOAT_PATH[torch.float64] = BT_F64     # the floating-point-activation entry points also take float64

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_f32 = ctypes.c_float

_SIGNATURES = {
    "bt_version": ([], _int),
    "bt_last_error": ([], ctypes.c_char_p),
    "bt_device_status": ([_p, _p], _int),
    "bt_set_tuning": ([_int, _int], _int),
    "bt_selftest_wait_timeout": ([_p], _int),
    "bt_dummy": ([_p, _p, ctypes.c_size_t, _p], _int),
    "bt_quantize_pack": ([_p, _int, _i64, _i64, _i64, _f32, _p, _p, _p, _p, _p], _int),
    "bt_pack_codes": ([_p, _i64, _i64, _p, _p], _int),
    "bt_unpack_codes": ([_p, _i64, _i64, _p, _p], _int),
    "bt_pack_codes_rows": ([_p, _i64, _i64, _p, _p], _int),
    "bt_unpack_codes_rows": ([_p, _i64, _i64, _p, _p], _int),
    "bt_act_quant_i8": ([_p, _int, _i64, _i64, _i64, _p, _p, _p, _p], _int),
    "bt_tiled_bytes": ([_i64, _i64], ctypes.c_size_t),
    "bt_retile_packed": ([_p, _i64, _i64, _p, _p], _int),
    "bt_untile_packed": ([_p, _i64, _i64, _p, _p], _int),
    "bt_gemv_packed_i8": ([_p, _p, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _p, _p], _int),
    "bt_gemv_tiled_i8": ([_p, _p, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _p, _int, _p], _int),
    "bt_gemv_tiled": ([_p, _int, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _p, _p, _p, _int, _p], _int),
    "bt_gemv_tiled_chained": ([_p, _int, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _p, _p, _i64, _int, _p], _int),
    "bt_gemv_tiled_float": ([_p, _int, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _int, _p], _int),
    "bt_float_planes_quant": ([_p, _int, _i64, _i64, _i64, _p, _p, _p, _p, _p], _int),
    "bt_float_planes_combine": ([_p, _i64, _i64, _p, _p, _p, _p, _p, _int, _i64, _p], _int),
    "bt_gemm_tiled_i8": ([_p, _p, _p, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _p, _p], _int),
    "bt_silu_mul_quant": ([_p, _int, _i64, _i64, _i64, _p, _p, _p, _p, _p], _int),
    "bt_add_rmsnorm_quant": ([_p, _p, _int, _i64, _i64, _i64, _i64, _p, _f32, _p, _p, _p, _p, _p], _int),
    "bt_linear_unpacked": ([_p, _int, _i64, _i64, _p, _i64, _p, _p, _p, _p], _int),
    "bt_linear_packed_float": ([_p, _int, _i64, _i64, _p, _i64, _p, _p, _p, _p], _int),
}


def _load() -> ctypes.CDLL:
    path = os.environ.get("BITTORCH_B200_LIB", _build.LIB_PATH)
    if not os.path.exists(path):
        raise ImportError(
            f"bittorch_b200: {path} has not been built; run `python -m bittorch_b200._build`"
        )
    try:
        lib = ctypes.CDLL(path)
    except OSError as exc:  # pragma: no cover - depends on the machine
        raise ImportError(f"bittorch_b200: cannot load {path}: {exc}") from exc
    for name, (argtypes, restype) in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise ImportError(f"bittorch_b200: {path} is stale (no symbol {name}); rebuild it with "
                              "`python -m bittorch_b200._build`") from exc
        fn.argtypes = argtypes
        fn.restype = restype
    return lib


_lib = _load()
LIB_PATH = _lib._name
EXPORTED = tuple(_SIGNATURES)


def version() -> int:
    return int(_lib.bt_version())


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(_lib.bt_last_error().decode("utf-8", "replace") or f"bittorch_b200 error {rc}")


def _ptr(t: Optional[Tensor]):
    return None if t is None else t.data_ptr()


def _stream(t: Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def _dtype_code(t: Tensor, what: str, float_path: bool = False) -> int:
    try:
        return (_DT_FLOAT_PATH if float_path else _DT)[t.dtype]
    except KeyError:
        raise RuntimeError(f"{what} must be float32, float16 or bfloat16"
                           f"{' or float64' if float_path else ''}, got {t.dtype}") from None


def _f32vec(t: Optional[Tensor]) -> Optional[Tensor]:
    """scale / bias cross the C ABI as contiguous float32 vectors."""
    if t is None:
        return None
    return t.detach().to(torch.float32).contiguous()


def set_tuning(knob: int, value: int) -> None:
    """Kernel-selection override for tests and tuning (``TUNE_*``); -1 = automatic.  Process-wide."""
    _check(_lib.bt_set_tuning(int(knob), int(value)))


def selftest_wait_timeout(device=None) -> None:
    """Enqueues the library's wait-timeout self-test kernel; ``device_status`` then reads 4 once."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _check(_lib.bt_selftest_wait_timeout(torch.cuda.current_stream(dev).cuda_stream))


def device_status(device=None) -> int:
    """Reads and clears the sticky device-side status word (synchronises the stream)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    out = ctypes.c_int(0)
    with torch.cuda.device(dev):
        _check(_lib.bt_device_status(ctypes.byref(out), torch.cuda.current_stream(dev).cuda_stream))
    return out.value


# ---------------------------------------------------------------------------------------
# New entry points (tensor-level wrappers; every tensor must live on a CUDA device)
# ---------------------------------------------------------------------------------------

def _require_cuda(*tensors: Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("All tensors must be CUDA")


def quantize_pack(
    weight: Tensor,
    threshold_factor: float = 0.05,
    want_packed: bool = True,
    want_codes: bool = False,
    want_tern: bool = False,
) -> dict:
    """Fused ternarize (+ pack) of a [N,K] master weight on the GPU.

    Returns a dict with ``scale`` (float32 [N]) and, as requested, ``packed_T``
    (uint8 [ceil(K/4),N]), ``codes`` (int8 [N,K]) and ``tern`` (weight dtype [N,K]).
    """
    _require_cuda(weight)
    if weight.dim() != 2:
        raise RuntimeError(f"weight must be 2D [N, K], got {weight.dim()}D")
    w = weight.detach()
    if w.stride(1) != 1 or w.stride(0) < w.shape[1]:
        w = w.contiguous()
    n, k = w.shape
    if n == 0 or k == 0:
        raise RuntimeError("weight is empty")
    dev = w.device
    out = {"scale": torch.empty(n, dtype=torch.float32, device=dev)}
    if want_packed:
        out["packed_T"] = torch.empty(((k + 3) // 4, n), dtype=torch.uint8, device=dev)
    if want_codes:
        out["codes"] = torch.empty((n, k), dtype=torch.int8, device=dev)
    if want_tern:
        out["tern"] = torch.empty((n, k), dtype=w.dtype, device=dev)
    with torch.cuda.device(dev):
        _check(_lib.bt_quantize_pack(
            _ptr(w), _dtype_code(w, "weight"), n, k, w.stride(0), float(threshold_factor),
            _ptr(out.get("packed_T")), _ptr(out["scale"]), _ptr(out.get("codes")), _ptr(out.get("tern")), _stream(w)))
    return out


def pack_codes(codes: Tensor) -> Tensor:
    """int8 codes [N,K] -> public packed uint8 [ceil(K/4), N]."""
    _require_cuda(codes)
    codes = codes.contiguous()
    n, k = codes.shape
    out = torch.empty(((k + 3) // 4, n), dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        _check(_lib.bt_pack_codes(_ptr(codes), n, k, _ptr(out), _stream(codes)))
    return out


def pack_codes_rows(codes: Tensor) -> Tensor:
    """int8 codes [N,K] -> packed uint8 [N, ceil(K/4)] (the row layout of ``pack_ternary``)."""
    _require_cuda(codes)
    codes = codes.contiguous()
    n, k = codes.shape
    out = torch.empty((n, (k + 3) // 4), dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        _check(_lib.bt_pack_codes_rows(_ptr(codes), n, k, _ptr(out), _stream(codes)))
    return out


def unpack_codes_rows(packed: Tensor, in_features: int) -> Tensor:
    """packed uint8 [N, ceil(K/4)] -> int8 codes [N,K]."""
    _require_cuda(packed)
    packed = packed.contiguous()
    n = packed.shape[0]
    out = torch.empty((n, in_features), dtype=torch.int8, device=packed.device)
    with torch.cuda.device(packed.device):
        _check(_lib.bt_unpack_codes_rows(_ptr(packed), n, in_features, _ptr(out), _stream(packed)))
    return out


def unpack_codes(packed_T: Tensor, in_features: int) -> Tensor:
    """public packed uint8 [ceil(K/4), N] -> int8 codes [N,K]."""
    _require_cuda(packed_T)
    packed_T = packed_T.contiguous()
    n = packed_T.shape[1]
    out = torch.empty((n, in_features), dtype=torch.int8, device=packed_T.device)
    with torch.cuda.device(packed_T.device):
        _check(_lib.bt_unpack_codes(_ptr(packed_T), n, in_features, _ptr(out), _stream(packed_T)))
    return out


def act_quant_i8(x2d: Tensor, want_sum: bool = False):
    """Per-row int8 quantization of a [M,K] activation matrix -> (int8 [M,K], float32 [M]),
    plus the int32 row sums of the codes when ``want_sum`` (an input of ``gemm_tiled_i8``)."""
    _require_cuda(x2d)
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    m, k = x2d.shape
    xq = torch.empty((m, k), dtype=torch.int8, device=x2d.device)
    sx = torch.empty((m,), dtype=torch.float32, device=x2d.device)
    xsum = torch.empty((m,), dtype=torch.int32, device=x2d.device) if want_sum else None
    with torch.cuda.device(x2d.device):
        _check(_lib.bt_act_quant_i8(_ptr(x2d), _dtype_code(x2d, "X"), m, k, x2d.stride(0), _ptr(xq), _ptr(sx), _ptr(xsum),
                                    _stream(x2d)))
    return (xq, sx, xsum) if want_sum else (xq, sx)


def silu_mul_quant(gate_up: Tensor, want_h: bool = False):
    """``silu(gate) * up`` of a fused gate/up output [M, 2F] (gate | up), quantized per row in the same kernel:
    (int8 [M, F], float32 scales [M], int32 row sums [M]) and, with ``want_h``, the unquantized product [M, F]."""
    _require_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2:
        raise RuntimeError("gate_up must be 2D [M, 2F]")
    if gate_up.stride(1) != 1:
        gate_up = gate_up.contiguous()
    m, f = gate_up.shape[0], gate_up.shape[1] // 2
    dev = gate_up.device
    hq = torch.empty((m, f), dtype=torch.int8, device=dev)
    sx = torch.empty((m,), dtype=torch.float32, device=dev)
    xsum = torch.empty((m,), dtype=torch.int32, device=dev)
    h = torch.empty((m, f), dtype=gate_up.dtype, device=dev) if want_h else None
    with torch.cuda.device(dev):
        _check(_lib.bt_silu_mul_quant(_ptr(gate_up), _dtype_code(gate_up, "gate_up"), m, f, gate_up.stride(0), _ptr(hq),
                                      _ptr(sx), _ptr(xsum), _ptr(h), _stream(gate_up)))
    return (hq, sx, xsum, h) if want_h else (hq, sx, xsum)


def add_rmsnorm_quant(x2d: Tensor, delta: Optional[Tensor], weight: Tensor, eps: float, want_y: bool = False):
    """``x2d += delta`` IN PLACE (``delta`` may be None), RMS-normalise with ``weight`` and quantize per row in one
    kernel: (int8 [M, D], float32 scales [M], int32 row sums [M]) and, with ``want_y``, the normalised rows."""
    _require_cuda(x2d, weight)
    if x2d.dim() != 2 or x2d.stride(1) != 1:
        raise RuntimeError("x2d must be 2D with contiguous rows (it is updated in place)")
    m, d = x2d.shape
    if delta is not None:
        if delta.shape != x2d.shape or delta.dtype != x2d.dtype:
            raise RuntimeError("delta must have the shape and dtype of x2d")
        if delta.stride(1) != 1:
            delta = delta.contiguous()
    w = weight.detach().to(x2d.dtype).contiguous()
    if w.shape != (d,):
        raise RuntimeError("weight must be [D]")
    dev = x2d.device
    yq = torch.empty((m, d), dtype=torch.int8, device=dev)
    sx = torch.empty((m,), dtype=torch.float32, device=dev)
    xsum = torch.empty((m,), dtype=torch.int32, device=dev)
    y = torch.empty((m, d), dtype=x2d.dtype, device=dev) if want_y else None
    with torch.cuda.device(dev):
        _check(_lib.bt_add_rmsnorm_quant(_ptr(x2d), _ptr(delta), _dtype_code(x2d, "x"), m, d, x2d.stride(0),
                                         0 if delta is None else delta.stride(0), _ptr(w), float(eps), _ptr(yq), _ptr(sx),
                                         _ptr(xsum), _ptr(y), _stream(x2d)))
    return (yq, sx, xsum, y) if want_y else (yq, sx, xsum)


def tiled_bytes(in_features: int, out_features: int) -> int:
    return int(_lib.bt_tiled_bytes(in_features, out_features))


def retile(packed_T: Tensor, in_features: int) -> Tensor:
    """Public packed buffer -> private tiled buffer (flat uint8)."""
    _require_cuda(packed_T)
    packed_T = packed_T.contiguous()
    n = packed_T.shape[1]
    out = torch.empty(tiled_bytes(in_features, n), dtype=torch.uint8, device=packed_T.device)
    with torch.cuda.device(packed_T.device):
        _check(_lib.bt_retile_packed(_ptr(packed_T), in_features, n, _ptr(out), _stream(packed_T)))
    return out


def untile(tiled: Tensor, in_features: int, out_features: int) -> Tensor:
    """Private tiled buffer -> public packed uint8 [ceil(K/4), N]."""
    _require_cuda(tiled)
    out = torch.empty(((in_features + 3) // 4, out_features), dtype=torch.uint8, device=tiled.device)
    with torch.cuda.device(tiled.device):
        _check(_lib.bt_untile_packed(_ptr(tiled), in_features, out_features, _ptr(out), _stream(tiled)))
    return out


def _int_linear(fn, xq: Tensor, sx: Tensor, w: Tensor, k: int, n: int, scale: Tensor, bias: Optional[Tensor],
                out_dtype: torch.dtype, want_acc: bool, out: Optional[Tensor] = None, flags: Optional[int] = None):
    m = xq.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device=xq.device) if out is None else out
    acc = torch.empty((m, n), dtype=torch.int32, device=xq.device) if want_acc else None
    extra = () if flags is None else (int(flags),)
    with torch.cuda.device(xq.device):
        _check(fn(_ptr(xq), _ptr(sx), m, k, _ptr(w), n, _ptr(scale), _ptr(bias), _ptr(y), _DT[out_dtype], y.stride(0),
                  _ptr(acc), *extra, _stream(xq)))
    return (y, acc) if want_acc else y


def gemv_packed_i8(xq, sx, packed_T, in_features, scale, bias=None, out_dtype=torch.float32, want_acc=False, out=None):
    """Decode-size integer linear on the public packed layout (M <= 16)."""
    return _int_linear(_lib.bt_gemv_packed_i8, xq, sx, packed_T, in_features, packed_T.shape[1], scale, bias,
                       out_dtype, want_acc, out)


def gemv_tiled_i8(xq, sx, tiled, in_features, out_features, scale, bias=None, out_dtype=torch.float32, want_acc=False,
                  out=None, fresh_weights: bool = False):
    """Decode-size integer linear on the tiled layout (M <= 16): the bandwidth-bound fast path.

    ``fresh_weights``: ``tiled`` / ``scale`` / ``bias`` were written by work enqueued just before this call on the
    same stream; the kernel is then launched fully stream-ordered instead of overlapping its predecessor."""
    return _int_linear(_lib.bt_gemv_tiled_i8, xq, sx, tiled, in_features, out_features, scale, bias, out_dtype,
                       want_acc, out, flags=LAUNCH_WEIGHTS_JUST_WRITTEN if fresh_weights else LAUNCH_DEFAULT)


def gemv_tiled(x2d: Tensor, tiled: Tensor, in_features: int, out_features: int, scale: Tensor,
               bias: Optional[Tensor] = None, out: Optional[Tensor] = None, want_debug: bool = False,
               fresh_weights: bool = False):
    """Decode-size linear from floating-point activations in one kernel (fused int8 quantizer).

    ``want_debug`` also returns the int8 activations, their scales and the int32 accumulators.
    ``fresh_weights``: see ``gemv_tiled_i8``.
    """
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    m = x2d.shape[0]
    y = torch.empty((m, out_features), dtype=x2d.dtype, device=x2d.device) if out is None else out
    xq = sx = acc = None
    if want_debug:
        xq = torch.empty((m, in_features), dtype=torch.int8, device=x2d.device)
        sx = torch.empty((m,), dtype=torch.float32, device=x2d.device)
        acc = torch.empty((m, out_features), dtype=torch.int32, device=x2d.device)
    with torch.cuda.device(x2d.device):
        _check(_lib.bt_gemv_tiled(_ptr(x2d), _dtype_code(x2d, "X"), m, in_features, x2d.stride(0), _ptr(tiled), out_features,
                                  _ptr(scale), _ptr(bias), _ptr(y), _DT[y.dtype], y.stride(0), _ptr(xq), _ptr(sx), _ptr(acc),
                                  LAUNCH_WEIGHTS_JUST_WRITTEN if fresh_weights else LAUNCH_DEFAULT, _stream(x2d)))
    return (y, xq, sx, acc) if want_debug else y


FLOAT_GEMV_MAX_K = 65536     # bt_gemv_tiled_float: digits reach -128, half the K of the int8 kernels


def gemv_tiled_float(x2d: Tensor, tiled: Tensor, in_features: int, out_features: int, scale: Tensor,
                     bias: Optional[Tensor] = None, out: Optional[Tensor] = None, fresh_weights: bool = False) -> Tensor:
    """Decode-size linear with floating-point activations (no activation quantization) on the tiled layout: the
    reference's float semantics computed exactly (four digit planes of a 32-bit fixed-point row through the integer
    pipeline).  M <= GEMV_MAX_M, K <= FLOAT_GEMV_MAX_K."""
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    m = x2d.shape[0]
    y = torch.empty((m, out_features), dtype=x2d.dtype, device=x2d.device) if out is None else out
    with torch.cuda.device(x2d.device):
        _check(_lib.bt_gemv_tiled_float(_ptr(x2d), _dtype_code(x2d, "X"), m, in_features, x2d.stride(0), _ptr(tiled),
                                        out_features, _ptr(scale), _ptr(bias), _ptr(y), _DT[y.dtype], y.stride(0),
                                        LAUNCH_WEIGHTS_JUST_WRITTEN if fresh_weights else LAUNCH_DEFAULT, _stream(x2d)))
    return y


FLOAT_GEMM_ROWS = 1024        # most activation rows per tensor-core call of the float path (4096 int8 rows)
FLOAT_GEMM_ACC_BYTES = 256 << 20   # and at most this much int32 accumulator scratch per call


def float_linear_tiled_ok(m: int, in_features: int, dtype: torch.dtype) -> bool:
    """Float mode runs on the tiled weights through the integer kernels (digit planes) when the shape allows:
    the decode kernel for small batches, the tensor-core GEMM above (K a multiple of 16); otherwise the general
    float kernel on the public layout."""
    if in_features > FLOAT_GEMV_MAX_K or dtype not in _DT:
        return False
    return m <= DECODE_MAX_M or in_features % 16 == 0


def float_linear_tiled(x2d: Tensor, tiled: Tensor, in_features: int, out_features: int, scale: Tensor,
                       bias: Optional[Tensor], fresh_weights: bool = False) -> Tensor:
    """Floating-point activations (no activation quantization) on the tiled weights, computed exactly by the
    integer kernels: ``gemv_tiled_float`` up to DECODE_MAX_M rows; above, digit planes -> tcgen05 GEMM -> combine,
    FLOAT_GEMM_ROWS activation rows at a time.  Call only when ``float_linear_tiled_ok``."""
    m = x2d.shape[0]
    if m <= DECODE_MAX_M:
        return gemv_tiled_float(x2d, tiled, in_features, out_features, scale, bias, fresh_weights=fresh_weights)
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    dev = x2d.device
    y = torch.empty((m, out_features), dtype=x2d.dtype, device=dev)
    rows = min(m, FLOAT_GEMM_ROWS, max(32, (FLOAT_GEMM_ACC_BYTES // (16 * out_features)) // 32 * 32))
    planes = torch.empty((4 * rows, in_features), dtype=torch.int8, device=dev)
    pw = torch.empty((rows,), dtype=torch.float32, device=dev)
    xsum = torch.empty((4 * rows,), dtype=torch.int32, device=dev)
    bad = torch.empty((rows,), dtype=torch.int32, device=dev)
    ones = torch.ones((4 * rows,), dtype=torch.float32, device=dev)
    acc = torch.empty((4 * rows, out_features), dtype=torch.int32, device=dev)
    scratch = torch.empty((4 * rows, out_features), dtype=torch.bfloat16, device=dev)     # the GEMM's own output, unused
    with torch.cuda.device(dev):
        st = _stream(x2d)
        for m0 in range(0, m, rows):
            r = min(rows, m - m0)
            xs = x2d[m0:m0 + r]
            _check(_lib.bt_float_planes_quant(_ptr(xs), _dtype_code(xs, "X"), r, in_features, xs.stride(0), _ptr(planes),
                                              _ptr(pw), _ptr(xsum), _ptr(bad), st))
            _check(_lib.bt_gemm_tiled_i8(_ptr(planes), _ptr(ones), _ptr(xsum), 4 * r, in_features, _ptr(tiled), out_features,
                                         _ptr(scale), None, _ptr(scratch), BT_BF16, out_features, _ptr(acc), st))
            ys = y[m0:m0 + r]
            _check(_lib.bt_float_planes_combine(_ptr(acc), r, out_features, _ptr(pw), _ptr(bad), _ptr(scale), _ptr(bias),
                                                _ptr(ys), _DT[y.dtype], ys.stride(0), st))
    return y


def new_amax_buffer(layers: int, rows: int, device) -> Tensor:
    """Zeroed row-maximum words for ``layers`` chained decode layers of ``rows`` rows each: ``buf[i]`` is what layer i
    publishes and layer i + 1 consumes.  Zero the whole buffer (``buf.zero_()``) before every pass over the chain."""
    return torch.zeros((layers, rows, AMAX_SLOTS), dtype=torch.int32, device=device)


def gemv_tiled_chained(x2d: Tensor, tiled: Tensor, in_features: int, out_features: int, scale: Tensor,
                       bias: Optional[Tensor] = None, out: Optional[Tensor] = None, amax_in: Optional[Tensor] = None,
                       amax_out: Optional[Tensor] = None, amax_cols: Optional[int] = None,
                       fresh_weights: bool = False) -> Tensor:
    """``gemv_tiled`` for layers that feed one another: publishes each output row's max |y| into ``amax_out``
    (int32 [M, AMAX_SLOTS], zero before the launch) over the leading ``amax_cols`` columns, and / or takes the
    activation rows' maxima from ``amax_in`` (what the producer of ``x2d`` published) instead of reducing them.
    Bit-identical to ``gemv_tiled``."""
    if x2d.stride(1) != 1:
        raise RuntimeError("gemv_tiled_chained: activation rows must be contiguous (the producer's layout)")
    m = x2d.shape[0]
    y = torch.empty((m, out_features), dtype=x2d.dtype, device=x2d.device) if out is None else out
    for name, buf in (("amax_in", amax_in), ("amax_out", amax_out)):
        if buf is not None and (buf.dtype != torch.int32 or tuple(buf.shape) != (m, AMAX_SLOTS) or not buf.is_contiguous()):
            raise RuntimeError(f"gemv_tiled_chained: {name} must be a contiguous int32 [{m}, {AMAX_SLOTS}] tensor")
    cols = out_features if amax_cols is None else int(amax_cols)
    with torch.cuda.device(x2d.device):
        _check(_lib.bt_gemv_tiled_chained(_ptr(x2d), _dtype_code(x2d, "X"), m, in_features, x2d.stride(0), _ptr(tiled),
                                          out_features, _ptr(scale), _ptr(bias), _ptr(y), _DT[y.dtype], y.stride(0),
                                          _ptr(amax_in), _ptr(amax_out), cols,
                                          LAUNCH_WEIGHTS_JUST_WRITTEN if fresh_weights else LAUNCH_DEFAULT, _stream(x2d)))
    return y


def gemm_tiled_i8(xq, sx, tiled, in_features, out_features, scale, bias=None, out_dtype=torch.float32, want_acc=False,
                  out=None, xsum=None):
    """Prefill-size integer linear on the tiled layout (tcgen05 tensor cores).

    ``xsum``: int32 row sums of ``xq`` as returned by ``act_quant_i8(..., want_sum=True)``;
    computed here with a torch reduction when not given (tests with hand-made ``xq``)."""
    if xsum is None:
        xsum = xq.sum(dim=1, dtype=torch.int32)
    m = xq.shape[0]
    y = torch.empty((m, out_features), dtype=out_dtype, device=xq.device) if out is None else out
    acc = torch.empty((m, out_features), dtype=torch.int32, device=xq.device) if want_acc else None
    with torch.cuda.device(xq.device):
        _check(_lib.bt_gemm_tiled_i8(_ptr(xq), _ptr(sx), _ptr(xsum), m, in_features, _ptr(tiled), out_features, _ptr(scale),
                                     _ptr(bias), _ptr(y), _DT[out_dtype], y.stride(0), _ptr(acc), _stream(xq)))
    return (y, acc) if want_acc else y


def int8_linear_tiled(x2d: Tensor, tiled: Tensor, in_features: int, out_features: int, scale: Tensor,
                      bias: Optional[Tensor], fresh_weights: bool = False) -> Tensor:
    """The integer path for any batch: one fused quantize+GEMV kernel for M <= DECODE_MAX_M
    (its dp4a arithmetic grows with M), activation quantizer + tcgen05 GEMM above (cost
    almost flat in M up to a full 128-row tile).

    K that is not a multiple of 16 cannot be described to the TMA engine; such ragged
    shapes go through the decode kernel in chunks of 16 rows.
    """
    m = x2d.shape[0]
    if m <= DECODE_MAX_M:
        return gemv_tiled(x2d, tiled, in_features, out_features, scale, bias, fresh_weights=fresh_weights)
    if in_features % 16 == 0:
        xq, sx, xsum = act_quant_i8(x2d, want_sum=True)
        return gemm_tiled_i8(xq, sx, tiled, in_features, out_features, scale, bias, x2d.dtype, xsum=xsum)
    y = torch.empty((m, out_features), dtype=x2d.dtype, device=x2d.device)
    for m0 in range(0, m, GEMV_MAX_M):
        m1 = min(m, m0 + GEMV_MAX_M)
        gemv_tiled(x2d[m0:m1], tiled, in_features, out_features, scale, bias, out=y[m0:m1], fresh_weights=fresh_weights)
    return y


# ---------------------------------------------------------------------------------------
# The four callables of the reference's extension module
# ---------------------------------------------------------------------------------------

def activation_mode() -> str:
    """``int8`` (default: per-token int8 activations, integer contraction) or ``float``
    (the reference's fp32-accumulate arithmetic), from ``BITTORCH_B200_ACT``."""
    mode = os.environ.get("BITTORCH_B200_ACT", "int8").lower()
    if mode not in ("int8", "float"):
        raise RuntimeError(f"BITTORCH_B200_ACT must be 'int8' or 'float', got {mode!r}")
    return mode


def dummy(input: Tensor) -> Tensor:
    """Clone of the input — replaces ``_C.dummy`` (csrc/core/dispatch.cpp:7-9).

    CUDA tensors are copied by the library (``bt_dummy``); a CPU tensor, which the
    reference's extension also accepts (tests/test_extension.py:43-58), is cloned by torch.
    """
    if not input.is_cuda:
        return input.clone()
    src = input.contiguous()
    out = torch.empty_like(src)
    with torch.cuda.device(src.device):
        _check(_lib.bt_dummy(_ptr(src), _ptr(out), src.numel() * src.element_size(), _stream(src)))
    return out


def _check_common(X: Tensor, W: Tensor, scale: Tensor, bias: Optional[Tensor], n: int) -> None:
    # Same order and messages as csrc/core/dispatch.cpp:58-79 / :112-133.
    if scale.dim() != 1:
        raise RuntimeError("scale must be 1D [N]")
    if scale.shape[0] != n:
        raise RuntimeError("scale size doesn't match N")
    if bias is not None and (bias.dim() != 1 or bias.shape[0] != n):
        raise RuntimeError("bias shape mismatch")
    if not (X.is_cuda and W.is_cuda and scale.is_cuda):
        raise RuntimeError("All tensors must be CUDA")


def ternary_linear_forward(X: Tensor, W_tern: Tensor, scale: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """Y = X @ (W_tern * scale).T + bias with int8 weights [N,K] and fp32 accumulation.

    Replaces ``_C.ternary_linear_forward`` (csrc/core/dispatch.cpp:52-87).
    """
    if X.dim() < 1:
        raise RuntimeError("X must have at least 1 dimension")
    if X.numel() == 0:
        raise RuntimeError("X is empty")
    if W_tern.dim() != 2:
        raise RuntimeError("W_tern must be 2D [N, K]")
    if W_tern.dtype != torch.int8:
        raise RuntimeError("W_tern must be int8")
    k = X.shape[-1]
    n, wk = W_tern.shape
    if k != wk:
        raise RuntimeError("input K doesn't match weight K")
    _check_common(X, W_tern, scale, bias, n)
    x2d = X.contiguous().reshape(-1, k)
    w = W_tern.contiguous()
    s32, b32 = _f32vec(scale), _f32vec(bias)
    y = torch.empty((x2d.shape[0], n), dtype=X.dtype, device=X.device)
    with torch.cuda.device(X.device):
        _check(_lib.bt_linear_unpacked(_ptr(x2d), _dtype_code(x2d, "X", float_path=True), x2d.shape[0], k, _ptr(w), n, _ptr(s32),
                                       _ptr(b32), _ptr(y), _stream(x2d)))
    return y.reshape(*X.shape[:-1], n)


def _packed_checks(X: Tensor, W_T: Tensor, scale: Tensor, bias: Optional[Tensor], in_features: int) -> Tuple[int, int]:
    if X.dim() < 1:
        raise RuntimeError("X must have at least 1 dimension")
    if X.numel() == 0:
        raise RuntimeError("X is empty")
    if W_T.dim() != 2:
        raise RuntimeError("W_T must be 2D [K_bytes, N]")
    if W_T.dtype != torch.uint8:
        raise RuntimeError("W_T must be uint8")
    k = X.shape[-1]
    k_bytes, n = W_T.shape
    if k != in_features:
        raise RuntimeError("input K doesn't match in_features")
    if k_bytes != (in_features + 3) // 4:
        raise RuntimeError("K_bytes doesn't match ceil(K/4)")
    _check_common(X, W_T, scale, bias, n)
    return k, n


def _packed_forward(X: Tensor, W_T: Tensor, scale: Tensor, bias: Optional[Tensor], k: int, n: int, mode: str) -> Tensor:
    x2d = X.contiguous().reshape(-1, k)
    w = W_T.contiguous()
    s32, b32 = _f32vec(scale), _f32vec(bias)
    m = x2d.shape[0]
    if mode == "float" or X.dtype == torch.float64:        # float64 exists on the float path only, as in the reference
        y = torch.empty((m, n), dtype=X.dtype, device=X.device)
        with torch.cuda.device(X.device):
            _check(_lib.bt_linear_packed_float(_ptr(x2d), _dtype_code(x2d, "X", float_path=True), m, k, _ptr(w), n, _ptr(s32), _ptr(b32),
                                               _ptr(y), _stream(x2d)))
    elif m <= DECODE_MAX_M:
        xq, sx = act_quant_i8(x2d)
        y = gemv_packed_i8(xq, sx, w, k, s32, b32, X.dtype)
    else:
        y = int8_linear_tiled(x2d, retile(w, k), k, n, s32, b32, fresh_weights=True)   # re-tiled just above
    return y.reshape(*X.shape[:-1], n)


def ternary_linear_packed_forward(X: Tensor, W_T: Tensor, scale: Tensor, bias: Optional[Tensor] = None,
                                  in_features: Optional[int] = None) -> Tensor:
    """Packed ternary linear on the public [ceil(K/4), N] buffer.

    Replaces ``_C.ternary_linear_packed_forward`` (csrc/core/dispatch.cpp:105-142).  Small
    batches run the decode kernel on the buffer as it is; larger ones re-tile it for the
    tensor-core kernel (modules cache that copy, this stateless call cannot).
    """
    if in_features is None:
        raise TypeError("ternary_linear_packed_forward() missing required argument: 'in_features'")
    k, n = _packed_checks(X, W_T, scale, bias, int(in_features))
    return _packed_forward(X, W_T, scale, bias, k, n, activation_mode())


def ternary_linear_tensor_core_forward(X: Tensor, W_T: Tensor, scale: Tensor, bias: Optional[Tensor] = None,
                                       in_features: Optional[int] = None, version: int = 1) -> Tensor:
    """Replaces ``_C.ternary_linear_tensor_core_forward``
    (csrc/kernels/ternary_gemm_tensor_core.cu:663-727): version 1 = float compute,
    version 2 = int8 activations on the tensor cores (per-row activation scales)."""
    if X.dim() != 2:
        raise RuntimeError("X must be 2D")
    if version not in (1, 2):
        raise RuntimeError("version must be 1 (V1 float) or 2 (V2 mma.sync)")
    if in_features is None:
        in_features = X.shape[-1]
    k, n = _packed_checks(X, W_T, scale, bias, int(in_features))
    if version == 1 and float_linear_tiled_ok(X.shape[0], k, X.dtype):
        # float compute on the tensor cores (digit planes); the stateless call re-tiles its weights every time
        tiled = retile(W_T.contiguous(), k)
        return float_linear_tiled(X.contiguous(), tiled, k, n, _f32vec(scale), _f32vec(bias), fresh_weights=True)
    return _packed_forward(X, W_T, scale, bias, k, n, "float" if version == 1 else "int8")
