"""ctypes/numpy front end of the C oracle (``bt_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Every function takes and returns numpy arrays.  Half-precision inputs are passed
widened to float32 together with a dtype tag saying how they were stored, so the
oracle can round intermediate results the way the reference's torch ops do.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor

import numpy as np

DT_F32, DT_F16, DT_BF16 = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libbt_oracle.so")
_lib = None
_lock = threading.Lock()

_i64 = ctypes.c_int64
_f32 = ctypes.c_float
_int = ctypes.c_int
_p = ctypes.c_void_p


def build(force: bool = False) -> str:
    """Compile ``bt_oracle.c`` with gcc (seconds).  Returns the library path."""
    src = os.path.join(_HERE, "bt_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libbt_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    with _lock:
        if _lib is None:
            build()
            lib = ctypes.CDLL(_LIB_PATH)
            lib.bto_ternarize.argtypes = [_p, _i64, _i64, _i64, _f32, _int, _p, _p]
            lib.bto_pack.argtypes = [_p, _i64, _i64, _p]
            lib.bto_pack_transposed.argtypes = [_p, _i64, _i64, _p]
            lib.bto_unpack.argtypes = [_p, _i64, _i64, _p]
            lib.bto_unpack_transposed.argtypes = [_p, _i64, _i64, _p]
            lib.bto_act_quant.argtypes = [_p, _i64, _i64, _i64, _p, _p]
            lib.bto_gemm_i32.argtypes = [_p, _i64, _i64, _p, _i64, _p]
            lib.bto_epilogue.argtypes = [_p, _i64, _i64, _p, _p, _p, _p]
            lib.bto_linear_float.argtypes = [_p, _i64, _i64, _p, _i64, _p, _p, _p]
            lib.bto_packed_forward_i8.argtypes = [_p, _p, _i64, _i64, _p, _i64, _i64, _i64, _p, _p, _p]
            lib.bto_silu_mul_quant.argtypes = [_p, _i64, _i64, _i64, _int, _p, _p, _p, _p]
            lib.bto_add_rmsnorm_quant.argtypes = [_p, _p, _i64, _i64, _i64, _i64, _p, _f32, _int, _p, _p, _p, _p]
            lib.bto_exp_plain.argtypes = [_f32]
            lib.bto_exp_plain.restype = _f32
            for name in (
                "bto_ternarize", "bto_pack", "bto_pack_transposed", "bto_unpack", "bto_unpack_transposed",
                "bto_act_quant", "bto_gemm_i32", "bto_epilogue", "bto_linear_float", "bto_packed_forward_i8",
                "bto_silu_mul_quant", "bto_add_rmsnorm_quant",
            ):
                getattr(lib, name).restype = None
            _lib = lib
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def ternarize(w, threshold_factor: float = 0.05, dtype: int = DT_F32):
    """(codes int8 [N,K] in {-1,0,1}, scale float32 [N]) — quant/ternary.py:100-150."""
    w = _c(w, np.float32)
    n, k = w.shape
    codes = np.empty((n, k), np.int8)
    scale = np.empty((n,), np.float32)
    _load().bto_ternarize(_ptr(w), n, k, k, np.float32(threshold_factor), dtype, _ptr(codes), _ptr(scale))
    return codes, scale


def pack(codes):
    """uint8 [N, ceil(K/4)] — quant/ternary_packed.py:22-75."""
    codes = _c(codes, np.int8)
    n, k = codes.shape
    out = np.empty((n, (k + 3) // 4), np.uint8)
    _load().bto_pack(_ptr(codes), n, k, _ptr(out))
    return out


def pack_transposed(codes):
    """uint8 [ceil(K/4), N] — quant/ternary_packed.py:174-206."""
    codes = _c(codes, np.int8)
    n, k = codes.shape
    out = np.empty(((k + 3) // 4, n), np.uint8)
    _load().bto_pack_transposed(_ptr(codes), n, k, _ptr(out))
    return out


def unpack(packed, k: int):
    """int8 [N,K] from uint8 [N, ceil(K/4)] — quant/ternary_packed.py:78-120."""
    packed = _c(packed, np.uint8)
    n = packed.shape[0]
    out = np.empty((n, k), np.int8)
    _load().bto_unpack(_ptr(packed), n, k, _ptr(out))
    return out


def unpack_transposed(packed_t, k: int):
    """int8 [N,K] from uint8 [ceil(K/4), N] — quant/ternary_packed.py:209-223."""
    packed_t = _c(packed_t, np.uint8)
    n = packed_t.shape[1]
    out = np.empty((n, k), np.int8)
    _load().bto_unpack_transposed(_ptr(packed_t), n, k, _ptr(out))
    return out


def act_quant(x):
    """(q int8 [M,K], sx float32 [M]) — per-row restatement of ternary_gemm_tensor_core.cu:343-347,431-441."""
    x = _c(x, np.float32)
    m, k = x.shape
    q = np.empty((m, k), np.int8)
    sx = np.empty((m,), np.float32)
    _load().bto_act_quant(_ptr(x), m, k, k, _ptr(q), _ptr(sx))
    return q, sx


def gemm_i32(q, codes):
    """int32 [M,N] accumulators: q [M,K] int8 times codes [N,K] in {-1,0,1}."""
    q = _c(q, np.int8)
    codes = _c(codes, np.int8)
    m, k = q.shape
    n = codes.shape[0]
    acc = np.empty((m, n), np.int32)
    _load().bto_gemm_i32(_ptr(q), m, k, _ptr(codes), n, _ptr(acc))
    return acc


def epilogue(acc, sx, scale, bias=None):
    """float32 [M,N]: (float(acc)*sx)*scale + bias — ternary_gemm_tensor_core.cu:648-652 with the 127 cancelled."""
    acc = _c(acc, np.int32)
    m, n = acc.shape
    sx = _c(sx, np.float32)
    scale = _c(scale, np.float32)
    bias = None if bias is None else _c(bias, np.float32)
    y = np.empty((m, n), np.float32)
    _load().bto_epilogue(_ptr(acc), m, n, _ptr(sx), _ptr(scale), _ptr(bias), _ptr(y))
    return y


def linear_float(x, codes, scale, bias=None):
    """float32 [M,N]: float-activation forward — ternary_gemm.cu:41-73 semantics."""
    x = _c(x, np.float32)
    codes = _c(codes, np.int8)
    m, k = x.shape
    n = codes.shape[0]
    scale = _c(scale, np.float32)
    bias = None if bias is None else _c(bias, np.float32)
    y = np.empty((m, n), np.float32)
    _load().bto_linear_float(_ptr(x), m, k, _ptr(codes), n, _ptr(scale), _ptr(bias), _ptr(y))
    return y


def packed_forward_i8(q, sx, packed_t, k: int, scale, bias=None, n0: int = 0, n1: int | None = None, out=None):
    """Integer path straight from packed bytes; fills y[:, n0:n1]."""
    q = _c(q, np.int8)
    sx = _c(sx, np.float32)
    packed_t = _c(packed_t, np.uint8)
    n = packed_t.shape[1]
    m = q.shape[0]
    scale = _c(scale, np.float32)
    bias = None if bias is None else _c(bias, np.float32)
    y = np.zeros((m, n), np.float32) if out is None else out
    n1 = n if n1 is None else n1
    _load().bto_packed_forward_i8(_ptr(q), _ptr(sx), m, k, _ptr(packed_t), n, n0, n1, _ptr(scale), _ptr(bias), _ptr(y))
    return y


def packed_forward_i8_threaded(x, packed_t, k: int, scale, bias=None, threads: int | None = None):
    """Activation quantizer + integer path over `threads` host threads (column ranges).

    ctypes releases the GIL during the C call, so the threads run in parallel.
    This is the timed CPU "port" baseline of the packed inference path.
    """
    threads = threads or os.cpu_count() or 1
    q, sx = act_quant(x)
    packed_t = _c(packed_t, np.uint8)
    n = packed_t.shape[1]
    y = np.zeros((q.shape[0], n), np.float32)
    bounds = np.linspace(0, n, threads + 1).astype(np.int64)
    with ThreadPoolExecutor(max_workers=threads) as ex:
        futs = [
            ex.submit(packed_forward_i8, q, sx, packed_t, k, scale, bias, int(bounds[i]), int(bounds[i + 1]), y)
            for i in range(threads)
            if bounds[i + 1] > bounds[i]
        ]
        for f in futs:
            f.result()
    return y


def silu_mul_quant(gate_up, dtype: int = DT_F32):
    """(int8 h [M,F], sx [M], row sums [M], h float32 [M,F]) of ``silu(gate) * up`` for gate_up [M, 2F] (values
    already representable in ``dtype``) - the definition the fused kernel is pinned to."""
    gu = _c(gate_up, np.float32)
    m, f2 = gu.shape
    f = f2 // 2
    hq, sx, xsum = np.empty((m, f), np.int8), np.empty(m, np.float32), np.empty(m, np.int32)
    h = np.empty((m, f), np.float32)
    _load().bto_silu_mul_quant(_ptr(gu), m, f, f2, dtype, _ptr(hq), _ptr(sx), _ptr(xsum), _ptr(h))
    return hq, sx, xsum, h


def add_rmsnorm_quant(x, delta, weight, eps: float, dtype: int = DT_F32):
    """(new x [M,D], int8 y, sx, row sums, y float32) of ``x += delta; y = x / rms(x) * weight`` followed by the
    per-row quantizer; ``delta`` may be None."""
    x = np.array(x, np.float32, copy=True, order="C")
    m, d = x.shape
    delta = None if delta is None else _c(delta, np.float32)
    w = _c(weight, np.float32)
    yq, sx, xsum = np.empty((m, d), np.int8), np.empty(m, np.float32), np.empty(m, np.int32)
    y = np.empty((m, d), np.float32)
    _load().bto_add_rmsnorm_quant(_ptr(x), _ptr(delta), m, d, d, d, _ptr(w), np.float32(eps), dtype, _ptr(yq), _ptr(sx),
                                  _ptr(xsum), _ptr(y))
    return x, yq, sx, xsum, y


def exp_plain(x: float) -> float:
    return float(_load().bto_exp_plain(np.float32(x)))


def ref_python_forward(x, weight, bias=None, threshold_factor: float = 0.05):
    """Eager-torch restatement of the reference's CPU "python backend" forward.

    Follows bittorch/nn/ternary_linear.py:196-213 and bittorch/quant/ternary.py:122-142,189: re-quantize the
    full-precision master weight on every call, apply the straight-through rewrite ``T.detach() - W.detach() + W``
    (two more passes over the weight, which the reference executes in inference too), build the effective weight
    ``w_q * scale`` in the input dtype and run a dense ``F.linear``.  Takes and returns torch CPU tensors; used as
    the timed CPU baseline next to the GPU numbers.
    """
    import torch
    import torch.nn.functional as F

    with torch.no_grad():
        absw = weight.abs()
        scale = absw.max(dim=1, keepdim=True).values.clamp(min=1e-8)
        thr = threshold_factor * scale
        t = torch.where(absw > thr, torch.sign(weight), torch.zeros_like(weight))
        w_q = t.detach() - weight.detach() + weight            # quant/ternary.py:189
        w_eff = (w_q * scale).to(x.dtype)
        b = None if bias is None else bias.to(x.dtype)
        return F.linear(x, w_eff, b)
