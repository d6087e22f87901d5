"""numpy front end of libbt_simt.so: the library's CUDA kernels compiled for the CPU, one OS thread per CUDA thread
(simt_host.h).  TEST INFRASTRUCTURE ONLY.  Same entry points and argument order as include/bittorch_b200.h, host
pointers instead of device pointers."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LIB = os.path.join(HERE, "libbt_simt.so")
CSRC = os.path.join(ROOT, "bittorch_b200", "csrc")
F32, F16, BF16, F64 = 0, 1, 2, 3

_p, _i64, _int, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
_lib = None


def cuda_include_dir() -> str:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "include", "cuda_runtime.h")):
            return os.path.join(cand, "include")
    raise RuntimeError("CUDA headers not found (cuda_runtime.h supplies the vector and half types)")


def build(force: bool = False) -> str:
    """Compiles libbt_simt.so (g++, about 20 s).  For a run under AddressSanitizer, which also catches reads and
    writes of the kernels outside the caller's buffers, add `-fsanitize=address -fno-omit-frame-pointer` to the
    command below, and start python with LD_PRELOAD=$(gcc -print-file-name=libasan.so) and
    ASAN_OPTIONS=detect_leaks=0:verify_asan_link_order=0 (the whole test file then takes about 6 minutes).
    The same with `-fsanitize=thread`, libtsan.so and TSAN_OPTIONS=halt_on_error=0:log_path=<file> is a race
    detector for the kernels' shared memory: CUDA threads are OS threads here and __syncthreads, named barriers,
    __syncwarp, shuffles and mbarriers are pthread / atomic operations ThreadSanitizer understands, so a shared-memory
    access pair with no barrier between them is reported (a kernel that reads a neighbour's word without
    __syncthreads is; the one report of a clean run is inside the framework's own OpenMP pool)."""
    sources = [os.path.join(HERE, f) for f in ("simt_lib.cpp", "simt_host.h")]
    sources += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    sources.append(os.path.join(ROOT, "include", "bittorch_b200.h"))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in sources):
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-g", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared",
                               "-pthread", "-Wno-attributes", "-I" + cuda_include_dir(), "-o", LIB,
                               os.path.join(HERE, "simt_lib.cpp")])
    return LIB


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.bt_last_error.restype = ctypes.c_char_p
        _lib.bt_tiled_bytes.restype = ctypes.c_size_t
        _lib.bt_tiled_bytes.argtypes = [_i64, _i64]
        sig = {
            "bt_quantize_pack": [_p, _int, _i64, _i64, _i64, _f32, _p, _p, _p, _p, _p],
            "bt_pack_codes": [_p, _i64, _i64, _p, _p], "bt_unpack_codes": [_p, _i64, _i64, _p, _p],
            "bt_pack_codes_rows": [_p, _i64, _i64, _p, _p], "bt_unpack_codes_rows": [_p, _i64, _i64, _p, _p],
            "bt_act_quant_i8": [_p, _int, _i64, _i64, _i64, _p, _p, _p, _p],
            "bt_retile_packed": [_p, _i64, _i64, _p, _p], "bt_untile_packed": [_p, _i64, _i64, _p, _p],
            "bt_gemv_tiled_i8": [_p, _p, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _p, _int, _p],
            "bt_gemv_tiled": [_p, _int, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _p, _p, _p, _int, _p],
            "bt_gemv_tiled_chained": [_p, _int, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _p, _p, _i64, _int, _p],
            "bt_gemv_tiled_float": [_p, _int, _i64, _i64, _i64, _p, _i64, _p, _p, _p, _int, _i64, _int, _p],
            "bt_linear_unpacked": [_p, _int, _i64, _i64, _p, _i64, _p, _p, _p, _p],
            "bt_linear_packed_float": [_p, _int, _i64, _i64, _p, _i64, _p, _p, _p, _p],
            "bt_float_planes_quant": [_p, _int, _i64, _i64, _i64, _p, _p, _p, _p, _p],
            "bt_float_planes_combine": [_p, _i64, _i64, _p, _p, _p, _p, _p, _int, _i64, _p],
            "bt_silu_mul_quant": [_p, _int, _i64, _i64, _i64, _p, _p, _p, _p, _p],
            "bt_add_rmsnorm_quant": [_p, _p, _int, _i64, _i64, _i64, _i64, _p, _f32, _p, _p, _p, _p, _p],
            "bt_device_status": [_p, _p], "simt_set_sm_count": [_int], "simt_take_errors": [ctypes.c_char_p, ctypes.c_size_t],
        }
        for name, argtypes in sig.items():
            getattr(_lib, name).argtypes = argtypes
    return _lib


def ptr(a):
    return None if a is None else a.ctypes.data_as(_p)


def check(rc: int) -> None:
    """Raises on a non-zero status, and on any rule of the emulated hardware that a kernel broke."""
    buf = ctypes.create_string_buffer(512)
    broken = lib().simt_take_errors(buf, 512)
    if rc != 0:
        raise RuntimeError(lib().bt_last_error().decode() or f"status {rc}")
    if broken:
        raise RuntimeError(f"emulated hardware rule broken: {buf.value.decode()}")


def device_status() -> int:
    out = ctypes.c_int(0)
    lib().bt_device_status(ctypes.byref(out), None)
    return out.value


def set_sm_count(n: int) -> None:
    lib().simt_set_sm_count(n)


def to_bits(x: np.ndarray, dtype: int) -> np.ndarray:
    """float32 array -> storage of `dtype` (uint16 for the half types), round to nearest even."""
    import torch

    t = torch.from_numpy(np.ascontiguousarray(x, np.float32))
    if dtype == BF16:
        return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    if dtype == F16:
        return t.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    if dtype == F64:
        return t.double().numpy()
    return t.numpy()


def from_bits(a: np.ndarray, dtype: int) -> np.ndarray:
    import torch

    if dtype == BF16:
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).float().numpy()
    if dtype == F16:
        return torch.from_numpy(a.view(np.int16)).view(torch.float16).float().numpy()
    return np.asarray(a, np.float32)


def empty_out(shape, dtype: int) -> np.ndarray:
    return np.empty(shape, {F32: np.float32, F64: np.float64}.get(dtype, np.uint16))


def retile(packed_t: np.ndarray, k: int) -> np.ndarray:
    n = packed_t.shape[1]
    # a 16-byte aligned buffer, as the bulk copy demands
    raw = np.empty(lib().bt_tiled_bytes(k, n) + 16, np.uint8)
    off = (-raw.ctypes.data) % 16
    tiled = raw[off:off + lib().bt_tiled_bytes(k, n)]
    check(lib().bt_retile_packed(ptr(np.ascontiguousarray(packed_t)), k, n, ptr(tiled), None))
    return tiled


def planes_reference(x32, codes, scale, bias):
    """bt_gemv_tiled_float's definition with numpy: 32-bit fixed point from the row maximum's power of two, exact
    integer contraction, one rounding to float, exact power of two, scale, bias (float32 operations, unfused)."""
    m = x32.shape[0]
    y = np.empty((m, codes.shape[0]), np.float32)
    for r in range(m):
        row = x32[r]
        if not np.isfinite(row).all():
            y[r] = np.nan
            continue
        amax = np.float32(np.abs(row).max())
        e = int(np.frexp(amax)[1])
        e = max(-96, min(127, e))
        v = np.rint(row * np.float32(2.0 ** (30 - e))).astype(np.int64)
        v = np.clip(v, -(1 << 30), 1 << 30)
        total = codes.astype(np.int64) @ v
        out = total.astype(np.float32) * np.float32(2.0 ** (e - 30))
        out = out * scale
        y[r] = out + bias if bias is not None else out
    return y
