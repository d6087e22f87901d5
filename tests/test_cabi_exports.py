"""CPU checks of the drop-in boundary: the library loads, exports every symbol the header
declares, and the Python shim rejects bad calls with the reference's messages."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "bittorch_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bt_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from bittorch_b200 import _build

    path = _build.build()
    lib = ctypes.CDLL(path)
    names = _declared_symbols()
    assert len(names) >= 16
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    lib.bt_version.restype = ctypes.c_int
    assert lib.bt_version() >= 100
    lib.bt_tiled_bytes.restype = ctypes.c_size_t
    lib.bt_tiled_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64]
    assert lib.bt_tiled_bytes(4096, 4096) == 4096 * 4096 // 4          # still 2 bits per weight
    assert lib.bt_tiled_bytes(33, 65) == 5 * 1 * 512                    # padded to 16 x 128 tiles
    assert lib.bt_tiled_bytes(0, 5) == 0


def test_shim_binds_every_declared_symbol():
    from bittorch_b200 import _C

    assert sorted(_C.EXPORTED) == _declared_symbols()


def test_argument_errors_come_back_as_codes_not_crashes():
    from bittorch_b200 import _build

    lib = ctypes.CDLL(_build.build())
    lib.bt_last_error.restype = ctypes.c_char_p
    i64, p = ctypes.c_int64, ctypes.c_void_p
    lib.bt_act_quant_i8.argtypes = [p, ctypes.c_int, i64, i64, i64, p, p, p, p]
    assert lib.bt_act_quant_i8(None, 0, 1, 1, 1, None, None, None, None) == 1          # BT_ERR_INVALID
    assert b"NULL" in lib.bt_last_error()
    lib.bt_quantize_pack.argtypes = [p, ctypes.c_int, i64, i64, i64, ctypes.c_float, p, p, p, p, p]
    assert lib.bt_quantize_pack(p(16), 7, 4, 4, 4, 0.05, None, p(16), None, None, None) == 1
    assert b"dtype" in lib.bt_last_error()
    assert lib.bt_quantize_pack(p(16), 0, 4, 8, 4, 0.05, None, p(16), None, None, None) == 1
    assert b"stride" in lib.bt_last_error()
    lib.bt_gemv_tiled_i8.argtypes = [p, p, i64, i64, p, i64, p, p, p, ctypes.c_int, i64, p, ctypes.c_int, p]
    assert lib.bt_gemv_tiled_i8(p(16), p(16), 17, 64, p(16), 64, p(16), None, p(16), 0, 64, None, 0, None) == 3  # unsupported M
    assert b"exceeds" in lib.bt_last_error()
    assert lib.bt_gemv_tiled_i8(p(16), p(16), 0, 64, p(16), 64, p(16), None, p(16), 0, 64, None, 0, None) == 1
    assert b"empty" in lib.bt_last_error()
    assert lib.bt_gemv_tiled_i8(p(16), p(16), 1, 64, p(16), 64, p(16), None, p(16), 0, 64, None, 6, None) == 1
    assert b"flags" in lib.bt_last_error()
    lib.bt_set_tuning.argtypes = [ctypes.c_int, ctypes.c_int]
    assert lib.bt_set_tuning(99, 1) == 1 and b"knob" in lib.bt_last_error()
    assert lib.bt_set_tuning(1, 128) == 0 and lib.bt_set_tuning(1, -1) == 0
    lib.bt_gemm_tiled_i8.argtypes = [p, p, p, i64, i64, p, i64, p, p, p, ctypes.c_int, i64, p, p]
    assert lib.bt_gemm_tiled_i8(p(16), p(16), p(16), 32, 40, p(16), 64, p(16), None, p(16), 0, 64, None, None) == 3
    assert b"multiple of 16" in lib.bt_last_error()


def test_reference_error_messages_on_cpu_tensors():
    """csrc/core/dispatch.cpp:58-79 / :112-133 — same strings, raised as RuntimeError."""
    from bittorch_b200 import _C

    x = torch.randn(2, 8)
    w = torch.zeros(4, 8, dtype=torch.int8)
    s = torch.ones(4)
    with pytest.raises(RuntimeError, match="All tensors must be CUDA"):
        _C.ternary_linear_forward(x, w, s)
    with pytest.raises(RuntimeError, match="W_tern must be int8"):
        _C.ternary_linear_forward(x, w.float(), s)
    with pytest.raises(RuntimeError, match="input K doesn't match weight K"):
        _C.ternary_linear_forward(torch.randn(2, 7), w, s)
    with pytest.raises(RuntimeError, match="X is empty"):
        _C.ternary_linear_forward(torch.randn(0, 8), w, s)
    with pytest.raises(RuntimeError, match="scale size doesn't match N"):
        _C.ternary_linear_forward(x, w, torch.ones(3))
    with pytest.raises(RuntimeError, match="bias shape mismatch"):
        _C.ternary_linear_forward(x, w, s, torch.ones(5))
    wp = torch.zeros(2, 4, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="K_bytes doesn't match"):
        _C.ternary_linear_packed_forward(x, torch.zeros(3, 4, dtype=torch.uint8), s, None, 8)
    with pytest.raises(RuntimeError, match="input K doesn't match in_features"):
        _C.ternary_linear_packed_forward(x, wp, s, None, 7)
    with pytest.raises(RuntimeError, match="W_T must be uint8"):
        _C.ternary_linear_packed_forward(x, wp.float(), s, None, 8)
    with pytest.raises(RuntimeError, match="All tensors must be CUDA"):
        _C.ternary_linear_packed_forward(x, wp, s, None, 8)
    with pytest.raises(RuntimeError, match="version must be 1"):
        _C.ternary_linear_tensor_core_forward(x, wp, s, None, 8, 3)
    assert torch.equal(_C.dummy(x), x)


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    """No silent fallback: with the library absent, importing the binding raises."""
    import importlib
    import sys

    monkeypatch.setenv("BITTORCH_B200_LIB", str(tmp_path / "nope.so"))
    import bittorch_b200

    saved = sys.modules.pop("bittorch_b200._C", None)
    saved_attr = bittorch_b200.__dict__.pop("_C", None)
    try:
        with pytest.raises(ImportError, match="has not been built"):
            importlib.import_module("bittorch_b200._C")
        from bittorch_b200._ext import require_ext
        with pytest.raises(RuntimeError, match="requires its CUDA extension"):
            require_ext()
    finally:
        sys.modules.pop("bittorch_b200._C", None)
        if saved is not None:
            sys.modules["bittorch_b200._C"] = saved
        if saved_attr is not None:
            bittorch_b200._C = saved_attr


def test_binding_stub_shown_to_reference_maintainers_matches_the_abi():
    """The ctypes stub in INTEGRATION.md is what a maintainer of the reference would paste: it must parse, and
    every argtypes list in it must have the arity of the real binding."""
    import ast
    import textwrap

    from bittorch_b200 import _C

    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    assert len(blocks) >= 2
    for block in blocks:
        ast.parse(textwrap.dedent(block))
    stub = max(blocks, key=len)
    bound = re.findall(r"_lib\.(bt_[a-z0-9_]+)\.argtypes = \[(.*?)\]", stub)
    assert len(bound) >= 6
    for name, args in bound:
        arity = len([a for a in args.split(",") if a.strip()])
        assert arity == len(_C._SIGNATURES[name][0]), name
