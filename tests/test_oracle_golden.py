"""Pins the CPU oracle against vectors produced by the reference itself.

The golden files were written by tests/golden/make_golden.py, which imports the
reference package and runs its own functions; every comparison of integer data
(ternary codes, packed bytes) and of fp32 scales is bit-exact.
"""

import numpy as np
import pytest

from conftest import golden_cases, load_golden


def _same_bits(a, b):
    a = np.ascontiguousarray(a, np.float32).view(np.uint32)
    b = np.ascontiguousarray(b, np.float32).view(np.uint32)
    nan_a = np.isnan(a.view(np.float32))
    nan_b = np.isnan(b.view(np.float32))
    return np.array_equal(nan_a, nan_b) and np.array_equal(a[~nan_a], b[~nan_b])


def _check_quant_case(oracle, c, dtype=0):
    tf = float(c["tf"]) if "tf" in c else 0.05
    codes, scale = oracle.ternarize(c["w"], tf, dtype)
    assert np.array_equal(codes, c["codes"])
    assert _same_bits(scale, c["scale"])
    if "packed" in c:
        assert np.array_equal(oracle.pack(codes), c["packed"])
        assert np.array_equal(oracle.unpack(c["packed"], codes.shape[1]), c["codes"])
    assert np.array_equal(oracle.pack_transposed(codes), c["packed_T"])
    assert np.array_equal(oracle.unpack_transposed(c["packed_T"], codes.shape[1]), c["codes"])


def test_known_answers(oracle):
    cases = golden_cases(load_golden("kat_quant_pack"))
    assert len(cases) >= 12
    for name, c in cases.items():
        _check_quant_case(oracle, c)
    # spot values the reference's tests assert literally
    assert cases["single"]["scale"][0] == 2.5 and cases["single"]["codes"][0, 0] == 1
    assert np.all(cases["all_pos"]["packed"] == 85) and np.all(cases["all_neg"]["packed"] == 170)
    assert list(cases["docstring"]["packed"].ravel()) == [0x49, 148]
    assert np.all(cases["thr_one"]["codes"] == 0)
    assert np.allclose(cases["rows"]["scale"], [4.0, 0.4, 40.0])


def test_config1_codes_scale_bytes(oracle):
    c = load_golden("c1_linear_512x256")
    _check_quant_case(oracle, c)
    zeros = float((c["codes"] == 0).mean())
    assert 0.03 < zeros < 0.07


def test_config1_float_forward(oracle):
    c = load_golden("c1_linear_512x256")
    y = oracle.linear_float(c["x"], c["codes"], c["scale"], c["bias"])
    assert np.allclose(y, c["y"], rtol=1e-4, atol=1e-4)
    assert np.allclose(y, c["y_infer"], rtol=1e-4, atol=1e-4)


def test_ragged_shapes(oracle):
    d = load_golden("ragged_forward")
    cases = golden_cases(d)
    assert len(cases) == len(d["shapes"])
    for name, c in cases.items():
        _check_quant_case(oracle, c)
        y = oracle.linear_float(c["x"], c["codes"], c["scale"], c["bias"])
        assert np.allclose(y, c["y"], rtol=1e-4, atol=1e-4), name


@pytest.mark.parametrize("tag,dtype", [("f16", 1), ("bf16", 2)])
def test_half_precision_masters(oracle, tag, dtype):
    cases = {k: v for k, v in golden_cases(load_golden("half_quant")).items() if k.startswith(tag + "_")}
    assert len(cases) == 3
    for name, c in cases.items():
        _check_quant_case(oracle, c, dtype)


def test_pack_roundtrips_and_reserved_code(oracle):
    cases = golden_cases(load_golden("pack_roundtrip"))
    for seed in (0, 42, 123, 999):
        c = cases[f"s{seed}"]
        assert np.array_equal(oracle.pack(c["codes"]), c["packed"])
        assert np.array_equal(oracle.pack_transposed(c["codes"]), c["packed_T"])
        assert np.array_equal(oracle.unpack_transposed(c["packed_T"], 128), c["codes"])
    ab = cases["all_bytes"]
    assert np.array_equal(oracle.unpack(ab["packed"], 1024), ab["codes"])


def test_packed_inference_float(oracle):
    c = load_golden("packed_infer_96x200")
    codes = oracle.unpack_transposed(c["packed_T"], 200)
    assert np.array_equal(codes, c["codes"])
    y = oracle.linear_float(c["x"], codes, c["scale"], c["bias"])
    assert np.allclose(y, c["y_f32"], rtol=1e-4, atol=1e-4)


def test_integer_path_is_self_consistent(oracle):
    """Integer path (parity unpinned by the reference): internal identities only."""
    c = load_golden("c1_linear_512x256")
    q, sx = oracle.act_quant(c["x"])
    assert q.min() >= -127 and q.max() <= 127
    assert np.all(np.abs(q).max(axis=1) == 127)
    assert _same_bits(sx, np.abs(c["x"]).max(axis=1) / np.float32(127.0))
    acc = oracle.gemm_i32(q, c["codes"])
    assert np.array_equal(acc, q.astype(np.int64) @ c["codes"].astype(np.int64).T)
    y = oracle.epilogue(acc, sx, c["scale"], c["bias"])
    y2 = oracle.packed_forward_i8(q, sx, c["packed_T"], 512, c["scale"], c["bias"])
    assert np.array_equal(y, y2)
    y3 = oracle.packed_forward_i8_threaded(c["x"], c["packed_T"], 512, c["scale"], c["bias"], threads=3)
    assert np.array_equal(y, y3)
    # int8 activations deviate from the float path by about 1e-2 of the output norm
    rel = np.linalg.norm(y - c["y"]) / np.linalg.norm(c["y"])
    assert rel < 3e-2


def test_act_quant_rounding_half_away_and_small_rows(oracle):
    x = np.zeros((3, 4), np.float32)
    x[0] = [127.0, 0.5, -0.5, 1.5]          # s = 1 -> q = 127, 1, -1, 2 (half away from zero)
    x[1] = [1e-7, -1e-7, 0, 0]              # max <= 1e-6 -> s = 1, q = 0
    x[2] = [2.0, -2.0, 1.0, 0.0078125]
    q, sx = oracle.act_quant(x)
    assert list(q[0]) == [127, 1, -1, 2] and sx[0] == 1.0
    assert list(q[1]) == [0, 0, 0, 0] and sx[1] == 1.0
    assert list(q[2][:3]) == [127, -127, 64] and sx[2] == np.float32(2.0) / np.float32(127.0)
