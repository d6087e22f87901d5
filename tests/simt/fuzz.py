"""Random shapes, strides, dtypes and emulated SM counts through the kernels that run on CPU threads, each case
compared bit for bit with the oracle (or, for the digit-plane path, with its definition).  TEST INFRASTRUCTURE ONLY.

    python -m tests.simt.fuzz [seed] [seconds]

Families: the decode kernel in its four modes (int8 rows, fused quantizer, published row maxima, float digit planes),
ternarize + pack, the packers and re-tiling, the activation quantizer, SiLU*up + quantizer, residual add + RMSNorm +
quantizer, digit planes around an exact integer contraction.  Prints one line per failing case and a summary line;
exit status 1 if any case failed."""

import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import numpy as np

import oracle
from tests.simt import harness as H

FLOAT_DTYPES = [H.F32, H.BF16, H.F16]


def bits_equal(a: np.ndarray, b: np.ndarray) -> bool:
    return np.array_equal(a.view(np.uint32), b.view(np.uint32))


def random_k(rng) -> int:
    return int(rng.choice([rng.integers(1, 64), rng.integers(64, 1200), rng.integers(1200, 9000)]))


def random_rows(rng, m: int, k: int, ld: int, dtype: int):
    """Activation rows with a stride, as stored bits and as the float32 values those bits hold."""
    x = rng.standard_normal((m, ld)).astype(np.float32) * np.float32(10.0 ** rng.integers(-2, 2))
    xb = H.to_bits(x, dtype)
    return xb, H.from_bits(np.ascontiguousarray(xb[:, :k]), dtype)


def decode_case(L, rng):
    m, k, n = int(rng.integers(1, 17)), random_k(rng), int(rng.integers(1, 140))
    sms, dtype, mode = int(rng.integers(1, 9)), int(rng.choice(FLOAT_DTYPES)), int(rng.integers(0, 4))
    ld = k + int(rng.choice([0, 4, 8, 3]))
    with_bias = bool(rng.random() < 0.5)
    case = dict(kernel="decode", mode=mode, m=m, k=k, n=n, sms=sms, dtype=dtype, ld=ld, bias=with_bias)
    H.set_sm_count(sms)
    codes = rng.integers(-1, 2, (n, k)).astype(np.int8)
    scale = (rng.random(n) * 0.5 + 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32) if with_bias else None
    tiled = H.retile(oracle.pack_transposed(codes), k)
    xb, x32 = random_rows(rng, m, k, ld, dtype)
    y = H.empty_out((m, n), dtype)
    q, sx = oracle.act_quant(x32)
    acc_ref = oracle.gemm_i32(q, codes)
    y_ref = H.to_bits(oracle.epilogue(acc_ref, sx, scale, bias), dtype)
    if mode == 0:
        acc = np.empty((m, n), np.int32)
        H.check(L.bt_gemv_tiled_i8(H.ptr(q), H.ptr(sx), m, k, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y), dtype, n,
                                   H.ptr(acc), 0, None))
        ok = np.array_equal(acc, acc_ref) and np.array_equal(y, y_ref)
    elif mode == 1:
        H.check(L.bt_gemv_tiled(H.ptr(xb), dtype, m, k, ld, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y), dtype, n,
                                None, None, None, 0, None))
        ok = np.array_equal(y, y_ref)
    elif mode == 2:
        amax_in = np.zeros((m, 8), np.uint32)                       # the row maximum sits in a random slot
        amax_in[np.arange(m), rng.integers(0, 8, m)] = np.abs(x32).max(axis=1).astype(np.float32).view(np.uint32)
        amax_out = np.zeros((m, 8), np.uint32)
        cols = int(rng.integers(1, n + 1))
        case["cols"] = cols
        H.check(L.bt_gemv_tiled_chained(H.ptr(xb), dtype, m, k, ld, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y),
                                        dtype, n, H.ptr(amax_in), H.ptr(amax_out), cols, 0, None))
        want = np.abs(H.from_bits(np.ascontiguousarray(y_ref[:, :cols]), dtype)).max(axis=1).astype(np.float32)
        ok = np.array_equal(y, y_ref) and bits_equal(amax_out.max(axis=1).view(np.float32), want)
    else:
        H.check(L.bt_gemv_tiled_float(H.ptr(xb), dtype, m, k, ld, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y),
                                      dtype, n, 0, None))
        ok = np.array_equal(y, H.to_bits(H.planes_reference(x32, codes, scale, bias), dtype))
    return case, ok


def quantize_pack_case(L, rng):
    n, k, dtype = int(rng.integers(1, 70)), int(rng.integers(1, 700)), int(rng.choice(FLOAT_DTYPES))
    case = dict(kernel="quantize_pack", n=n, k=k, dtype=dtype)
    w = rng.standard_normal((n, k)).astype(np.float32) * np.float32(10.0 ** rng.integers(-3, 2))
    w[rng.integers(0, n), :] = 0.0                                  # an all-zero channel: the 1e-8 floor
    wb = H.to_bits(w, dtype)
    packed = np.empty(((k + 3) // 4, n), np.uint8)
    scale, codes, tern = np.empty(n, np.float32), np.empty((n, k), np.int8), H.empty_out((n, k), dtype)
    H.check(L.bt_quantize_pack(H.ptr(wb), dtype, n, k, k, 0.05, H.ptr(packed), H.ptr(scale), H.ptr(codes), H.ptr(tern), None))
    codes_ref, scale_ref = oracle.ternarize(H.from_bits(wb, dtype), 0.05, dtype)
    ok = (np.array_equal(codes, codes_ref) and bits_equal(scale, scale_ref)
          and np.array_equal(packed, oracle.pack_transposed(codes_ref))
          and np.array_equal(H.from_bits(tern, dtype), codes_ref.astype(np.float32)))
    return case, ok


def packers_case(L, rng):
    n, k = int(rng.integers(1, 90)), int(rng.integers(1, 900))
    case = dict(kernel="packers", n=n, k=k)
    codes = rng.integers(-1, 2, (n, k)).astype(np.int8)
    kb = (k + 3) // 4
    packed_t, packed_r = np.empty((kb, n), np.uint8), np.empty((n, kb), np.uint8)
    H.check(L.bt_pack_codes(H.ptr(codes), n, k, H.ptr(packed_t), None))
    H.check(L.bt_pack_codes_rows(H.ptr(codes), n, k, H.ptr(packed_r), None))
    back_t, back_r = np.empty_like(codes), np.empty_like(codes)
    H.check(L.bt_unpack_codes(H.ptr(packed_t), n, k, H.ptr(back_t), None))
    H.check(L.bt_unpack_codes_rows(H.ptr(packed_r), n, k, H.ptr(back_r), None))
    again = np.empty_like(packed_t)
    H.check(L.bt_untile_packed(H.ptr(H.retile(packed_t, k)), k, n, H.ptr(again), None))
    ok = (np.array_equal(packed_t, oracle.pack_transposed(codes)) and np.array_equal(packed_r, oracle.pack(codes))
          and np.array_equal(back_t, codes) and np.array_equal(back_r, codes) and np.array_equal(again, packed_t))
    return case, ok


def act_quant_case(L, rng):
    m, k, dtype = int(rng.integers(1, 6)), random_k(rng), int(rng.choice(FLOAT_DTYPES))
    ld = k + int(rng.choice([0, 4, 8, 3]))
    case = dict(kernel="act_quant", m=m, k=k, ld=ld, dtype=dtype)
    xb, x32 = random_rows(rng, m, k, ld, dtype)
    xq, sx, xsum = np.empty((m, k), np.int8), np.empty(m, np.float32), np.empty(m, np.int32)
    H.check(L.bt_act_quant_i8(H.ptr(xb), dtype, m, k, ld, H.ptr(xq), H.ptr(sx), H.ptr(xsum), None))
    q_ref, sx_ref = oracle.act_quant(x32)
    ok = np.array_equal(xq, q_ref) and bits_equal(sx, sx_ref) and np.array_equal(xsum, q_ref.astype(np.int32).sum(axis=1))
    return case, ok


def silu_mul_case(L, rng):
    m, f, dtype = int(rng.integers(1, 5)), int(rng.choice([rng.integers(1, 40), rng.integers(40, 5000)])), int(rng.choice(FLOAT_DTYPES))
    ld = 2 * f + int(rng.choice([0, 8, 3]))
    case = dict(kernel="silu_mul_quant", m=m, f=f, ld=ld, dtype=dtype)
    gu = rng.standard_normal((m, ld)).astype(np.float32) * np.float32(rng.choice([0.1, 1.0, 4.0, 30.0]))
    gub = H.to_bits(gu, dtype)
    hq, sx, xsum = np.empty((m, f), np.int8), np.empty(m, np.float32), np.empty(m, np.int32)
    h = H.empty_out((m, f), dtype)
    H.check(L.bt_silu_mul_quant(H.ptr(gub), dtype, m, f, ld, H.ptr(hq), H.ptr(sx), H.ptr(xsum), H.ptr(h), None))
    q_ref, sx_ref, sum_ref, h_ref = oracle.silu_mul_quant(H.from_bits(gub, dtype)[:, : 2 * f], dtype)
    ok = (np.array_equal(h, H.to_bits(h_ref, dtype)) and np.array_equal(hq, q_ref) and bits_equal(sx, sx_ref)
          and np.array_equal(xsum, sum_ref))
    return case, ok


def add_rmsnorm_case(L, rng):
    m, d, dtype = int(rng.integers(1, 5)), int(rng.choice([rng.integers(1, 40), rng.integers(40, 5000)])), int(rng.choice(FLOAT_DTYPES))
    with_delta = bool(rng.random() < 0.7)
    case = dict(kernel="add_rmsnorm_quant", m=m, d=d, dtype=dtype, delta=with_delta)
    x = H.to_bits(rng.standard_normal((m, d)).astype(np.float32) * np.float32(rng.choice([0.05, 2.0, 50.0])), dtype)
    delta = H.to_bits(rng.standard_normal((m, d)).astype(np.float32), dtype) if with_delta else None
    w = H.to_bits(rng.standard_normal((1, d)).astype(np.float32) * 0.5 + 1.0, dtype)
    x_before = H.from_bits(x.copy(), dtype)
    yq, sx, xsum = np.empty((m, d), np.int8), np.empty(m, np.float32), np.empty(m, np.int32)
    y = H.empty_out((m, d), dtype)
    H.check(L.bt_add_rmsnorm_quant(H.ptr(x), H.ptr(delta), dtype, m, d, d, d, H.ptr(w), 1e-5, H.ptr(yq), H.ptr(sx),
                                   H.ptr(xsum), H.ptr(y), None))
    x_ref, q_ref, sx_ref, sum_ref, y_ref = oracle.add_rmsnorm_quant(
        x_before, None if delta is None else H.from_bits(delta, dtype), H.from_bits(w, dtype)[0], 1e-5, dtype)
    ok = (np.array_equal(x, H.to_bits(x_ref, dtype)) and np.array_equal(y, H.to_bits(y_ref, dtype))
          and np.array_equal(yq, q_ref) and bits_equal(sx, sx_ref) and np.array_equal(xsum, sum_ref))
    return case, ok


def float_planes_case(L, rng):
    m, k, n, dtype = int(rng.integers(1, 6)), int(rng.integers(1, 2500)), int(rng.integers(1, 60)), int(rng.choice(FLOAT_DTYPES))
    ld = k + int(rng.choice([0, 4, 3]))
    case = dict(kernel="float_planes", m=m, k=k, n=n, ld=ld, dtype=dtype)
    codes = rng.integers(-1, 2, (n, k)).astype(np.int8)
    scale = (rng.random(n) * 0.5 + 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    xb, x32 = random_rows(rng, m, k, ld, dtype)
    planes = np.empty((4 * m, k), np.int8)
    pw, xsum, bad = np.empty(m, np.float32), np.empty(4 * m, np.int32), np.empty(m, np.int32)
    H.check(L.bt_float_planes_quant(H.ptr(xb), dtype, m, k, ld, H.ptr(planes), H.ptr(pw), H.ptr(xsum), H.ptr(bad), None))
    acc = (planes.astype(np.int64) @ codes.astype(np.int64).T).astype(np.int32)       # stands in for the tensor cores
    y = H.empty_out((m, n), dtype)
    H.check(L.bt_float_planes_combine(H.ptr(acc), m, n, H.ptr(pw), H.ptr(bad), H.ptr(scale), H.ptr(bias), H.ptr(y), dtype, n, None))
    ok = (np.array_equal(xsum, planes.astype(np.int32).sum(axis=1)) and not bad.any()
          and np.array_equal(y, H.to_bits(H.planes_reference(x32, codes, scale, bias), dtype)))
    return case, ok


# the decode kernel is the one with a barrier protocol: it gets most of the draws
FAMILIES = [(decode_case, 0.55), (quantize_pack_case, 0.08), (packers_case, 0.07), (act_quant_case, 0.08),
            (silu_mul_case, 0.08), (add_rmsnorm_case, 0.07), (float_planes_case, 0.07)]


def main(seed: int, budget_s: float) -> int:
    L = H.lib()
    rng = np.random.default_rng(seed)
    weights = np.array([w for _, w in FAMILIES])
    t0, counts, fails = time.time(), {}, 0
    while time.time() - t0 < budget_s:
        family = FAMILIES[int(rng.choice(len(FAMILIES), p=weights / weights.sum()))][0]
        case = {"kernel": family.__name__}
        try:
            case, ok = family(L, rng)
            ok = ok and H.device_status() == 0
        except Exception as e:                                       # a refused launch is a failure of the case too
            ok, case["exception"] = False, str(e)[:200]
        counts[case["kernel"]] = counts.get(case["kernel"], 0) + 1
        if not ok:
            fails += 1
            print("FAIL", json.dumps(case), flush=True)
    print(json.dumps({"seed": seed, "cases": counts, "fails": fails, "seconds": round(time.time() - t0, 1)}))
    return 1 if fails else 0


if __name__ == "__main__":
    sys.exit(main(int(sys.argv[1]) if len(sys.argv) > 1 else 0, float(sys.argv[2]) if len(sys.argv) > 2 else 600.0))
