"""The library's own kernel sources, executed on the CPU with one OS thread per CUDA thread (tests/simt/), against
the oracle.  The kernels are the files under bittorch_b200/csrc compiled by g++ with the device primitives
(thread indices, barriers, warp shuffles, mbarriers with byte counts, the bulk copy, atomics, arithmetic intrinsics)
supplied by tests/simt/simt_host.h, so what runs here is the shipped index arithmetic, the shipped barrier protocol
and the shipped integer / float arithmetic - with real concurrency inside a CTA - not a restatement of them.
Covered: ternarize + pack, the packers, the activation quantizer, re-tiling, the decode kernel in all its modes (int8
rows, fused quantizer, published row maxima, floating-point digit planes) and the float tile kernel.  Not covered: the
tensor-core GEMMs and the cluster kernel of the public layout (their hardware has no stand-in here), timing, and
memory-ordering effects."""

import numpy as np
import pytest

from tests.simt import harness as H


@pytest.fixture(scope="module")
def L():
    return H.lib()


def _weights(rng, n, k):
    codes = rng.integers(-1, 2, (n, k)).astype(np.int8)
    scale = (rng.random(n) * 0.5 + 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    return codes, scale, bias


def _int_reference(oracle, x32, codes, scale, bias):
    q, sx = oracle.act_quant(x32)
    acc = oracle.gemm_i32(q, codes)
    return q, sx, acc, oracle.epilogue(acc, sx, scale, bias)


# ---------------------------------------------------------------------------------------------------------------
# weight side: ternarize + pack, packers, re-tiling
# ---------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("n,k,dtype", [(16, 128, H.F32), (37, 203, H.F32), (5, 7, H.BF16), (33, 64, H.F16), (1, 1, H.F32)])
def test_quantize_pack_kernel(L, oracle, n, k, dtype):
    rng = np.random.default_rng(n * 100 + k)
    w = rng.standard_normal((n, k)).astype(np.float32)
    w[0, : min(3, k)] = 0.0
    wb = H.to_bits(w, dtype)
    w32 = H.from_bits(wb, dtype)
    packed = np.empty(((k + 3) // 4, n), np.uint8)
    scale = np.empty(n, np.float32)
    codes = np.empty((n, k), np.int8)
    tern = H.empty_out((n, k), dtype)
    H.check(L.bt_quantize_pack(H.ptr(wb), dtype, n, k, k, 0.05, H.ptr(packed), H.ptr(scale), H.ptr(codes), H.ptr(tern), None))
    codes_ref, scale_ref = oracle.ternarize(w32, 0.05, dtype)
    assert np.array_equal(codes, codes_ref)
    assert np.array_equal(scale.view(np.uint32), scale_ref.view(np.uint32))
    assert np.array_equal(packed, oracle.pack_transposed(codes_ref))
    assert np.array_equal(H.from_bits(tern, dtype), codes_ref.astype(np.float32))


@pytest.mark.parametrize("n,k", [(1, 1), (5, 7), (33, 130), (48, 512)])
def test_pack_unpack_retile_kernels(L, oracle, n, k):
    rng = np.random.default_rng(n + k)
    codes = rng.integers(-1, 2, (n, k)).astype(np.int8)
    kb = (k + 3) // 4
    packed_t, packed_r = np.empty((kb, n), np.uint8), np.empty((n, kb), np.uint8)
    H.check(L.bt_pack_codes(H.ptr(codes), n, k, H.ptr(packed_t), None))
    H.check(L.bt_pack_codes_rows(H.ptr(codes), n, k, H.ptr(packed_r), None))
    assert np.array_equal(packed_t, oracle.pack_transposed(codes)) and np.array_equal(packed_r, oracle.pack(codes))
    back_t, back_r = np.empty_like(codes), np.empty_like(codes)
    H.check(L.bt_unpack_codes(H.ptr(packed_t), n, k, H.ptr(back_t), None))
    H.check(L.bt_unpack_codes_rows(H.ptr(packed_r), n, k, H.ptr(back_r), None))
    assert np.array_equal(back_t, codes) and np.array_equal(back_r, codes)
    tiled = H.retile(packed_t, k)
    assert tiled.size == ((n + 15) // 16) * ((k + 127) // 128) * 512
    again = np.empty_like(packed_t)
    H.check(L.bt_untile_packed(H.ptr(tiled), k, n, H.ptr(again), None))
    assert np.array_equal(again, packed_t)
    # reserved pattern 11 decodes to zero everywhere
    reserved = np.full((kb, n), 0xFF, np.uint8)
    out = np.empty_like(codes)
    H.check(L.bt_unpack_codes(H.ptr(reserved), n, k, H.ptr(out), None))
    assert not out.any()


@pytest.mark.parametrize("m,k,dtype", [(1, 512, H.BF16), (3, 33, H.F32), (2, 1000, H.F16), (1, 1, H.F32)])
def test_act_quant_kernel(L, oracle, m, k, dtype):
    rng = np.random.default_rng(m * 7 + k)
    xb = H.to_bits(rng.standard_normal((m, k)).astype(np.float32) * 3.0, dtype)
    xq, sx, xsum = np.empty((m, k), np.int8), np.empty(m, np.float32), np.empty(m, np.int32)
    H.check(L.bt_act_quant_i8(H.ptr(xb), dtype, m, k, k, H.ptr(xq), H.ptr(sx), H.ptr(xsum), None))
    q_ref, sx_ref = oracle.act_quant(H.from_bits(xb, dtype))
    assert np.array_equal(xq, q_ref) and np.array_equal(sx.view(np.uint32), sx_ref.view(np.uint32))
    assert np.array_equal(xsum, q_ref.astype(np.int32).sum(axis=1))


# ---------------------------------------------------------------------------------------------------------------
# the decode kernel
# ---------------------------------------------------------------------------------------------------------------

# (m, k, n, emulated SM count): ragged shapes, several column blocks per CTA, K tiles that are not a multiple of a
# warp's four, a weight stream longer than the ring (the stages wrap and the "empty" barriers are used), rows split
# over two launches
DECODE_CASES = [(1, 300, 80, 6), (1, 8192, 64, 1), (3, 200, 50, 2), (4, 1024, 96, 6), (8, 130, 33, 6), (11, 64, 17, 6),
                (2, 640, 16, 6), (1, 5, 3, 6), (16, 257, 40, 3)]


@pytest.mark.parametrize("m,k,n,sms", DECODE_CASES)
def test_decode_kernel_on_int8_rows(L, oracle, m, k, n, sms):
    H.set_sm_count(sms)
    rng = np.random.default_rng(m * 1000 + k + n)
    codes, scale, bias = _weights(rng, n, k)
    tiled = H.retile(oracle.pack_transposed(codes), k)
    xq = rng.integers(-127, 128, (m, k)).astype(np.int8)
    sx = (rng.random(m) * 0.05 + 1e-3).astype(np.float32)
    y, acc = np.empty((m, n), np.float32), np.empty((m, n), np.int32)
    H.check(L.bt_gemv_tiled_i8(H.ptr(xq), H.ptr(sx), m, k, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y), H.F32, n,
                               H.ptr(acc), 0, None))
    acc_ref = oracle.gemm_i32(xq, codes)
    assert np.array_equal(acc, acc_ref)
    assert np.array_equal(y.view(np.uint32), oracle.epilogue(acc_ref, sx, scale, bias).view(np.uint32))
    assert H.device_status() == 0


@pytest.mark.parametrize("dtype", [H.BF16, H.F32, H.F16])
@pytest.mark.parametrize("m,k,n,sms", [(1, 300, 80, 6), (1, 8500, 32, 2), (3, 200, 50, 2), (8, 130, 33, 6), (11, 64, 17, 6)])
def test_decode_kernel_with_fused_quantizer(L, oracle, m, k, n, sms, dtype):
    """K = 8500 does not fit the threads' registers: the row is read twice (maximum, then quantizer)."""
    H.set_sm_count(sms)
    rng = np.random.default_rng(m * 1000 + k + n + dtype)
    codes, scale, bias = _weights(rng, n, k)
    tiled = H.retile(oracle.pack_transposed(codes), k)
    wide = H.to_bits(rng.standard_normal((m, k + 24)).astype(np.float32) * 2.5, dtype)      # rows with a stride
    xb = wide[:, :k]
    y = H.empty_out((m, n), dtype)
    xq, sx, acc = np.empty((m, k), np.int8), np.empty(m, np.float32), np.empty((m, n), np.int32)
    H.check(L.bt_gemv_tiled(H.ptr(wide), dtype, m, k, k + 24, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y), dtype, n,
                            H.ptr(xq), H.ptr(sx), H.ptr(acc), 1, None))
    q_ref, sx_ref, acc_ref, y_ref = _int_reference(oracle, H.from_bits(np.ascontiguousarray(xb), dtype), codes, scale, bias)
    assert np.array_equal(xq, q_ref) and np.array_equal(sx.view(np.uint32), sx_ref.view(np.uint32))
    assert np.array_equal(acc, acc_ref)
    assert np.array_equal(y, H.to_bits(y_ref, dtype))
    assert H.device_status() == 0


@pytest.mark.parametrize("m,dtype", [(1, H.BF16), (3, H.F32), (11, H.BF16)])
def test_chained_layers_publish_and_consume_row_maxima(L, oracle, m, dtype):
    """Three layers, each reading the leading K columns of the previous output.  Layer i publishes max |y| per row
    into 8 words by atomic maximum (several CTAs), layer i + 1 derives its quantization scale from them: outputs equal
    the plain kernel's bit for bit, the published words hold the maximum of the stored values, a row of zeros takes
    the scale rule's other branch, the long layer (K = 8500) skips its reduction pass altogether."""
    H.set_sm_count(4)
    shapes = [(8500, 160), (136, 130), (130, 48)]
    rng = np.random.default_rng(m + dtype)
    layers = []
    for k, n in shapes:
        codes = rng.integers(-1, 2, (n, k)).astype(np.int8)
        layers.append((k, n, codes, H.retile(oracle.pack_transposed(codes), k),
                       (rng.random(n) * 0.02 + 0.001).astype(np.float32), (rng.standard_normal(n) * 0.01).astype(np.float32)))
    x0 = rng.standard_normal((m, 8500)).astype(np.float32)
    if m >= 3:
        x0[1] = 0.0
    x0 = H.to_bits(x0, dtype)

    def run(chained):
        amax = np.zeros((len(layers), m, 8), np.uint32)
        x, ldx, outs = x0, x0.shape[1], []
        for i, (k, n, codes, tiled, scale, bias) in enumerate(layers):
            y = H.empty_out((m, n), dtype)
            if chained:
                next_k = layers[i + 1][0] if i + 1 < len(layers) else n
                H.check(L.bt_gemv_tiled_chained(H.ptr(x), dtype, m, k, ldx, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y),
                                                dtype, n, H.ptr(amax[i - 1]) if i > 0 else None, H.ptr(amax[i]), next_k, 0, None))
            else:
                H.check(L.bt_gemv_tiled(H.ptr(x), dtype, m, k, ldx, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y), dtype, n,
                                        None, None, None, 0, None))
            outs.append(y)
            x, ldx = y, n
        return outs, amax

    plain, _ = run(False)
    chained, amax = run(True)
    for i, (a, b) in enumerate(zip(plain, chained)):
        assert np.array_equal(a, b), i
        k, n, codes, _, scale, bias = layers[i]
        x_in = H.from_bits(np.ascontiguousarray((x0 if i == 0 else plain[i - 1])[:, :k]), dtype)
        assert np.array_equal(a, H.to_bits(_int_reference(oracle, x_in, codes, scale, bias)[3], dtype)), i
        next_k = layers[i + 1][0] if i + 1 < len(layers) else n
        want = np.abs(H.from_bits(np.ascontiguousarray(b[:, :next_k]), dtype)).max(axis=1)
        assert np.array_equal(amax[i].max(axis=1).view(np.float32), want.astype(np.float32)), i
    assert H.device_status() == 0


_planes_reference = H.planes_reference


@pytest.mark.parametrize("dtype", [H.F32, H.BF16, H.F16])
@pytest.mark.parametrize("m,k,n,sms", [(1, 300, 80, 6), (2, 200, 50, 2), (1, 8500, 32, 2), (3, 130, 33, 6), (5, 64, 17, 6)])
def test_decode_kernel_on_float_digit_planes(L, oracle, m, k, n, sms, dtype):
    """Floating-point activations through the integer pipeline as four signed-byte digit planes: bit-identical to
    the definition (exact contraction of the fixed-point row), and within the reference's own tolerance of its float
    semantics (fp64-accumulated oracle, 1e-4)."""
    H.set_sm_count(sms)
    rng = np.random.default_rng(m * 1000 + k + n + 7 * dtype)
    codes, scale, bias = _weights(rng, n, k)
    tiled = H.retile(oracle.pack_transposed(codes), k)
    x = rng.standard_normal((m, k)).astype(np.float32) * 10.0 ** rng.integers(-3, 1 if dtype == H.F16 else 4)   # fp16 outputs stay finite
    x[0, : min(4, k)] *= 1e-6                                   # elements far below the row maximum
    xb = H.to_bits(x, dtype)
    x32 = H.from_bits(xb, dtype)
    y = H.empty_out((m, n), dtype)
    H.check(L.bt_gemv_tiled_float(H.ptr(xb), dtype, m, k, k, H.ptr(tiled), n, H.ptr(scale), H.ptr(bias), H.ptr(y), dtype, n, 0, None))
    assert np.array_equal(y, H.to_bits(_planes_reference(x32, codes, scale, bias), dtype))
    y_float = oracle.linear_float(x32, codes, scale, bias)
    tol = 1e-4 if dtype == H.F32 else 1e-2                       # half outputs: their own rounding dominates
    assert np.allclose(H.from_bits(y, dtype), y_float, rtol=tol, atol=tol * max(1.0, float(np.abs(y_float).max())))
    assert H.device_status() == 0


def test_float_digit_planes_special_rows(L, oracle):
    """A row of zeros, a row with an infinity (NaN out, as a float sum would propagate it), tiny and huge rows, no
    bias."""
    H.set_sm_count(3)
    rng = np.random.default_rng(3)
    k, n = 260, 40
    codes, scale, _ = _weights(rng, n, k)
    tiled = H.retile(oracle.pack_transposed(codes), k)
    x = rng.standard_normal((4, k)).astype(np.float32)
    x[0] = 0.0
    x[1, 17] = np.inf
    x[2] *= 1e-30
    x[3] *= 1e30
    y = np.empty((4, n), np.float32)
    H.check(L.bt_gemv_tiled_float(H.ptr(x), H.F32, 4, k, k, H.ptr(tiled), n, H.ptr(scale), None, H.ptr(y), H.F32, n, 0, None))
    want = _planes_reference(x, codes, scale, None)
    assert np.array_equal(np.isnan(y), np.isnan(want)) and np.isnan(y[1]).all() and not y[0].any()
    ok = ~np.isnan(want)
    assert np.array_equal(y[ok].view(np.uint32), want[ok].view(np.uint32))
    ref = oracle.linear_float(x[2:], codes, scale, None)
    assert np.allclose(y[2:], ref, rtol=1e-4, atol=1e-4 * float(np.abs(ref).max()))


@pytest.mark.parametrize("dtype", [H.F32, H.BF16, H.F64])
def test_float_tile_kernel(L, oracle, dtype):
    """The general float kernel (any M), unpacked and packed weights, float64 containers included."""
    rng = np.random.default_rng(dtype)
    m, k, n = 70, 45, 66
    codes, scale, bias = _weights(rng, n, k)
    xb = H.to_bits(rng.standard_normal((m, k)).astype(np.float32), dtype)
    x32 = np.asarray(xb, np.float32) if dtype == H.F64 else H.from_bits(xb, dtype)
    y_ref = oracle.linear_float(x32, codes, scale, bias)
    tol = 1e-4 if dtype != H.BF16 else 2e-2
    for packed in (False, True):
        y = H.empty_out((m, n), dtype)
        if packed:
            w = oracle.pack_transposed(codes)
            H.check(L.bt_linear_packed_float(H.ptr(xb), dtype, m, k, H.ptr(w), n, H.ptr(scale), H.ptr(bias), H.ptr(y), None))
        else:
            H.check(L.bt_linear_unpacked(H.ptr(xb), dtype, m, k, H.ptr(codes), n, H.ptr(scale), H.ptr(bias), H.ptr(y), None))
        got = np.asarray(y, np.float32) if dtype == H.F64 else H.from_bits(y, dtype)
        assert np.allclose(got, y_ref, rtol=tol, atol=tol * 10)


def test_the_emulated_hardware_rules_are_enforced(L, oracle):
    """The stand-in for the bulk copy refuses what the hardware refuses: a tiled buffer that is not 16-byte aligned is
    rejected by the entry point before any launch (BT_ERR_INVALID), as on the GPU."""
    rng = np.random.default_rng(9)
    k, n = 128, 16
    codes, scale, _ = _weights(rng, n, k)
    good = H.retile(oracle.pack_transposed(codes), k)
    raw = np.empty(good.size + 32, np.uint8)
    off = (-raw.ctypes.data) % 16 + 4                            # 4 bytes past a 16-byte boundary
    bad = raw[off:off + good.size]
    bad[:] = good
    xq = rng.integers(-127, 128, (1, k)).astype(np.int8)
    sx = np.ones(1, np.float32)
    y = np.empty((1, n), np.float32)
    rc = L.bt_gemv_tiled_i8(H.ptr(xq), H.ptr(sx), 1, k, H.ptr(bad), n, H.ptr(scale), None, H.ptr(y), H.F32, n, None, 0, None)
    assert rc == 1 and b"16-byte aligned" in L.bt_last_error()


# ---------------------------------------------------------------------------------------------------------------
# decoder-block elementwise steps fused with the quantizer
# ---------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [H.BF16, H.F32, H.F16])
@pytest.mark.parametrize("m,f", [(1, 1500), (3, 64), (2, 1), (1, 4096)])
def test_silu_mul_quant_kernel(L, oracle, m, f, dtype):
    rng = np.random.default_rng(m * 10 + f + dtype)
    gu = rng.standard_normal((m, 2 * f + 8)).astype(np.float32) * 4.0          # rows with a stride
    gu[0, : min(3, f)] = [-90.0, 90.0, 0.0][: min(3, f)]                        # the exponential's clamped ends, zero
    gub = H.to_bits(gu, dtype)
    hq, sx, xsum = np.empty((m, f), np.int8), np.empty(m, np.float32), np.empty(m, np.int32)
    h = H.empty_out((m, f), dtype)
    H.check(L.bt_silu_mul_quant(H.ptr(gub), dtype, m, f, 2 * f + 8, H.ptr(hq), H.ptr(sx), H.ptr(xsum), H.ptr(h), None))
    q_ref, sx_ref, sum_ref, h_ref = oracle.silu_mul_quant(H.from_bits(gub, dtype)[:, : 2 * f], dtype)
    assert np.array_equal(h, H.to_bits(h_ref, dtype))
    assert np.array_equal(hq, q_ref) and np.array_equal(sx.view(np.uint32), sx_ref.view(np.uint32))
    assert np.array_equal(xsum, sum_ref)
    # and it is the product a framework computes, to the last bit of the storage type but for the exponential's ulp
    import torch
    t = torch.from_numpy(H.from_bits(gub, dtype)[:, : 2 * f])
    tdt = {H.BF16: torch.bfloat16, H.F16: torch.float16, H.F32: torch.float32}[dtype]
    want = (torch.nn.functional.silu(t[:, :f].to(tdt)) * t[:, f:].to(tdt)).float().numpy()
    got = H.from_bits(h, dtype)
    ulp = {H.BF16: 2.0 ** -7, H.F16: 2.0 ** -10, H.F32: 2.0 ** -20}[dtype]
    assert np.all(np.abs(got - want) <= ulp * np.maximum(np.abs(want), 1e-3))


@pytest.mark.parametrize("dtype", [H.BF16, H.F32, H.F16])
@pytest.mark.parametrize("m,d,with_delta", [(1, 2560, True), (3, 70, True), (2, 1, False), (1, 1024, False), (2, 1500, True)])
def test_add_rmsnorm_quant_kernel(L, oracle, m, d, with_delta, dtype):
    rng = np.random.default_rng(m * 10 + d + dtype)
    x = H.to_bits(rng.standard_normal((m, d)).astype(np.float32) * 2.0, dtype)
    delta = H.to_bits(rng.standard_normal((m, d)).astype(np.float32), dtype) if with_delta else None
    w = H.to_bits(rng.standard_normal((1, d)).astype(np.float32) * 0.5 + 1.0, dtype)
    x_before = H.from_bits(x.copy(), dtype)
    yq, sx, xsum = np.empty((m, d), np.int8), np.empty(m, np.float32), np.empty(m, np.int32)
    y = H.empty_out((m, d), dtype)
    H.check(L.bt_add_rmsnorm_quant(H.ptr(x), H.ptr(delta), dtype, m, d, d, d, H.ptr(w), 1e-5, H.ptr(yq), H.ptr(sx),
                                   H.ptr(xsum), H.ptr(y), None))
    x_ref, q_ref, sx_ref, sum_ref, y_ref = oracle.add_rmsnorm_quant(
        x_before, None if delta is None else H.from_bits(delta, dtype), H.from_bits(w, dtype)[0], 1e-5, dtype)
    assert np.array_equal(x, H.to_bits(x_ref, dtype))             # the residual stream, updated in place
    assert np.array_equal(y, H.to_bits(y_ref, dtype))
    assert np.array_equal(yq, q_ref) and np.array_equal(sx.view(np.uint32), sx_ref.view(np.uint32))
    assert np.array_equal(xsum, sum_ref)
    # against the framework's RMSNorm on the same rows (its own summation order: the last bit may differ)
    import torch
    tdt = {H.BF16: torch.bfloat16, H.F16: torch.float16, H.F32: torch.float32}[dtype]
    xt = torch.from_numpy(x_ref).to(tdt).float()
    want = ((xt / torch.sqrt(xt.pow(2).mean(-1, keepdim=True) + 1e-5)) * torch.from_numpy(H.from_bits(w, dtype)[0])).to(tdt).float().numpy()
    ulp = {H.BF16: 2.0 ** -7, H.F16: 2.0 ** -10, H.F32: 2.0 ** -20}[dtype]
    assert np.all(np.abs(H.from_bits(y, dtype) - want) <= ulp * np.maximum(np.abs(want), 1e-3))


@pytest.mark.parametrize("dtype", [H.F32, H.BF16])
@pytest.mark.parametrize("m,k,n", [(3, 300, 40), (1, 2100, 16), (5, 16, 300)])
def test_float_planes_around_an_integer_contraction(L, oracle, m, k, n, dtype):
    """bt_float_planes_quant -> (an exact integer contraction standing in for the tensor-core GEMM, which subtracts
    nothing here: weights as -1/0/+1) -> bt_float_planes_combine reproduces the definition of the float path bit for
    bit: digits are balanced bytes that recompose to the fixed-point value, their row sums are exact, a row with an
    infinity is flagged and comes out as NaN."""
    rng = np.random.default_rng(m + k + n + dtype)
    codes, scale, bias = _weights(rng, n, k)
    x = rng.standard_normal((m, k)).astype(np.float32) * 10.0 ** rng.integers(-2, 3)
    if m >= 3:
        x[1, 5] = np.inf
        x[2] = 0.0
    xb = H.to_bits(x, dtype)
    x32 = H.from_bits(xb, dtype)
    planes = np.empty((4 * m, k), np.int8)
    pw, xsum, bad = np.empty(m, np.float32), np.empty(4 * m, np.int32), np.empty(m, np.int32)
    H.check(L.bt_float_planes_quant(H.ptr(xb), dtype, m, k, k, H.ptr(planes), H.ptr(pw), H.ptr(xsum), H.ptr(bad), None))
    assert np.array_equal(xsum, planes.astype(np.int32).sum(axis=1))
    assert np.array_equal(bad != 0, ~np.isfinite(x32).all(axis=1))
    p = planes.astype(np.int64).reshape(m, 4, k)
    value = ((p[:, 3] * 256 + p[:, 2]) * 256 + p[:, 1]) * 256 + p[:, 0]
    assert np.abs(p[:, 3]).max() <= 64
    for r in range(m):
        if bad[r]:
            continue
        e = max(-96, min(127, int(np.frexp(np.float32(np.abs(x32[r]).max()))[1])))
        assert np.array_equal(value[r], np.rint(x32[r] * np.float32(2.0 ** (30 - e))).astype(np.int64))
        assert pw[r] == np.float32(2.0 ** (e - 30))
    acc = (planes.astype(np.int64) @ codes.astype(np.int64).T).astype(np.int32)            # [4M, N], exact
    y = H.empty_out((m, n), dtype)
    H.check(L.bt_float_planes_combine(H.ptr(acc), m, n, H.ptr(pw), H.ptr(bad), H.ptr(scale), H.ptr(bias), H.ptr(y), dtype, n, None))
    want = _planes_reference(x32, codes, scale, bias)
    got = H.from_bits(y, dtype)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(H.to_bits(np.where(ok, want, 0), dtype)[ok], y[ok])


def test_chained_consumer_with_a_long_row_skips_its_reduction_pass(L, oracle):
    """A consumer whose rows do not fit the threads' registers (K = 8600 at one row) normally reads them twice
    (maximum, then quantizer); with the producer's published maximum it reads them once.  Same bits either way."""
    H.set_sm_count(5)
    rng = np.random.default_rng(77)
    shapes = [(200, 8600), (8600, 40)]
    layers = []
    for k, n in shapes:
        codes = rng.integers(-1, 2, (n, k)).astype(np.int8)
        layers.append((k, n, H.retile(oracle.pack_transposed(codes), k), (rng.random(n) * 0.02 + 0.001).astype(np.float32)))
    x0 = H.to_bits(rng.standard_normal((1, 200)).astype(np.float32), H.BF16)
    outs = {}
    for chained in (False, True):
        amax = np.zeros((2, 1, 8), np.uint32)
        x, ldx = x0, 200
        for i, (k, n, tiled, scale) in enumerate(layers):
            y = H.empty_out((1, n), H.BF16)
            if chained:
                H.check(L.bt_gemv_tiled_chained(H.ptr(x), H.BF16, 1, k, ldx, H.ptr(tiled), n, H.ptr(scale), None, H.ptr(y), H.BF16, n,
                                                H.ptr(amax[i - 1]) if i > 0 else None, H.ptr(amax[i]), n, 0, None))
            else:
                H.check(L.bt_gemv_tiled(H.ptr(x), H.BF16, 1, k, ldx, H.ptr(tiled), n, H.ptr(scale), None, H.ptr(y), H.BF16, n,
                                        None, None, None, 0, None))
            x, ldx = y, n
        outs[chained] = x
    assert np.array_equal(outs[False], outs[True]) and H.device_status() == 0
