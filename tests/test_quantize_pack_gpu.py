"""GPU parity of the fused ternarizer + packer: bit-exact against the golden vectors
produced by the reference and against the CPU oracle (codes, packed bytes, fp32 scale bits)."""

import numpy as np
import pytest
import torch

from conftest import golden_cases, load_golden

pytestmark = pytest.mark.gpu

DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def _bits_equal(a, b):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    na, nb = np.isnan(a), np.isnan(b)
    return np.array_equal(na, nb) and np.array_equal(a.view(np.uint32)[~na], b.view(np.uint32)[~nb])


def _run(w_np, tf, dtype_code=0):
    from bittorch_b200 import _C

    w = torch.from_numpy(np.ascontiguousarray(w_np)).to(DT[dtype_code]).cuda()
    out = _C.quantize_pack(w, tf, want_packed=True, want_codes=True, want_tern=True)
    torch.cuda.synchronize()
    return w, {k: v.cpu() for k, v in out.items()}


def _check_case(c, dtype_code=0):
    tf = float(c["tf"]) if "tf" in c else 0.05
    w, out = _run(c["w"], tf, dtype_code)
    assert np.array_equal(out["codes"].numpy(), c["codes"])
    assert _bits_equal(out["scale"].numpy(), c["scale"])
    assert np.array_equal(out["packed_T"].numpy(), c["packed_T"])
    assert out["tern"].dtype == w.dtype
    assert np.array_equal(out["tern"].float().numpy(), c["codes"].astype(np.float32))


def test_known_answers():
    for name, c in golden_cases(load_golden("kat_quant_pack")).items():
        _check_case(c)


def test_config1_bit_exact():
    _check_case(load_golden("c1_linear_512x256"))


def test_ragged_shapes():
    for name, c in golden_cases(load_golden("ragged_forward")).items():
        _check_case(c)


@pytest.mark.parametrize("tag,code", [("f16", 1), ("bf16", 2)])
def test_half_precision_masters(tag, code):
    cases = {k: v for k, v in golden_cases(load_golden("half_quant")).items() if k.startswith(tag + "_")}
    assert len(cases) == 3
    for name, c in cases.items():
        c = dict(c)
        c.pop("packed", None)
        _check_case(c, code)


@pytest.mark.parametrize("n,k,seed", [(4096, 4096, 0), (1000, 4100, 42), (11008, 512, 123), (33, 8191, 999)])
def test_against_oracle_large(oracle, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g)
    codes_ref, scale_ref = oracle.ternarize(w.numpy(), 0.05)
    _, out = _run(w.numpy(), 0.05)
    assert np.array_equal(out["codes"].numpy(), codes_ref)
    assert _bits_equal(out["scale"].numpy(), scale_ref)
    assert np.array_equal(out["packed_T"].numpy(), oracle.pack_transposed(codes_ref))


@pytest.mark.parametrize("dtype_code", [0, 1, 2])
def test_special_rows_in_every_dtype(oracle, dtype_code):
    """NaN and Inf rows, a row of zeros and a partial last group of rows, in fp32 / fp16 / bf16 masters
    (the arithmetic runs in the storage type), against the oracle."""
    from bittorch_b200 import _C

    for (n, k, seed) in [(4096, 4096, 1), (37, 1024, 2), (4, 8192, 3), (1001, 2560, 4), (130, 11008, 5)]:
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(n, k, generator=g)
        w[0, 3] = float("nan")
        w[1, 5] = float("inf")
        w[2, :] = 0.0
        w = w.to(DT[dtype_code])
        codes_ref, scale_ref = oracle.ternarize(w.float().numpy(), 0.05, dtype=dtype_code)
        out = _C.quantize_pack(w.cuda(), 0.05, want_packed=True, want_codes=True, want_tern=True)
        torch.cuda.synchronize()
        assert _C.device_status() == 0
        assert np.array_equal(out["codes"].cpu().numpy(), codes_ref)
        assert _bits_equal(out["scale"].cpu().numpy(), scale_ref)
        assert np.array_equal(out["packed_T"].cpu().numpy(), oracle.pack_transposed(codes_ref))


def test_strided_rows_and_optional_outputs():
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(3)
    big = torch.randn(40, 100, generator=g).cuda()
    view = big[:, :64]                                # row stride 100, K = 64
    out = _C.quantize_pack(view, 0.05, want_packed=True)
    ref = _C.quantize_pack(view.contiguous(), 0.05, want_packed=True)
    assert set(out) == {"scale", "packed_T"}
    assert torch.equal(out["packed_T"], ref["packed_T"]) and torch.equal(out["scale"], ref["scale"])


def test_pack_unpack_kernels_roundtrip():
    from bittorch_b200 import _C

    cases = golden_cases(load_golden("pack_roundtrip"))
    for seed in (0, 42, 123, 999):
        c = cases[f"s{seed}"]
        codes = torch.from_numpy(c["codes"]).cuda()
        packed = _C.pack_codes(codes)
        assert np.array_equal(packed.cpu().numpy(), c["packed_T"])
        assert torch.equal(_C.unpack_codes(packed, 128), codes)
    ab = cases["all_bytes"]                          # reserved pattern 11 -> 0
    packed_T = torch.from_numpy(ab["packed"]).cuda().T.contiguous()
    assert np.array_equal(_C.unpack_codes(packed_T, 1024).cpu().numpy(), ab["codes"])


@pytest.mark.parametrize("k,n", [(4096, 4096), (33, 65), (5, 1), (100, 300), (8192, 1000)])
def test_tiled_layout_roundtrips_to_public_bytes(k, n):
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(k + n)
    codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8).cuda()
    packed = _C.pack_codes(codes)
    tiled = _C.retile(packed, k)
    assert tiled.numel() == _C.tiled_bytes(k, n)
    assert torch.equal(_C.untile(tiled, k, n), packed)


def test_quant_api_matches_reference_semantics():
    """bittorch.quant functions on CUDA tensors: shapes, dtypes and golden values."""
    from bittorch_b200 import quant

    c = load_golden("c1_linear_512x256")
    w = torch.from_numpy(c["w"]).cuda()
    t, s = quant.ternary_quantize(w)
    assert t.dtype == torch.float32 and t.shape == w.shape and s.shape == (256,)
    assert np.array_equal(t.cpu().numpy(), c["codes"].astype(np.float32))
    assert _bits_equal(s.cpu().numpy(), c["scale"])
    p, k = quant.pack_ternary(t)
    pt, _ = quant.pack_ternary_transposed(t)
    assert k == 512 and np.array_equal(p.cpu().numpy(), c["packed"]) and np.array_equal(pt.cpu().numpy(), c["packed_T"])
    assert np.array_equal(quant.unpack_ternary(p, k).cpu().numpy(), c["codes"])
    assert np.array_equal(quant.unpack_ternary_transposed(pt, k).cpu().numpy(), c["codes"])
    fused, s2, _ = quant.quantize_pack_transposed(w)
    assert torch.equal(fused, pt) and torch.equal(s2, s)
    t_g, s_g = quant.ternary_quantize(w, per_channel=False)
    assert s_g.dim() == 0 and float(s_g) == float(w.abs().max())
    thr = 0.05 * s_g
    assert torch.equal(t_g, torch.where(w.abs() > thr, torch.sign(w), torch.zeros_like(w)))
    w2 = w.clone().requires_grad_(True)
    t_ste, _ = quant.ternary_quantize_ste(w2)
    t_ste.sum().backward()
    assert torch.equal(w2.grad, torch.ones_like(w2))       # tests/test_ternary_quant.py:103-116
    assert quant.get_packed_size(4096, 4096) == 4 * 1024 * 1024
