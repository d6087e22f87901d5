"""Variants of the tiled decode kernel added after its first GPU runs: the launch flag for freshly written weights,
chained layers that publish their row maxima, floating-point activations as digit planes (decode kernel, and around
the tensor-core GEMM: float mode of the modules, which the reference's own float tests exercise).
(Collected after the files whose tests have already passed on a B200, so that a run that stops at the first failure
has run those first.)"""

import numpy as np
import pytest
import torch

from conftest import golden_cases, load_golden

pytestmark = pytest.mark.gpu


def test_fresh_weights_flag_gives_the_same_bits(oracle):
    """BT_LAUNCH_WEIGHTS_JUST_WRITTEN only changes how the decode kernel is ordered against its predecessor: the
    re-tile, the scale conversion and the kernel enqueued back to back, results equal to the default launch."""
    from bittorch_b200 import _C

    for (m, k, n) in [(1, 4096, 1024), (3, 520, 200)]:
        g = torch.Generator().manual_seed(m + n)
        codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
        scale16 = (torch.rand(n, generator=g) + 0.1).to(torch.bfloat16).cuda()
        packed = _C.pack_codes(codes.cuda())
        torch.cuda.synchronize()
        tiled = _C.retile(packed, k)                              # written by the kernel just before ...
        scale = scale16.float()                                   # ... and so is the float32 scale
        y_fresh = _C.gemv_tiled(x, tiled, k, n, scale, None, fresh_weights=True)
        torch.cuda.synchronize()
        y = _C.gemv_tiled(x, tiled, k, n, scale, None)
        xq, sx = _C.act_quant_i8(x)
        y_i8 = _C.gemv_tiled_i8(xq, sx, tiled, k, n, scale, None, torch.bfloat16, fresh_weights=True)
        assert torch.equal(y_fresh, y) and torch.equal(y_i8, y)
    assert _C.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m", [1, 3, 8, 11])
def test_chained_layers_with_published_row_maxima_give_the_same_bits(oracle, m, dtype):
    """Three layers in a row, each reading the leading K columns of the previous output: with the row maxima
    published by the producing kernel (bt_gemv_tiled_chained) every output equals the plain kernels', bit for bit -
    ragged shapes, a row of zeros (scale rule's 1e-6 branch), an infinite value, more output columns than the next
    layer reads."""
    from bittorch_b200 import _C

    shapes = [(200, 520), (264, 330), (330, 96)]                 # (K, N); the next K is smaller than this N
    g = torch.Generator().manual_seed(100 * m + len(str(dtype)))
    layers = []
    for k, n in shapes:
        codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
        scale = (torch.rand(n, generator=g) * 0.02 + 0.001).cuda()
        bias = (torch.randn(n, generator=g) * 0.01).cuda()
        layers.append((k, n, _C.retile(_C.pack_codes(codes.cuda()), k), scale, bias))
    x0 = torch.randn(m, 200, generator=g).to(dtype)
    if m >= 3:
        x0[1] = 0                                                 # max |x| <= 1e-6: scale 1
    if m >= 8:
        x0[5, 17] = float("inf")
    x0 = x0.cuda()
    torch.cuda.synchronize()

    def run(chained):
        amax = _C.new_amax_buffer(len(layers), m, x0.device)
        x, outs = x0, []
        for i, (k, n, tiled, scale, bias) in enumerate(layers):
            xin = x[:, :k]
            if chained:
                next_k = layers[i + 1][0] if i + 1 < len(layers) else n
                y = _C.gemv_tiled_chained(xin, tiled, k, n, scale, bias, amax_in=amax[i - 1] if i > 0 else None,
                                          amax_out=amax[i], amax_cols=next_k)
            else:
                y = _C.gemv_tiled(xin, tiled, k, n, scale, bias)
            outs.append(y)
            x = y
        torch.cuda.synchronize()
        return outs, amax

    plain, _ = run(False)
    chained, amax = run(True)
    for a, b in zip(plain, chained):
        assert torch.equal(a.view(torch.int16 if a.element_size() == 2 else torch.int32),
                           b.view(torch.int16 if b.element_size() == 2 else torch.int32))
    # what was published is the maximum of the stored values over the columns the next layer reads
    for i, y in enumerate(chained):
        next_k = layers[i + 1][0] if i + 1 < len(layers) else layers[i][1]
        vals = y[:, :next_k].float().abs()
        want = torch.where(torch.isnan(vals), torch.zeros_like(vals), vals).max(dim=1).values
        got = amax[i].max(dim=1).values.view(torch.float32) if amax[i].dtype == torch.int32 else None
        assert torch.equal(got.cpu(), want.cpu())
    assert _C.device_status() == 0


def _planes_definition(x32, codes, scale, bias):
    """bt_gemv_tiled_float's definition in numpy: fixed point from the row maximum's power of two, exact integer
    contraction, one rounding to float32, exact power of two, scale, bias (unfused float32 operations)."""
    y = np.empty((x32.shape[0], codes.shape[0]), np.float32)
    for r in range(x32.shape[0]):
        row = x32[r]
        e = max(-96, min(127, int(np.frexp(np.float32(np.abs(row).max()))[1])))
        v = np.clip(np.rint(row * np.float32(2.0 ** (30 - e))).astype(np.int64), -(1 << 30), 1 << 30)
        total = codes.astype(np.int64) @ v
        out = (total.astype(np.float32) * np.float32(2.0 ** (e - 30))) * scale
        y[r] = out + bias if bias is not None else out
    return y


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (1, 4096, 11008), (2, 2560, 6912), (4, 1024, 640), (3, 200, 50),
                                   (1, 28672, 256), (16, 65, 129), (1, 1, 1), (5, 100, 300)])
def test_float_activation_gemv_is_the_exact_contraction(oracle, m, k, n, dtype):
    """Float mode at decode sizes (bt_gemv_tiled_float): bit-identical to its definition (the exact contraction of
    the fixed-point rows), and within the reference's own tolerance (1e-4, tests/test_packed_kernel.py:50) of the
    float semantics as the oracle states them (fp64 accumulation)."""
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(m * 3 + k + n)
    codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
    x = (torch.randn(m, k, generator=g) * 0.7).to(dtype)
    scale = torch.rand(n, generator=g) * 0.05 + 0.01
    bias = torch.randn(n, generator=g)
    tiled = _C.retile(_C.pack_codes(codes.cuda()), k)
    torch.cuda.synchronize()
    y = _C.gemv_tiled_float(x.cuda(), tiled, k, n, scale.cuda(), bias.cuda())
    torch.cuda.synchronize()
    assert _C.device_status() == 0
    want = _planes_definition(x.float().numpy(), codes.numpy(), scale.numpy(), bias.numpy())
    assert torch.equal(y.cpu(), torch.from_numpy(want).to(dtype))
    y_ref = oracle.linear_float(x.float().numpy(), codes.numpy(), scale.numpy(), bias.numpy())
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    assert np.allclose(y.float().cpu().numpy(), y_ref, rtol=tol, atol=tol)


def test_float_mode_of_the_inference_module_streams_the_tiled_weights(oracle, monkeypatch):
    """BITTORCH_B200_ACT=float: small batches go through bt_gemv_tiled_float, large ones through the general float
    kernel; both within 1e-4 of the float semantics, and of each other."""
    import bittorch_b200 as bt

    monkeypatch.setenv("BITTORCH_B200_ACT", "float")
    g = torch.Generator().manual_seed(12)
    k, n = 520, 200
    w = torch.randn(n, k, generator=g)
    layer = bt.nn.create_ternary_linear_inference(k, n, w.cuda(), torch.randn(n, generator=g).cuda())
    codes, scale = oracle.ternarize(w.numpy(), 0.05)
    x = torch.randn(40, k, generator=g)
    y_ref = oracle.linear_float(x.numpy(), codes, scale, layer.bias.cpu().numpy())
    small = torch.cat([layer(x[i:i + 4].cuda()) for i in range(0, 40, 4)])      # decode kernel, 4 rows at a time
    large = layer(x.cuda())                                                       # general kernel
    assert np.allclose(small.cpu().numpy(), y_ref, rtol=1e-4, atol=1e-4)
    assert np.allclose(large.cpu().numpy(), y_ref, rtol=1e-4, atol=1e-4)


def test_float_mode_matches_reference_outputs(monkeypatch):
    """BITTORCH_B200_ACT=float reproduces the reference's float path at its own 1e-4."""
    import bittorch_b200 as bt

    monkeypatch.setenv("BITTORCH_B200_ACT", "float")
    c = load_golden("c1_linear_512x256")
    layer = bt.nn.TernaryLinear(512, 256, backend="cuda").cuda()
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(c["w"]))
        layer.bias.copy_(torch.from_numpy(c["bias"]))
        y = layer(torch.from_numpy(c["x"]).cuda()).cpu().numpy()
    assert np.allclose(y, c["y"], rtol=1e-4, atol=1e-4)
    for name, r in golden_cases(load_golden("ragged_forward")).items():
        pt = torch.from_numpy(r["packed_T"]).cuda()
        y = bt.ops.ternary_linear_packed_forward(torch.from_numpy(r["x"]).cuda(), pt, torch.from_numpy(r["scale"]).cuda(),
                                                 r["x"].shape[1], torch.from_numpy(r["bias"]).cuda())
        assert np.allclose(y.cpu().numpy(), r["y"], rtol=1e-4, atol=1e-4), name
        y2 = bt.ops.ternary_linear_forward_cuda(torch.from_numpy(r["x"]).cuda(), torch.from_numpy(r["codes"]).cuda(),
                                                torch.from_numpy(r["scale"]).cuda(), torch.from_numpy(r["bias"]).cuda())
        assert np.allclose(y2.cpu().numpy(), r["y"], rtol=1e-4, atol=1e-4), name


def test_training_step_gradients_match_python_backend(monkeypatch):
    """Float mode: forward within 1e-4 of the eager backend and identical STE gradients
    (tests/test_ternary_linear.py:395-412, tests/test_gradient_consistency.py)."""
    import bittorch_b200 as bt

    monkeypatch.setenv("BITTORCH_B200_ACT", "float")
    torch.manual_seed(0)
    ref = bt.nn.TernaryLinear(64, 48, backend="python").cuda()
    cu = bt.nn.TernaryLinear(64, 48, backend="cuda").cuda()
    cu.load_state_dict(ref.state_dict())
    x = torch.randn(10, 64, device="cuda")
    x1, x2 = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    y1, y2 = ref(x1), cu(x2)
    assert torch.allclose(y1, y2, rtol=1e-4, atol=1e-5)
    gy = torch.randn_like(y1)
    y1.backward(gy)
    y2.backward(gy)
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-4, atol=1e-5)
    assert torch.allclose(ref.weight.grad, cu.weight.grad, rtol=1e-4, atol=1e-5)
    assert torch.allclose(ref.bias.grad, cu.bias.grad, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,k,n", [(5, 64, 48), (32, 512, 256), (200, 1024, 640), (1300, 256, 96), (17, 4096, 1024)])
def test_float_activation_gemm_through_digit_planes(oracle, m, k, n, dtype):
    """Float mode above the decode sizes: digit planes -> tcgen05 GEMM (4M int8 rows, exact int32 accumulators) ->
    combine.  Bit-identical to the definition, hence to bt_gemv_tiled_float on the same rows, and within the
    reference's 1e-4 of the float semantics; 1300 rows go through two GEMM calls."""
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(m + k + n)
    codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
    x = (torch.randn(m, k, generator=g) * 0.7).to(dtype)
    scale = torch.rand(n, generator=g) * 0.05 + 0.01
    bias = torch.randn(n, generator=g)
    tiled = _C.retile(_C.pack_codes(codes.cuda()), k)
    torch.cuda.synchronize()
    assert _C.float_linear_tiled_ok(m, k, dtype)
    y = _C.float_linear_tiled(x.cuda(), tiled, k, n, scale.cuda(), bias.cuda())
    torch.cuda.synchronize()
    assert _C.device_status() == 0
    want = _planes_definition(x.float().numpy(), codes.numpy(), scale.numpy(), bias.numpy())
    assert torch.equal(y.cpu(), torch.from_numpy(want).to(dtype))
    rows = _C.gemv_tiled_float(x[:4].cuda(), tiled, k, n, scale.cuda(), bias.cuda())
    assert torch.equal(y[:4], rows)
    y_ref = oracle.linear_float(x.float().numpy(), codes.numpy(), scale.numpy(), bias.numpy())
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    assert np.allclose(y.float().cpu().numpy(), y_ref, rtol=tol, atol=tol)


def test_tensor_core_forward_versions(oracle):
    """`ternary_linear_tensor_core_forward` (csrc/kernels/ternary_gemm_tensor_core.cu:663-727): version 1 = float
    compute (here: exact, on the tensor cores through digit planes), version 2 = int8 activations."""
    import bittorch_b200 as bt

    g = torch.Generator().manual_seed(21)
    m, k, n = 48, 256, 160
    w = torch.randn(n, k, generator=g)
    codes, scale = oracle.ternarize(w.numpy(), 0.05)
    packed = torch.from_numpy(oracle.pack_transposed(codes)).cuda()
    x = torch.randn(m, k, generator=g)
    bias = torch.randn(n, generator=g)
    s = torch.from_numpy(scale).cuda()
    y1 = bt.ops.ternary_linear_tensor_core_forward(x.cuda(), packed, s, k, bias.cuda(), version=1)
    assert np.allclose(y1.cpu().numpy(), oracle.linear_float(x.numpy(), codes, scale, bias.numpy()), rtol=1e-4, atol=1e-4)
    y2 = bt.ops.ternary_linear_tensor_core_forward(x.cuda(), packed, s, k, bias.cuda(), version=2)
    q, sx = oracle.act_quant(x.numpy())
    y2_ref = oracle.epilogue(oracle.gemm_i32(q, codes), sx, scale, bias.numpy())
    assert np.array_equal(y2.cpu().numpy().view(np.uint32), y2_ref.view(np.uint32))
