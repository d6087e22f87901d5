"""GPU tests of the public API (nn modules, ops) — the reference's own test expectations
re-pointed at this backend.  The integer path is gated against the oracle; the float mode
against the reference's golden outputs at its own tolerances."""

import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import EMULATED, golden_cases, load_golden, needs_real_gpu

pytestmark = pytest.mark.gpu


def _oracle_int8_forward(oracle, x, codes, scale, bias):
    q, sx = oracle.act_quant(x)
    return oracle.epilogue(oracle.gemm_i32(q, codes), sx, scale, bias)


def _rel(y, y_ref):
    return float(np.linalg.norm(y - y_ref) / max(np.linalg.norm(y_ref), 1e-30))


def test_config1_ternary_linear_cuda_backend(oracle):
    """TernaryLinear(512 -> 256, bias, 0.05, backend="cuda") with the golden weights."""
    import bittorch_b200 as bt

    c = load_golden("c1_linear_512x256")
    layer = bt.nn.TernaryLinear(512, 256, bias=True, threshold_factor=0.05, backend="cuda").cuda()
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(c["w"]))
        layer.bias.copy_(torch.from_numpy(c["bias"]))
    x = torch.from_numpy(c["x"]).cuda()
    t, s = layer.get_quantized_weight()
    assert t.dtype == torch.float32 and np.array_equal(t.cpu().numpy(), c["codes"].astype(np.float32))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), c["scale"].view(np.uint32))
    with torch.no_grad():
        y = layer(x).cpu().numpy()
    y_ref = _oracle_int8_forward(oracle, c["x"], c["codes"], c["scale"], c["bias"])
    assert np.array_equal(y.view(np.uint32), y_ref.view(np.uint32))          # integer path: bit exact
    assert _rel(y, c["y"]) < 2e-2                                             # reported, not gated: int8 activations
    with torch.no_grad():
        y_again = layer(x).cpu().numpy()                                      # served from the packed-weight cache
    assert np.array_equal(y, y_again)


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


def test_ragged_shapes_integer_path(oracle):
    import bittorch_b200 as bt

    for name, r in golden_cases(load_golden("ragged_forward")).items():
        k = r["x"].shape[1]
        infer = bt.nn.TernaryLinearInference(k, r["codes"].shape[0], torch.from_numpy(r["packed_T"]).cuda(),
                                             torch.from_numpy(r["scale"]).cuda(), torch.from_numpy(r["bias"]).cuda())
        y = infer(torch.from_numpy(r["x"]).cuda()).cpu().numpy()
        y_ref = _oracle_int8_forward(oracle, r["x"], r["codes"], r["scale"], r["bias"])
        assert np.array_equal(y.view(np.uint32), y_ref.view(np.uint32)), name
        y_op = bt.ops.ternary_linear_packed_forward(torch.from_numpy(r["x"]).cuda(), infer.weight_packed, infer.scale, k,
                                                    infer.bias).cpu().numpy()
        assert np.array_equal(y_op.view(np.uint32), y_ref.view(np.uint32)), name


@pytest.mark.parametrize("m", [1, 4, 16, 40, 300])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_inference_module_batches_and_dtypes(oracle, m, dtype):
    import bittorch_b200 as bt

    g = torch.Generator().manual_seed(m)
    k, n = 768, 1152
    w = torch.randn(n, k, generator=g)
    b = torch.randn(n, generator=g)
    infer = bt.nn.create_ternary_linear_inference(k, n, w.cuda(), b.cuda())
    codes, scale = oracle.ternarize(w.numpy(), 0.05)
    assert np.array_equal(infer.weight_packed.cpu().numpy(), oracle.pack_transposed(codes))
    x = torch.randn(2, m, k, generator=g).to(dtype)                # leading batch dims are flattened
    y = infer(x.cuda())
    assert y.shape == (2, m, n) and y.dtype == dtype
    y_ref = _oracle_int8_forward(oracle, x.float().reshape(-1, k).numpy(), codes, scale, b.numpy())
    assert torch.equal(y.cpu().reshape(-1, n), torch.from_numpy(y_ref).to(dtype))


def test_inference_module_state_dict_and_cache_invalidation(oracle, tmp_path):
    import bittorch_b200 as bt

    g = torch.Generator().manual_seed(1)
    k, n = 200, 96
    a = bt.nn.create_ternary_linear_inference(k, n, torch.randn(n, k, generator=g).cuda(), None)
    b = bt.nn.create_ternary_linear_inference(k, n, torch.randn(n, k, generator=g).cuda(), None)
    x = torch.randn(5, k, generator=g).cuda()
    ya, yb = a(x), b(x)
    assert not torch.equal(ya, yb)
    assert set(a.state_dict()) == {"weight_packed", "scale"}         # the tiled copy is never serialized
    path = str(tmp_path / "ckpt.pt")
    bt.utils.save_ternary_checkpoint(a, path, {"note": "a"})
    assert bt.utils.load_ternary_checkpoint(path, b) == {"note": "a"}
    assert torch.equal(b(x), ya)                                        # derived copy rebuilt after load
    if not EMULATED:
        with pytest.raises(RuntimeError, match="CUDA tensor"):
            a(x.cpu())
    # a checkpoint packed by the reference loads unchanged
    c = load_golden("packed_infer_96x200")
    sd = {"weight_packed": torch.from_numpy(c["packed_T"]), "scale": torch.from_numpy(c["scale"])}
    b.load_state_dict(sd)
    y = b(torch.from_numpy(c["x"]).cuda()).cpu().numpy()
    y_ref = _oracle_int8_forward(oracle, c["x"], c["codes"], c["scale"], None)
    assert np.array_equal(y.view(np.uint32), y_ref.view(np.uint32))


@needs_real_gpu
def test_backend_selection_and_errors():
    import bittorch_b200 as bt

    with pytest.raises(ValueError, match="backend must be"):
        bt.nn.TernaryLinear(4, 4, backend="triton")
    layer = bt.nn.TernaryLinear(8, 4, backend="cuda")
    with pytest.raises(RuntimeError, match="requires input and weights on CUDA"):
        layer(torch.randn(2, 8))
    with pytest.raises(RuntimeError, match="requires CUDA"):
        bt.nn.TernaryLinearCUDA(8, 4)(torch.randn(2, 8))
    with pytest.warns(DeprecationWarning):
        assert bt.nn.TernaryLinear(8, 4, use_cuda_kernel=False).backend == "python"
    debug = bt.nn.TernaryLinear(8, 4, quantize=False).cuda()
    x = torch.randn(3, 8).cuda()
    assert torch.allclose(debug(x), torch.nn.functional.linear(x, debug.weight, debug.bias))
    assert bt.has_cuda_ext() and bt.ops.has_packed_cuda_support()
    assert torch.equal(bt._C.dummy(x), x)


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


def test_training_forward_requantizes_after_an_update():
    import bittorch_b200 as bt

    torch.manual_seed(1)
    layer = bt.nn.TernaryLinear(128, 64, backend="cuda").cuda()
    x = torch.randn(4, 128, device="cuda")
    opt = torch.optim.SGD(layer.parameters(), lr=0.5)
    with torch.no_grad():
        y0 = layer(x)
    layer(x).square().mean().backward()
    opt.step()
    with torch.no_grad():
        y1 = layer(x)
    assert not torch.equal(y0, y1)
    t, s = layer.get_quantized_weight()
    infer = bt.utils.ternary_linear_to_infer(layer)
    assert torch.equal(infer(x), y1)


def test_convert_linear_layers():
    import bittorch_b200 as bt

    torch.manual_seed(2)
    model = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), bt.nn.TernaryLinear(32, 16), nn.Linear(16, 10)).cuda()
    conv = bt.utils.convert_linear_layers(model, skip_names=["3"])
    assert isinstance(conv[0], bt.nn.TernaryLinearInference) and isinstance(conv[2], bt.nn.TernaryLinearInference)
    assert isinstance(conv[3], nn.Linear) and isinstance(model[0], nn.Linear)
    x = torch.randn(5, 64, device="cuda")
    assert conv(x).shape == (5, 10)
    counts = bt.utils.count_ternary_params(conv)
    assert counts["packed_ternary"] == 64 * 32 + 32 * 16 and counts["fp32"] == 160
    mem = bt.utils.get_model_memory_bytes(conv)
    assert mem["packed_ternary"] == 16 * 32 + 8 * 16


@needs_real_gpu
def test_autocast_forward_backward():
    import bittorch_b200 as bt

    torch.manual_seed(3)
    layer = bt.nn.TernaryLinear(64, 32, backend="cuda").cuda()
    x = torch.randn(8, 64, device="cuda", requires_grad=True)
    with torch.autocast("cuda", dtype=torch.float16):
        y = layer(x)
    assert y.dtype == torch.float16
    y.float().sum().backward()
    assert layer.weight.grad is not None and layer.weight.grad.dtype == torch.float32
    assert torch.isfinite(layer.weight.grad).all() and x.grad is not None


def test_writes_through_data_are_seen_by_the_cached_paths(oracle):
    """`p.data.copy_(w)` bumps no version counter.  Every cached path must still use the new weights on the next
    inference-mode forward: the training modules (packed copy of the master), the inference module (tiled copy of
    the packed buffer) and the decoder's fused sibling layers."""
    import bittorch_b200 as bt
    from bittorch_b200.utils.decoder import _FusedColumns

    g = torch.Generator().manual_seed(7)
    k, n = 256, 96
    w0, w1 = torch.randn(n, k, generator=g).cuda(), torch.randn(n, k, generator=g).cuda()
    x = torch.randn(3, k, generator=g).cuda()
    for cls in (bt.nn.TernaryLinear, bt.nn.TernaryLinearCUDA):
        layer = cls(k, n, bias=False).cuda() if cls is bt.nn.TernaryLinearCUDA else cls(k, n, bias=False, backend="cuda").cuda()
        with torch.no_grad():
            layer.weight.data.copy_(w0)
            y0 = layer(x)
            assert torch.equal(layer(x), y0)                          # served from the cache
            version = layer.weight._version
            layer.weight.data.copy_(w1)
            assert layer.weight._version == version                   # the write the version counter cannot see
            y1 = layer(x)
        codes, scale = oracle.ternarize(w1.cpu().numpy(), 0.05)
        assert np.array_equal(y1.cpu().numpy().view(np.uint32),
                              _oracle_int8_forward(oracle, x.cpu().numpy(), codes, scale, None).view(np.uint32))
        assert not torch.equal(y0, y1)

    a = bt.nn.create_ternary_linear_inference(k, n, w0, None)
    b = bt.nn.create_ternary_linear_inference(k, n, w1, None)
    ya, yb = a(x), b(x)
    a.weight_packed.data.copy_(b.weight_packed)
    a.scale.data.copy_(b.scale)
    assert torch.equal(a(x), yb) and not torch.equal(ya, yb)

    # with the content check off only the explicit call helps
    c = bt.nn.create_ternary_linear_inference(k, n, w0, None)
    c.verify_buffers = False
    yc = c(x)
    c.weight_packed.data.copy_(b.weight_packed)
    assert torch.equal(c(x), yc)                                      # stale by construction
    c.invalidate_cache()
    want = bt.nn.TernaryLinearInference(k, n, b.weight_packed.clone(), c.scale.clone())(x)
    assert torch.equal(c(x), want) and not torch.equal(want, yc)

    # fused sibling layers follow their members
    m1 = bt.nn.create_ternary_linear_inference(k, n, w0, None)
    m2 = bt.nn.create_ternary_linear_inference(k, 32, w1[:32].contiguous(), None)
    fused = _FusedColumns(m1, m2)
    o1, o2 = fused(x)
    assert torch.equal(o1, m1(x)) and torch.equal(o2, m2(x))          # one launch == the members, bit for bit
    m1.weight_packed.data.copy_(b.weight_packed)
    m1.scale.data.copy_(b.scale)
    o1, o2 = fused(x)
    assert torch.equal(o1, yb) and torch.equal(o2, m2(x))


def test_float64_inputs_run_the_float_path(oracle):
    """The reference dispatches its float kernels for float64 too (AT_DISPATCH_FLOATING_TYPES_AND_HALF) and computes in
    float32 (tests/test_gradient_consistency.py:233-237 feeds float64): same here, through the unpacked entry, the
    packed entry and the training module's forward and backward."""
    import bittorch_b200 as bt
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(9)
    k, n = 40, 24
    w = torch.randn(n, k, generator=g, dtype=torch.float64)
    x = torch.randn(5, k, generator=g, dtype=torch.float64)
    bias = torch.randn(n, generator=g, dtype=torch.float64)
    codes, scale = oracle.ternarize(w.float().numpy(), 0.05)
    y_ref = oracle.linear_float(x.float().numpy(), codes, scale, bias.float().numpy())
    y = _C.ternary_linear_forward(x.cuda(), torch.from_numpy(codes).cuda(), torch.from_numpy(scale).double().cuda(), bias.cuda())
    assert y.dtype == torch.float64 and np.allclose(y.cpu().numpy(), y_ref, rtol=1e-4, atol=1e-4)
    packed = _C.pack_codes(torch.from_numpy(codes).cuda())
    y = _C.ternary_linear_packed_forward(x.cuda(), packed, torch.from_numpy(scale).double().cuda(), bias.cuda(), k)
    assert y.dtype == torch.float64 and np.allclose(y.cpu().numpy(), y_ref, rtol=1e-4, atol=1e-4)

    ref = bt.nn.TernaryLinear(k, n, backend="python").double().cuda()
    cu = bt.nn.TernaryLinear(k, n, backend="cuda").double().cuda()
    cu.load_state_dict(ref.state_dict())
    x1, x2 = x.cuda().clone().requires_grad_(True), x.cuda().clone().requires_grad_(True)
    y1, y2 = ref(x1), cu(x2)
    assert y2.dtype == torch.float64 and torch.allclose(y1, y2, rtol=1e-4, atol=1e-5)      # float32 arithmetic inside
    gy = torch.randn(5, n, generator=g, dtype=torch.float64).cuda()
    y1.backward(gy)
    y2.backward(gy)
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-6, atol=1e-8)
    assert torch.allclose(ref.weight.grad, cu.weight.grad, rtol=1e-6, atol=1e-8)


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """The give-up path of the library's bounded device-side waits, through its self-test kernel (a barrier that
    nothing arrives on, a few thousand polls): the kernel returns, the status word reads BT_ERR_DEVICE_WAIT once and
    is clear afterwards, and the next kernel runs normally.  Nothing faults or traps."""
    from bittorch_b200 import _C

    assert _C.device_status() == 0
    _C.selftest_wait_timeout()
    assert _C.device_status() == 4
    assert _C.device_status() == 0
    x = torch.arange(12, dtype=torch.float32).reshape(3, 4).cuda()
    assert torch.equal(_C.dummy(x), x)
    assert _C.device_status() == 0
