"""Host-side caches under writes through `.data`, float64 inputs, the wait self-test and the row-layout packer: module
behaviour and entry points added after the first GPU runs.
(Collected after the files whose tests have already passed on a B200, so that a run that stops at the first failure
has run those first.)"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle_int8_forward(oracle, x, codes, scale, bias):
    q, sx = oracle.act_quant(x)
    return oracle.epilogue(oracle.gemm_i32(q, codes), sx, scale, bias)


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


def test_the_content_check_can_be_switched_off_for_a_whole_model():
    """`verify_weight_contents(model, False)` reaches the training modules' caches and the inference modules alike;
    from then on a write through `.data` is seen only after `invalidate_cache()`, and switching the check back on
    restores the default behaviour."""
    import bittorch_b200 as bt

    g = torch.Generator().manual_seed(8)
    k, n = 128, 48
    w0, w1 = torch.randn(n, k, generator=g).cuda(), torch.randn(n, k, generator=g).cuda()
    x = torch.randn(2, k, generator=g).cuda()
    model = torch.nn.Sequential(bt.nn.TernaryLinear(k, n, bias=False, backend="cuda"), bt.nn.TernaryLinearCUDA(k, n, bias=False),
                                bt.nn.create_ternary_linear_inference(k, n, w0, None)).cuda()
    assert bt.nn.verify_weight_contents(model, False) == 3
    with torch.no_grad():
        for layer in model[:2]:
            layer.weight.data.copy_(w0)
            layer.invalidate_cache()
            y0 = layer(x)
            layer.weight.data.copy_(w1)
            assert torch.equal(layer(x), y0)                          # stale by construction
            layer.invalidate_cache()
            y1 = layer(x)
            assert not torch.equal(y1, y0)
            assert torch.equal(y1, model[2].__class__(k, n, *_packed(bt, w1))(x))
        assert bt.nn.verify_weight_contents(model, True) == 3
        model[0].weight.data.copy_(w0)
        assert torch.equal(model[0](x), y0)                           # seen again without any call


def _packed(bt, w):
    """(weight_packed, scale) of the inference form of master weights `w`."""
    layer = bt.nn.create_ternary_linear_inference(w.shape[1], w.shape[0], w, None)
    return layer.weight_packed, layer.scale


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


def test_row_layout_packer_and_unpacker(oracle):
    """pack_ternary / unpack_ternary ([N, ceil(K/4)], bittorch/quant/ternary_packed.py:22-120) as kernels of their
    own: the oracle's bytes, the docstring's known answer, ragged K, the reserved pattern."""
    import bittorch_b200 as bt

    kat = torch.tensor([[1, -1, 0, 1], [0, 1, 1, -1]], dtype=torch.float32).cuda()
    packed, k = bt.quant.pack_ternary(kat)
    assert k == 4 and packed.cpu().tolist() == [[73], [148]]                 # 0x49 and its neighbour
    for (n, k) in [(1, 1), (5, 7), (33, 130), (64, 256), (17, 1023)]:
        g = torch.Generator().manual_seed(n * 1000 + k)
        codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
        packed, k_out = bt.quant.pack_ternary(codes.cuda())
        assert k_out == k and packed.shape == (n, (k + 3) // 4) and packed.dtype == torch.uint8
        assert np.array_equal(packed.cpu().numpy(), oracle.pack(codes.numpy()))
        back = bt.quant.unpack_ternary(packed, k)
        assert back.dtype == torch.int8 and torch.equal(back.cpu(), codes)
        assert torch.equal(packed.T.contiguous(), bt.quant.pack_ternary_transposed(codes.cuda())[0])
    reserved = torch.full((3, 2), 0xFF, dtype=torch.uint8).cuda()
    assert int(bt.quant.unpack_ternary(reserved, 8).abs().sum()) == 0       # pattern 11 decodes to 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_fused_elementwise_kernels_are_the_oracles_arithmetic(oracle, dtype):
    """bt_silu_mul_quant and bt_add_rmsnorm_quant against their CPU definition, bit for bit: the unquantized values in
    the activation type, the int8 codes, the scales, the row sums, the residual stream updated in place."""
    from bittorch_b200 import _C

    code = {torch.float32: oracle.DT_F32, torch.float16: oracle.DT_F16, torch.bfloat16: oracle.DT_BF16}[dtype]
    g = torch.Generator().manual_seed(31)
    for m, f in ((1, 6912), (5, 1024), (33, 40), (2, 1)):
        gu = (torch.randn(m, 2 * f, generator=g) * 4.0).to(dtype)
        hq, sx, xsum, h = _C.silu_mul_quant(gu.cuda(), want_h=True)
        q_ref, sx_ref, sum_ref, h_ref = oracle.silu_mul_quant(gu.float().numpy(), code)
        assert torch.equal(h.cpu(), torch.from_numpy(h_ref).to(dtype))
        assert np.array_equal(hq.cpu().numpy(), q_ref) and np.array_equal(xsum.cpu().numpy(), sum_ref)
        assert np.array_equal(sx.cpu().numpy().view(np.uint32), sx_ref.view(np.uint32))
    for m, d, with_delta in ((1, 2560, True), (4, 256, True), (40, 70, False), (2, 1, True)):
        x = (torch.randn(m, d, generator=g) * 2.0).to(dtype)
        delta = torch.randn(m, d, generator=g).to(dtype) if with_delta else None
        w = (torch.randn(d, generator=g) * 0.5 + 1.0).to(dtype)
        x_dev = x.clone().cuda()                                                    # updated in place by the kernel
        yq, sx, xsum, y = _C.add_rmsnorm_quant(x_dev, None if delta is None else delta.cuda(), w.cuda(), 1e-5, want_y=True)
        x_ref, q_ref, sx_ref, sum_ref, y_ref = oracle.add_rmsnorm_quant(
            x.float().numpy(), None if delta is None else delta.float().numpy(), w.float().numpy(), 1e-5, code)
        assert torch.equal(x_dev.cpu(), torch.from_numpy(x_ref).to(dtype))         # in place
        assert torch.equal(y.cpu(), torch.from_numpy(y_ref).to(dtype))
        assert np.array_equal(yq.cpu().numpy(), q_ref) and np.array_equal(xsum.cpu().numpy(), sum_ref)
        assert np.array_equal(sx.cpu().numpy().view(np.uint32), sx_ref.view(np.uint32))
    assert _C.device_status() == 0


def test_the_smoke_entry_point_and_its_report_of_the_newer_paths(monkeypatch):
    """`__graft_entry__.smoke()` passes, and what its child process would report about the newer entry points (here
    computed in this process) is all true with a clean device status."""
    import __graft_entry__ as entry

    monkeypatch.setattr(entry, "_report_newer_paths", lambda: None)
    entry.smoke()
    report = entry.newer_paths()["newer_paths"]
    assert report.pop("device_status") == 0
    assert report and all(v is True for v in report.values()), report
