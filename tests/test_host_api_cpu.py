"""CPU tests of the host-side API: the explicitly requested eager backend against the
golden outputs of the reference, and the no-CPU-fallback policy of everything else."""

import numpy as np
import pytest
import torch

from conftest import load_golden


def test_python_backend_reproduces_reference_config1():
    import bittorch_b200 as bt

    c = load_golden("c1_linear_512x256")
    torch.manual_seed(0)
    layer = bt.nn.TernaryLinear(512, 256, bias=True, threshold_factor=0.05, backend="python")
    # same initialisation stream as the reference's constructor (kaiming-uniform, then bias)
    assert np.array_equal(layer.weight.detach().numpy(), c["w"])
    assert np.array_equal(layer.bias.detach().numpy(), c["bias"])
    x = torch.randn(32, 512)
    assert np.array_equal(x.numpy(), c["x"])
    with torch.no_grad():
        y = layer(x)
    assert np.allclose(y.numpy(), c["y"], rtol=1e-5, atol=1e-6)
    t, s = layer.get_quantized_weight()
    assert np.array_equal(t.numpy(), c["codes"].astype(np.float32))
    assert np.array_equal(s.numpy().view(np.uint32), c["scale"].view(np.uint32))


def test_python_backend_ste_gradients():
    import bittorch_b200 as bt

    torch.manual_seed(0)
    layer = bt.nn.TernaryLinear(16, 8, backend="python")
    x = torch.randn(4, 16, requires_grad=True)
    layer(x).sum().backward()
    _, scale = layer.get_quantized_weight()
    expected = x.detach().sum(0).unsqueeze(0) * scale.unsqueeze(1)       # d y / d w = x * scale (STE)
    assert torch.allclose(layer.weight.grad, expected, atol=1e-6)
    assert torch.allclose(layer.bias.grad, torch.full((8,), 4.0))


def test_no_cpu_fallback_anywhere():
    import bittorch_b200 as bt

    w = torch.randn(4, 8)
    for fn in (lambda: bt.quant.ternary_quantize(w),
               lambda: bt.quant.pack_ternary(torch.sign(w)),
               lambda: bt.quant.unpack_ternary(torch.zeros(4, 2, dtype=torch.uint8), 8),
               lambda: bt.quant.quantize_pack_transposed(w),
               lambda: bt.nn.TernaryLinear(8, 4)(torch.randn(2, 8)),
               lambda: bt.nn.TernaryLinear(8, 4).get_quantized_weight(),
               lambda: bt.nn.create_ternary_linear_inference(8, 4, w)):
        with pytest.raises(RuntimeError):
            fn()
    infer = bt.nn.TernaryLinearInference(8, 4, torch.zeros(2, 4, dtype=torch.uint8), torch.ones(4))
    with pytest.raises(RuntimeError, match="no CPU path"):
        infer(torch.randn(2, 8))
    assert bt.quant.get_packed_size(4096, 4096) == 4 * 1024 * 1024      # tests/test_packed_ternary.py:119-123
    assert abs(bt.quant.get_memory_reduction(4096, 4096) - 16.0) < 0.1
