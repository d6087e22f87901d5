"""GPU parity of the per-token int8 activation quantizer: int8 codes and fp32 row scales
bit-exact against the CPU oracle (integer path: parity unpinned by the reference's tests)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,k", [(1, 4096), (16, 4096), (7, 33), (1, 1), (3, 5), (257, 520), (2048, 1024), (5, 11008)])
def test_bit_exact(oracle, dtype, m, k):
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(m * 131 + k)
    x = (torch.randn(m, k, generator=g) * 3.0).to(dtype)
    xq, sx = _C.act_quant_i8(x.cuda())
    q_ref, sx_ref = oracle.act_quant(x.float().numpy())
    assert np.array_equal(xq.cpu().numpy(), q_ref)
    assert np.array_equal(sx.cpu().numpy().view(np.uint32), sx_ref.view(np.uint32))


def test_edge_rows(oracle):
    from bittorch_b200 import _C

    x = torch.zeros(5, 64)
    x[1] = 1e-7                                    # below the 1e-6 floor -> scale 1
    x[2, :4] = torch.tensor([127.0, 0.5, -0.5, 1.5])  # ties round away from zero
    x[3] = torch.linspace(-1e4, 1e4, 64)
    x[4, 0] = -3.0
    xq, sx = _C.act_quant_i8(x.cuda())
    q_ref, sx_ref = oracle.act_quant(x.numpy())
    assert np.array_equal(xq.cpu().numpy(), q_ref)
    assert np.array_equal(sx.cpu().numpy().view(np.uint32), sx_ref.view(np.uint32))
    assert list(xq[2, :4].cpu()) == [127, 1, -1, 2] and float(sx[0]) == 1.0 and float(sx[1]) == 1.0


def test_strided_input(oracle):
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(9)
    big = torch.randn(6, 200, generator=g).cuda()
    view = big[:, 8:136]
    xq, sx = _C.act_quant_i8(view)
    q_ref, sx_ref = oracle.act_quant(view.cpu().numpy())
    assert np.array_equal(xq.cpu().numpy(), q_ref)
