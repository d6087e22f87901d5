"""The config-3 prefill cells of the tensor-core GEMM at full size, every row.
(Collected after the files whose tests have already passed on a B200, so that a run that stops at the first failure
has run those first.)"""

import numpy as np
import pytest
import torch

from conftest import needs_real_gpu

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n", [pytest.param(2048, 4096, 4096, marks=needs_real_gpu),
                                   pytest.param(2048, 4096, 11008, marks=needs_real_gpu),
                                   pytest.param(256, 4096, 11008, marks=needs_real_gpu), (300, 512, 320)])
def test_gemm_config3_cells_every_row_exact(oracle, m, k, n):
    """The config-3 prefill cells at full size, EVERY row: int32 accumulators against an exact contraction (float64
    matmul: products <= 127 and sums <= 127 K are integers far below 2^53, so it is exact whatever the summation
    order), outputs against the oracle's epilogue arithmetic written with separate (unfused) torch operations, and
    a sample of rows spread over every row tile against the scalar CPU oracle itself."""
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(m + k + n)
    codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
    xq = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    sx = torch.rand(m, generator=g) * 0.05 + 1e-3
    scale = torch.rand(n, generator=g) + 0.1
    bias = torch.randn(n, generator=g)
    tiled = _C.retile(_C.pack_codes(codes.cuda()), k)
    y, acc = _C.gemm_tiled_i8(xq.cuda(), sx.cuda(), tiled, k, n, scale.cuda(), bias.cuda(), torch.float32, want_acc=True)
    torch.cuda.synchronize()
    assert _C.device_status() == 0
    exact = torch.empty((m, n), dtype=torch.int32, device=acc.device)
    cd = codes.cuda().double()
    for m0 in range(0, m, 256):                                  # blocks of rows keep the float64 operands small
        exact[m0:m0 + 256] = torch.matmul(xq[m0:m0 + 256].cuda().double(), cd.T).to(torch.int32)
    assert torch.equal(acc, exact)
    y_want = (exact.float() * sx.cuda()[:, None]) * scale.cuda()[None, :] + bias.cuda()[None, :]
    assert torch.equal(y, y_want)
    rows = sorted({(17 * i) % m for i in range(24)} | {0, m - 1} | set(range(127, m, 128)))[:40]
    acc_ref = oracle.gemm_i32(xq[rows].numpy(), codes.numpy())
    y_ref = oracle.epilogue(acc_ref, sx[rows].numpy(), scale.numpy(), bias.numpy())
    assert np.array_equal(acc[rows].cpu().numpy(), acc_ref)
    assert np.array_equal(y[rows].cpu().numpy().view(np.uint32), y_ref.view(np.uint32))
