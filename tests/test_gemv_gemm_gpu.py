"""GPU parity of the integer contraction kernels through the C ABI.

int32 accumulators: bit-exact against the CPU oracle.  Float outputs: the epilogue is the
oracle's arithmetic ((float(acc)*sx)*scale + bias, no fused multiply-add), so fp32 outputs
are compared bit for bit and bf16/fp16 outputs after the same final rounding; the gate the
path is specified with (rtol 1e-3 / atol 1e-3 relative to the output norm) is asserted too.
"""

import numpy as np
import pytest
import torch

from conftest import needs_real_gpu

pytestmark = pytest.mark.gpu


def _problem(m, k, n, seed, bias=True):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
    xq = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    sx = torch.rand(m, generator=g) * 0.05 + 1e-3
    scale = torch.rand(n, generator=g) + 0.1
    b = torch.randn(n, generator=g) if bias else None
    return codes, xq, sx, scale, b


def _reference(oracle, codes, xq, sx, scale, b):
    acc = oracle.gemm_i32(xq.numpy(), codes.numpy())
    y = oracle.epilogue(acc, sx.numpy(), scale.numpy(), None if b is None else b.numpy())
    return acc, y


def _within_gate(y, y_ref):
    y = np.asarray(y, np.float64)
    y_ref = np.asarray(y_ref, np.float64)
    norm = np.linalg.norm(y_ref) / np.sqrt(y_ref.size)          # rms of the output
    return np.max(np.abs(y - y_ref)) <= 1e-3 * norm + 1e-3


def _run(fn_name, codes, xq, sx, scale, b, out_dtype, tiled=True):
    from bittorch_b200 import _C

    k = codes.shape[1]
    n = codes.shape[0]
    packed = _C.pack_codes(codes.cuda())
    dev = lambda t: None if t is None else t.cuda()
    if tiled:
        w = _C.retile(packed, k)
        y, acc = getattr(_C, fn_name)(dev(xq), dev(sx), w, k, n, dev(scale), dev(b), out_dtype, want_acc=True)
    else:
        y, acc = _C.gemv_packed_i8(dev(xq), dev(sx), packed, k, dev(scale), dev(b), out_dtype, want_acc=True)
    torch.cuda.synchronize()
    assert _C.device_status() == 0
    return y.cpu(), acc.cpu()


GEMV_SHAPES = [(1, 4096, 4096), (4, 4096, 4096), (16, 4096, 4096), (1, 4096, 11008), (16, 4096, 11008),
               (1, 1, 1), (7, 33, 17), (3, 5, 2), (16, 65, 129), (9, 31, 64), (1, 13, 67), (8, 2560, 6912),
               (1, 8192, 3584), (2, 28672, 1024), (16, 6912, 2560), (5, 100, 300), (1, 32, 64), (13, 48, 200)]


@pytest.mark.parametrize("m,k,n", GEMV_SHAPES)
def test_gemv_tiled_bit_exact(oracle, m, k, n):
    prob = _problem(m, k, n, seed=m + k + n)
    acc_ref, y_ref = _reference(oracle, *prob)
    y, acc = _run("gemv_tiled_i8", *prob, torch.float32)
    assert np.array_equal(acc.numpy(), acc_ref)
    assert np.array_equal(y.numpy().view(np.uint32), y_ref.view(np.uint32))
    assert _within_gate(y.numpy(), y_ref)


@pytest.mark.parametrize("m,k,n", GEMV_SHAPES)
def test_gemv_public_layout_bit_exact(oracle, m, k, n):
    prob = _problem(m, k, n, seed=2 * (m + k + n))
    acc_ref, y_ref = _reference(oracle, *prob)
    y, acc = _run("gemv_packed_i8", *prob, torch.float32, tiled=False)
    assert np.array_equal(acc.numpy(), acc_ref)
    assert np.array_equal(y.numpy().view(np.uint32), y_ref.view(np.uint32))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemv_half_outputs_and_no_bias(oracle, dtype):
    prob = _problem(4, 1024, 640, seed=77, bias=False)
    acc_ref, y_ref = _reference(oracle, *prob)
    y, acc = _run("gemv_tiled_i8", *prob, dtype)
    assert np.array_equal(acc.numpy(), acc_ref)
    assert torch.equal(y, torch.from_numpy(y_ref).to(dtype))
    assert _within_gate(y.float().numpy(), y_ref) or dtype != torch.float32


def test_gemv_extreme_values(oracle):
    """All-(+1) weights against all-(+-127) activations: the largest accumulators."""
    k, n = 28672, 128
    codes = torch.ones(n, k, dtype=torch.int8)
    codes[1::2] = -1
    xq = torch.full((2, k), 127, dtype=torch.int8)
    xq[1] = -127
    sx, scale = torch.ones(2), torch.ones(n)
    acc_ref, y_ref = _reference(oracle, codes, xq, sx, scale, None)
    y, acc = _run("gemv_tiled_i8", codes, xq, sx, scale, None, torch.float32)
    assert np.array_equal(acc.numpy(), acc_ref) and abs(int(acc[0, 0])) == 127 * k


GEMM_SHAPES = [(256, 4096, 4096), (2048, 1024, 1024), (17, 128, 256), (128, 128, 256), (129, 256, 64), (300, 512, 320),
               (256, 4096, 1376), (520, 2560, 6912), (33, 48, 70), (64, 16, 5), (257, 272, 513), (20, 8192, 512)]


@pytest.mark.parametrize("m,k,n", GEMM_SHAPES)
def test_gemm_tcgen05_bit_exact(oracle, m, k, n):
    prob = _problem(m, k, n, seed=3 * (m + k + n))
    acc_ref, y_ref = _reference(oracle, *prob)
    y, acc = _run("gemm_tiled_i8", *prob, torch.float32)
    assert np.array_equal(acc.numpy(), acc_ref)
    assert np.array_equal(y.numpy().view(np.uint32), y_ref.view(np.uint32))
    assert _within_gate(y.numpy(), y_ref)


@pytest.mark.parametrize("bn", ["64", "128", "256"])
def test_gemm_every_tile_width_gives_the_same_bits(oracle, bn, tuning):
    """The launcher picks the output-tile width from the problem size; force each one."""
    from bittorch_b200 import _C

    tuning(_C.TUNE_GEMM_BN, int(bn))
    for (m, k, n) in [(300, 1024, 720), (17, 4096, 256), (1, 128, 16), (130, 144, 1000)]:
        prob = _problem(m, k, n, seed=int(bn) + m)
        acc_ref, y_ref = _reference(oracle, *prob)
        y, acc = _run("gemm_tiled_i8", *prob, torch.float32)
        assert np.array_equal(acc.numpy(), acc_ref)
        assert np.array_equal(y.numpy().view(np.uint32), y_ref.view(np.uint32))


@pytest.mark.parametrize("m,k,n", [(256, 128, 256), (300, 1024, 720), (129, 4096, 256), (1000, 2560, 6912),
                                   (512, 144, 1000), (2, 128, 16), (2048, 1024, 1024)])
def test_gemm_cta_pair_kernel_bit_exact(oracle, m, k, n, tuning):
    """The cta_group::2 kernel (two CTAs share a 256 x 256 tile), forced for every shape."""
    from bittorch_b200 import _C

    tuning(_C.TUNE_GEMM_PAIR, 1)
    prob = _problem(m, k, n, seed=m + 2 * k + 3 * n)
    acc_ref, y_ref = _reference(oracle, *prob)
    y, acc = _run("gemm_tiled_i8", *prob, torch.float32)
    assert np.array_equal(acc.numpy(), acc_ref)
    assert np.array_equal(y.numpy().view(np.uint32), y_ref.view(np.uint32))


@pytest.mark.parametrize("split", ["1", "2", "4", "8"])
@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (16, 4096, 11008), (32, 2560, 6912), (5, 1024, 300), (17, 128, 256),
                                   (9, 48, 70), (20, 8192, 512), (3, 16, 5), (32, 1040, 513)])
def test_gemm_narrow_batch_every_k_split_gives_the_same_bits(oracle, m, k, n, split, tuning):
    """Up to 32 rows: full-width tiles with K split over a thread-block cluster, partial accumulators
    exchanged through distributed shared memory.  Every cluster size gives the oracle's bits."""
    from bittorch_b200 import _C

    tuning(_C.TUNE_GEMM_SPLIT, int(split))
    prob = _problem(m, k, n, seed=int(split) + m + n)
    acc_ref, y_ref = _reference(oracle, *prob)
    y, acc = _run("gemm_tiled_i8", *prob, torch.float32)
    assert np.array_equal(acc.numpy(), acc_ref)
    assert np.array_equal(y.numpy().view(np.uint32), y_ref.view(np.uint32))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_half_outputs(oracle, dtype):
    prob = _problem(200, 384, 328, seed=5)
    acc_ref, y_ref = _reference(oracle, *prob)
    y, acc = _run("gemm_tiled_i8", *prob, dtype)
    assert np.array_equal(acc.numpy(), acc_ref)
    assert torch.equal(y, torch.from_numpy(y_ref).to(dtype))


@needs_real_gpu
def test_gemm_full_size_properties():
    """2048 x 4096 x 11008: too large for the scalar oracle in seconds, so checked through
    size-independent properties: agreement with the decode kernel on row blocks, linearity
    in the activation scale, and column-shard consistency."""
    from bittorch_b200 import _C

    m, k, n = 2048, 4096, 11008
    g = torch.Generator().manual_seed(11)
    codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8).cuda()
    xq = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).cuda()
    sx = (torch.rand(m, generator=g) * 0.05 + 1e-3).cuda()
    scale = (torch.rand(n, generator=g) + 0.1).cuda()
    packed = _C.pack_codes(codes)
    tiled = _C.retile(packed, k)
    y, acc = _C.gemm_tiled_i8(xq, sx, tiled, k, n, scale, None, torch.float32, want_acc=True)
    for m0 in (0, 1040, 2032):
        y2, acc2 = _C.gemv_tiled_i8(xq[m0:m0 + 16], sx[m0:m0 + 16], tiled, k, n, scale, None, torch.float32, want_acc=True)
        assert torch.equal(acc[m0:m0 + 16], acc2) and torch.equal(y[m0:m0 + 16], y2)
    ref = torch.matmul(xq[:64].double(), codes.double().T).to(torch.int32)      # exact in float64
    assert torch.equal(acc[:64], ref)
    y_doubled = _C.gemm_tiled_i8(xq, sx * 2, tiled, k, n, scale, None, torch.float32)
    assert torch.equal(y_doubled, y * 2)
    shard = _C.retile(packed[:, 2752:5504].contiguous(), k)
    y_shard = _C.gemm_tiled_i8(xq, sx, shard, k, 2752, scale[2752:5504].contiguous(), None, torch.float32)
    assert torch.equal(y_shard, y[:, 2752:5504])
    assert _C.device_status() == 0


FUSED_SHAPES = [(1, 4096, 4096), (1, 4096, 11008), (2, 4096, 4096), (3, 2560, 6912), (4, 4096, 11008), (7, 33, 17),
                (8, 1024, 640), (1, 1, 1), (16, 4096, 4096), (9, 8192, 1024), (5, 100, 300), (13, 48, 200),
                (1, 28672, 256), (16, 65, 129)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("m,k,n", FUSED_SHAPES)
def test_gemv_fused_quantizer_bit_exact(oracle, m, k, n, dtype):
    """One-kernel decode layer (activation quantizer inside the GEMV): int8 activations,
    row scales, int32 accumulators and outputs all equal the oracle's, bit for bit."""
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(m * 7 + k + n)
    codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
    x = (torch.randn(m, k, generator=g) * 2.5).to(dtype)
    scale = torch.rand(n, generator=g) + 0.1
    bias = torch.randn(n, generator=g)
    tiled = _C.retile(_C.pack_codes(codes.cuda()), k)
    y, xq, sx, acc = _C.gemv_tiled(x.cuda(), tiled, k, n, scale.cuda(), bias.cuda(), want_debug=True)
    torch.cuda.synchronize()
    assert _C.device_status() == 0
    q_ref, sx_ref = oracle.act_quant(x.float().numpy())
    acc_ref = oracle.gemm_i32(q_ref, codes.numpy())
    y_ref = oracle.epilogue(acc_ref, sx_ref, scale.numpy(), bias.numpy())
    assert np.array_equal(xq.cpu().numpy(), q_ref)
    assert np.array_equal(sx.cpu().numpy().view(np.uint32), sx_ref.view(np.uint32))
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert torch.equal(y.cpu(), torch.from_numpy(y_ref).to(dtype))


@pytest.mark.parametrize("split", ["1", "2", "4", "8"])
def test_public_layout_every_k_split_gives_the_same_bits(oracle, split, tuning):
    """The compatibility kernel splits K over a thread-block cluster; every split size must
    produce the oracle's accumulators."""
    from bittorch_b200 import _C

    tuning(_C.TUNE_GEMV_SPLIT, int(split))
    for (m, k, n) in [(1, 4096, 1024), (6, 1000, 200), (16, 2048, 512)]:
        prob = _problem(m, k, n, seed=int(split) + m)
        acc_ref, y_ref = _reference(oracle, *prob)
        y, acc = _run("gemv_packed_i8", *prob, torch.float32, tiled=False)
        assert np.array_equal(acc.numpy(), acc_ref)
        assert np.array_equal(y.numpy().view(np.uint32), y_ref.view(np.uint32))


def test_fused_and_two_kernel_paths_agree(oracle):
    from bittorch_b200 import _C

    for (m, k, n) in [(1, 4096, 1024), (6, 1000, 200), (16, 2048, 512), (11, 28672, 64)]:
        g = torch.Generator().manual_seed(m)
        codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
        scale = (torch.rand(n, generator=g) + 0.1).cuda()
        tiled = _C.retile(_C.pack_codes(codes.cuda()), k)
        y = _C.gemv_tiled(x, tiled, k, n, scale, None)
        xq, sx = _C.act_quant_i8(x)
        assert torch.equal(y, _C.gemv_tiled_i8(xq, sx, tiled, k, n, scale, None, torch.bfloat16))
    assert _C.device_status() == 0


def test_gemv_fused_strided_rows(oracle):
    """Activations that are a column slice of a wider matrix (row stride > K)."""
    from bittorch_b200 import _C

    g = torch.Generator().manual_seed(21)
    k, n = 512, 384
    codes = torch.randint(-1, 2, (n, k), generator=g, dtype=torch.int8)
    wide = torch.randn(4, 1408, generator=g).to(torch.bfloat16).cuda()
    x = wide[:, :k]
    scale = (torch.rand(n, generator=g) + 0.1).cuda()
    tiled = _C.retile(_C.pack_codes(codes.cuda()), k)
    y, xq, sx, acc = _C.gemv_tiled(x, tiled, k, n, scale, None, want_debug=True)
    q_ref, sx_ref = oracle.act_quant(x.float().cpu().numpy())
    assert np.array_equal(xq.cpu().numpy(), q_ref)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i32(q_ref, codes.numpy()))
