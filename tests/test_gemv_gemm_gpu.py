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
