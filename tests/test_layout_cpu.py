"""The private tiled layout and the tensor-core operand layout, restated in Python from the formulas in the kernel
files' comments, checked for self-consistency on CPU: every weight of a tile has exactly one slot, the two ways the
kernels read a tile (dp4a planes, tensor-core operand rows) see the weights the formula says they see, and the
128-byte swizzle used for the unpacked tiles is a permutation without bank conflicts for the stores that write it."""

import itertools

import numpy as np


def slot(n_local: int, k_local: int):
    """Word index and bit shift of weight (n_local, k_local) in a 512-byte tile (csrc/retile.cuh: tile_slot)."""
    g, qlo = n_local & 7, n_local >> 3
    t, r = k_local >> 5, k_local & 31
    i, qhi, j = r >> 3, (r >> 2) & 1, r & 3
    return (4 * g + t) * 4 + (qlo | (qhi << 1)), 8 * j + 2 * i


def test_every_weight_of_a_tile_has_exactly_one_two_bit_slot():
    seen = set()
    for n, k in itertools.product(range(16), range(128)):
        word, shift = slot(n, k)
        assert 0 <= word < 128 and shift in range(0, 32, 2)
        seen.add((word, shift))
    assert len(seen) == 16 * 128                      # 128 words x 16 fields, all used once


def _tile_words(codes):
    """codes: int array [16, 128] in {-1,0,1} -> the tile's 128 32-bit words (weights stored as t + 1)."""
    words = np.zeros(128, dtype=np.uint64)
    for n, k in itertools.product(range(16), range(128)):
        word, shift = slot(n, k)
        words[word] |= np.uint64(int(codes[n, k]) + 1) << np.uint64(shift)
    return words.astype(np.uint32)


def test_a_masked_plane_is_four_consecutive_inputs_of_one_column():
    """Decode kernel: lane 4g+t, word q, plane i -> bytes (t+1) * 4^i of column g + 8(q&1),
    inputs 32t + 8i + 4(q>>1) + 0..3."""
    rng = np.random.default_rng(0)
    codes = rng.integers(-1, 2, size=(16, 128))
    words = _tile_words(codes)
    for lane, q, i in itertools.product(range(32), range(4), range(4)):
        g, t = lane >> 2, lane & 3
        w = int(words[lane * 4 + q])
        plane = (w >> (2 * i)) & 0x03030303
        n = g + 8 * (q & 1)
        k0 = 32 * t + 8 * i + 4 * (q >> 1)
        got = [((plane >> (8 * j)) & 0xFF) - 1 for j in range(4)]
        assert got == [int(codes[n, k0 + j]) for j in range(4)]


def test_unpacked_operand_rows_and_swizzle():
    """Tensor-core kernels: lane (g,t) writes, for column g + 8h, chunk 2t + c (16 bytes = inputs 32t + 16c + 0..15,
    planes 2c and 2c+1 of the words h and h+2) of a K-major 128-byte row, at chunk position (2t + c) ^ (row & 7).
    Read back through the same swizzle, row n must be inputs 0..127 of column n in order."""
    rng = np.random.default_rng(1)
    codes = rng.integers(-1, 2, size=(16, 128))
    words = _tile_words(codes).reshape(32, 4)
    smem = np.full((16, 128), 255, dtype=np.uint8)           # 16 rows x 128 bytes (two 8-row swizzle atoms)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        w = [int(x) for x in words[lane]]
        for h in range(2):
            row = g + 8 * h
            for c in range(2):
                v = [(w[h] >> (4 * c)) & 0x03030303, (w[h + 2] >> (4 * c)) & 0x03030303,
                     (w[h] >> (4 * c + 2)) & 0x03030303, (w[h + 2] >> (4 * c + 2)) & 0x03030303]
                chunk = ((2 * t + c) ^ (row & 7)) * 16
                for wi, word in enumerate(v):
                    for b in range(4):
                        smem[row, chunk + 4 * wi + b] = (word >> (8 * b)) & 0xFF
    assert smem.max() <= 2                                   # every byte written
    for n in range(16):
        row = np.concatenate([smem[n, ((c ^ (n & 7)) * 16):((c ^ (n & 7)) * 16 + 16)] for c in range(8)])
        assert np.array_equal(row.astype(np.int64) - 1, codes[n])


def test_the_stores_of_a_quarter_warp_touch_every_bank_once():
    """A 16-byte store is issued per quarter warp (8 lanes = 2 values of g x 4 values of t): the eight chunks must
    fall into eight different 16-byte bank groups of the 128-byte row."""
    for h, c, quarter in itertools.product(range(2), range(2), range(4)):
        groups = set()
        for lane in range(8 * quarter, 8 * quarter + 8):
            g, t = lane >> 2, lane & 3
            row = g + 8 * h
            groups.add((2 * t + c) ^ (row & 7))              # rows are 128 bytes apart: same banks, chunk decides
        assert len(groups) == 8


def test_plane_arithmetic_of_the_decode_kernel_is_exact():
    """Decode kernel: planes 0..2 enter dp4a as unsigned codes (t+1) * 4^i, plane 3 as the signed bytes
    (field ^ 0x40) = -t * 64; the fold acc0 + (acc1 >> 2) + (acc2 >> 4) - (acc3 >> 6) minus the activation sum over
    the inputs that met planes 0..2 must be the plain ternary dot product (arithmetic shifts of exact multiples)."""
    rng = np.random.default_rng(2)
    for _ in range(50):
        t = rng.integers(-1, 2, size=(4, 64))                 # plane i, 64 weights each
        x = rng.integers(-127, 128, size=(4, 64))
        acc = []
        for i in range(3):
            acc.append(int(((t[i] + 1) * 4 ** i * x[i]).sum()))
        field = (t[3] + 1) << 6                                # 0x00, 0x40, 0x80 in the top two bits
        signed = ((field ^ 0x40) + 128) % 256 - 128            # as signed bytes: +64, 0, -64
        assert set(np.unique(signed)).issubset({64, 0, -64}) and np.array_equal(signed, -t[3] * 64)
        acc.append(int((signed * x[3]).sum()))
        folded = acc[0] + (acc[1] >> 2) + (acc[2] >> 4) - (acc[3] >> 6)
        want = int((t * x).sum())
        assert folded - int(x[:3].sum()) == want


def test_row_sum_correction_of_the_tensor_core_kernels_is_exact():
    """GEMM kernels multiply u8 codes t + 1 and subtract the int8 row sum: sum((t+1) x) - sum(x) = sum(t x), and
    128 * 127 * K stays inside int32 for the largest supported K."""
    rng = np.random.default_rng(3)
    t = rng.integers(-1, 2, size=(5, 777))
    x = rng.integers(-127, 128, size=(3, 777))
    acc = x @ (t + 1).T - x.sum(axis=1, keepdims=True)
    assert np.array_equal(acc, x @ t.T)
    assert 2 * 127 * 131072 < 2 ** 31                          # worst accumulator before the correction


def test_k_split_of_the_narrow_batch_gemm_covers_every_block_once():
    """Narrow-batch GEMM: CTA r of a cluster of s contracts K blocks [r*KB/s, (r+1)*KB/s) and finishes columns
    [r*256/s, (r+1)*256/s) of the tile; every 32-column chunk of an accumulator goes to exactly one owner."""
    for kb_total in (1, 2, 3, 8, 31, 32, 86, 224):
        for s in (2, 4, 8):
            if s > kb_total:
                continue
            covered = []
            for r in range(s):
                lo, hi = r * kb_total // s, (r + 1) * kb_total // s
                assert hi > lo                                   # no idle CTA when s <= number of blocks
                covered += list(range(lo, hi))
            assert covered == list(range(kb_total))
    for s in (2, 4, 8):
        cols_own = 256 // s
        owners = [(c0 // cols_own, c0 % cols_own) for c0 in range(0, 256, 32)]
        assert sorted(set(o for o, _ in owners)) == list(range(s))
        assert all(off + 32 <= cols_own for _, off in owners)


def test_a_published_row_maximum_is_the_maximum_the_consumer_would_reduce():
    """Chained decode layers: the producer publishes max |y as stored| by an atomic maximum on float BIT PATTERNS,
    the consumer turns the winning pattern back into a float and derives its scale from it.  For the result to be
    bit-identical to the consumer reducing the row itself, (1) non-negative floats must order like their unsigned
    bit patterns, infinities included, (2) the maximum must be taken over the values after rounding to the storage
    type, and (3) NaN must be dropped the way fmaxf drops it.  Checked here with numpy on bf16 / fp16 / fp32 storage."""
    import torch

    rng = np.random.default_rng(5)
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for trial in range(20):
            y = torch.from_numpy((rng.standard_normal(300) * 10.0 ** rng.integers(-6, 5)).astype(np.float32))
            if trial % 5 == 1:
                y[7] = float("inf")
            if trial % 5 == 2:
                y[3], y[11] = float("nan"), -0.0
            stored = y.to(dtype).float()                               # what the consumer reads back
            clean = torch.where(torch.isnan(stored), torch.zeros_like(stored), stored.abs())
            want = float(clean.max())                                  # fmaxf-style reduction: NaN dropped
            bits = clean.numpy().view(np.uint32)
            got = np.array([bits.max()], dtype=np.uint32).view(np.float32)[0]
            assert got == want or (np.isinf(got) and np.isinf(want))
            order = np.argsort(clean.numpy(), kind="stable")
            assert np.all(np.diff(bits[order].astype(np.int64)) >= 0)  # value order == bit-pattern order
    # spread over slots: the row's value is the maximum of its slots, zero slots are neutral
    slots = np.zeros(8, dtype=np.uint32)
    for v in (0.5, 3.25, 1e-9):
        s = rng.integers(0, 8)
        slots[s] = max(slots[s], np.array([v], np.float32).view(np.uint32)[0])
    assert slots.max().view(np.float32) == np.float32(3.25)
