"""Generate the golden vectors in this directory by running the reference itself.

Run where the reference checkout is mounted (it is imported, never copied):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

Everything is computed on CPU with the reference's own public functions
(``bittorch.quant.ternary_quantize``, ``pack_ternary[_transposed]``,
``unpack_ternary[_transposed]``, ``bittorch.nn.TernaryLinear(backend="python")``,
``TernaryLinearInference``) and stored as small ``.npz`` files.  bfloat16 tensors
are stored widened to float32 (exact) because numpy has no bfloat16.
"""

from __future__ import annotations

import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BITTORCH_REFERENCE", "")
if not REF:
    raise SystemExit("usage: make_golden.py <path to a checkout of the reference> (or set BITTORCH_REFERENCE)")
sys.path.insert(0, REF)
warnings.filterwarnings("ignore")

import bittorch  # noqa: E402  (the reference)
from bittorch.nn import TernaryLinear, TernaryLinearInference  # noqa: E402
from bittorch.quant import (  # noqa: E402
    pack_ternary,
    pack_ternary_transposed,
    ternary_quantize,
    unpack_ternary,
    unpack_ternary_transposed,
)

assert os.path.realpath(os.path.dirname(bittorch.__file__)).startswith(os.path.realpath(REF))


def f32(t):
    return t.detach().to(torch.float32).contiguous().numpy()


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KiB")


def quant_case(w, tf=0.05):
    t, s = ternary_quantize(w, threshold_factor=tf)
    p, k = pack_ternary(t)
    pt, _ = pack_ternary_transposed(t)
    assert torch.equal(unpack_ternary(p, k), t.to(torch.int8))
    assert torch.equal(unpack_ternary_transposed(pt, k), t.to(torch.int8))
    return {
        "w": f32(w),
        "tf": np.float64(tf),
        "codes": t.to(torch.int8).numpy(),
        "scale": f32(s),
        "packed": p.numpy(),
        "packed_T": pt.numpy(),
    }


def main():
    torch.set_num_threads(1)

    # ---- known-answer tests of the reference's own test-suite -------------------
    kat = {}
    cases = {
        "single": (torch.tensor([[2.5]]), 0.05),                               # tests/test_ternary_quant.py:171-178
        "half_ones": (torch.ones(4, 8) * 0.5, 0.05),                           # :238-245
        "rows": (torch.tensor([[1.0, 2.0, 3.0, 4.0], [0.1, 0.2, 0.3, 0.4], [10.0, 20.0, 30.0, 40.0]]), 0.05),  # :247-258
        "docstring": (torch.tensor([[1.0, -1.0, 0.0, 1.0], [0.0, 1.0, 1.0, -1.0]]), 0.05),  # quant/ternary_packed.py:91-94
        "all_pos": (torch.ones(4, 8), 0.05),                                   # tests/test_packed_ternary.py:72-79 (byte 85)
        "all_neg": (-torch.ones(4, 8), 0.05),                                  # :81-88 (byte 170)
        "zeros": (torch.zeros(3, 5), 0.05),                                    # clamp(min=1e-8) branch
        "k6": (torch.tensor([[1.0, -1.0, 0.0, 1.0, -1.0, 1.0], [0.0, 0.0, 1.0, -1.0, 1.0, 0.0]]), 0.05),  # :44-54 padding
        "tiny": (torch.full((2, 4), 1e-10), 0.05),                              # below the 1e-8 floor
        "with_nan": (torch.tensor([[1.0, float("nan"), -2.0, 0.5], [1.0, 2.0, -3.0, 0.01]]), 0.05),
        "with_inf": (torch.tensor([[1.0, float("inf"), -2.0, 0.5]]), 0.05),
    }
    g = torch.Generator().manual_seed(7)
    cases["thr_one"] = (torch.randn(32, 64, generator=g), 1.0)                 # tests/test_ternary_quant.py:191-197
    cases["thr_zero"] = (torch.randn(32, 64, generator=g), 0.0)                # :180-189
    for name, (w, tf) in cases.items():
        for key, val in quant_case(w, tf).items():
            kat[f"{name}.{key}"] = val
    save("kat_quant_pack", **kat)

    # ---- config 1: TernaryLinear(512 -> 256, bias, 0.05), seed 0, python backend ----
    torch.manual_seed(0)
    layer = TernaryLinear(512, 256, bias=True, threshold_factor=0.05, backend="python")
    x = torch.randn(32, 512)
    with torch.no_grad():
        y = layer(x)
    qc = quant_case(layer.weight.detach(), 0.05)
    t2, s2 = layer.get_quantized_weight()
    assert np.array_equal(t2.to(torch.int8).numpy(), qc["codes"]) and np.array_equal(f32(s2), qc["scale"])
    infer = TernaryLinearInference.from_unpacked(t2, s2, layer.bias.detach())
    with torch.no_grad():
        y_inf = infer(x)
    save("c1_linear_512x256", x=f32(x), bias=f32(layer.bias), y=f32(y), y_infer=f32(y_inf), **qc)

    # ---- ragged shapes: quantize + pack + float forward ---------------------------
    ragged = {}
    shapes = [(1, 1, 1), (7, 33, 17), (3, 5, 2), (2, 6, 9), (4, 7, 31), (5, 9, 64), (1, 13, 67),
              (17, 17, 5), (8, 31, 33), (16, 65, 129), (17, 123, 67), (2, 100, 300)]   # (M, K, N)
    for i, (m, k, n) in enumerate(shapes):
        gg = torch.Generator().manual_seed([0, 42, 123, 999][i % 4])
        w = torch.randn(n, k, generator=gg)
        b = torch.randn(n, generator=gg)
        xx = torch.randn(m, k, generator=gg)
        layer = TernaryLinear(k, n, bias=True, backend="python")
        with torch.no_grad():
            layer.weight.copy_(w)
            layer.bias.copy_(b)
            yy = layer(xx)
        qc = quant_case(w, 0.05)
        tag = f"m{m}_k{k}_n{n}"
        for key, val in qc.items():
            ragged[f"{tag}.{key}"] = val
        ragged[f"{tag}.x"] = f32(xx)
        ragged[f"{tag}.bias"] = f32(b)
        ragged[f"{tag}.y"] = f32(yy)
    ragged["shapes"] = np.array(shapes, dtype=np.int64)
    save("ragged_forward", **ragged)

    # ---- half-precision master weights (scale/threshold arithmetic in the storage type) ----
    half = {}
    for dt_name, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        for j, (n, k) in enumerate([(8, 64), (33, 70), (5, 3)]):
            gg = torch.Generator().manual_seed(100 + j)
            w = (torch.randn(n, k, generator=gg) * (0.02 if j == 1 else 1.0)).to(dt)
            if j == 2:
                w[0].zero_()                                                   # exercises the 1e-8 floor in half types
            t, s = ternary_quantize(w, threshold_factor=0.05)
            pt, _ = pack_ternary_transposed(t)
            tag = f"{dt_name}_{n}x{k}"
            half[f"{tag}.w"] = f32(w)
            half[f"{tag}.codes"] = t.to(torch.int8).numpy()
            half[f"{tag}.scale"] = f32(s)
            half[f"{tag}.packed_T"] = pt.numpy()
    save("half_quant", **half)

    # ---- random round trips with the reference's habitual seeds --------------------
    rt = {}
    for seed in (0, 42, 123, 999):                                            # tests/test_packed_ternary.py:106-113
        torch.manual_seed(seed)
        t = torch.randint(-1, 2, (64, 128)).float()
        p, k = pack_ternary(t)
        pt, _ = pack_ternary_transposed(t)
        rt[f"s{seed}.codes"] = t.to(torch.int8).numpy()
        rt[f"s{seed}.packed"] = p.numpy()
        rt[f"s{seed}.packed_T"] = pt.numpy()
    # reserved code 3 must decode to 0 (quant/ternary_packed.py:112-115)
    raw = torch.arange(256, dtype=torch.uint8).reshape(1, 256)
    rt["all_bytes.packed"] = raw.numpy()
    rt["all_bytes.codes"] = unpack_ternary(raw, 1024).numpy()
    save("pack_roundtrip", **rt)

    # ---- packed inference, bf16 / fp16 activations on the CPU fallback --------------
    pi = {}
    gg = torch.Generator().manual_seed(5)
    w = torch.randn(96, 200, generator=gg)
    t, s = ternary_quantize(w)
    b = torch.randn(96, generator=gg)
    infer = TernaryLinearInference.from_unpacked(t, s, b)
    xx = torch.randn(6, 200, generator=gg)
    with torch.no_grad():
        pi["y_f32"] = f32(infer(xx))
    pi["x"] = f32(xx)
    pi["packed_T"] = infer.weight_packed.numpy()
    pi["scale"] = f32(s)
    pi["bias"] = f32(b)
    pi["codes"] = t.to(torch.int8).numpy()
    save("packed_infer_96x200", **pi)


if __name__ == "__main__":
    main()
