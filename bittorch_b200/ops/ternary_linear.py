"""Functional ternary linear on unpacked int8 weights (bittorch/ops/ternary_linear.py)."""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .._ext import require_ext
from ..quant.ternary import ternary_quantize


def ternary_linear_forward_cuda(x: Tensor, w_tern: Tensor, scale: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """Y = X @ (W_tern * scale).T + bias, W_tern int8 [N,K], fp32 accumulation
    (bittorch/ops/ternary_linear.py:15-49).  Raises RuntimeError for non-CUDA tensors."""
    C = require_ext()
    return C.ternary_linear_forward(x.contiguous(), w_tern.contiguous(), scale, bias)


def ternary_linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, threshold_factor: float = 0.05,
                   per_channel: bool = True) -> Tensor:
    """Quantize ``weight`` on the fly, then ``ternary_linear_forward_cuda``
    (bittorch/ops/ternary_linear.py:52-87)."""
    C = require_ext()
    if not per_channel:
        w_tern, scale = ternary_quantize(weight, threshold_factor, per_channel=False)
        return ternary_linear_forward_cuda(x, w_tern.to(torch.int8), scale.expand(weight.shape[0]), bias)
    out = C.quantize_pack(weight, threshold_factor, want_packed=False, want_codes=True)
    return ternary_linear_forward_cuda(x, out["codes"], out["scale"], bias)
