"""Functional packed ternary linear (bittorch/ops/ternary_linear_packed.py)."""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .._ext import require_ext


def ternary_linear_packed_forward(x: Tensor, w_packed_T: Tensor, scale: Tensor, in_features: int,
                                  bias: Optional[Tensor] = None) -> Tensor:
    """Y = X @ (W * scale).T + bias from the public packed buffer uint8 [ceil(K/4), N]
    (bittorch/ops/ternary_linear_packed.py:21-77).

    Activations are quantized per token to int8 and contracted in integers unless
    ``BITTORCH_B200_ACT=float`` selects the reference's fp32-accumulate arithmetic.
    """
    C = require_ext()
    return C.ternary_linear_packed_forward(x, w_packed_T, scale, bias, in_features)


def has_packed_cuda_support() -> bool:
    """True when the library is built and a CUDA device is present
    (bittorch/ops/ternary_linear_packed.py:80-90)."""
    try:
        require_ext()
    except RuntimeError:
        return False
    return torch.cuda.is_available()
