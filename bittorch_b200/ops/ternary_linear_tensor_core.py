"""Functional tensor-core ternary linear (bittorch/ops/ternary_linear_tensor_core.py)."""

from __future__ import annotations

from typing import Optional

from torch import Tensor

from .._ext import require_ext


def ternary_linear_tensor_core_forward(x: Tensor, w_packed_T: Tensor, scale: Tensor, in_features: int,
                                       bias: Optional[Tensor] = None, version: int = 1) -> Tensor:
    """2-D input only.  ``version=1``: float compute; ``version=2``: per-token int8
    activations on the tensor cores (bittorch/ops/ternary_linear_tensor_core.py:17-46)."""
    C = require_ext()
    return C.ternary_linear_tensor_core_forward(x, w_packed_T, scale, bias, in_features, version)
