"""Weight ternarizer on the GPU.

Same functions as the reference's ``bittorch/quant/ternary.py``; the arithmetic
(:122-142 there) runs in one fused CUDA kernel (``bt_quantize_pack``) instead of six
ATen passes.  Tensors must be CUDA tensors.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
from torch import Tensor

from .._ext import require_cuda_tensor, require_ext


def ternary_quantize(weight: Tensor, threshold_factor: float = 0.05, per_channel: bool = True) -> Tuple[Tensor, Tensor]:
    """Quantize weights to {-1, 0, +1} (bittorch/quant/ternary.py:100-150).

    Returns ``(w_tern, scale)``: ``w_tern`` has the shape and dtype of ``weight``;
    ``scale`` is ``(out_features,)`` for ``per_channel`` and 0-dim otherwise.
    """
    require_cuda_tensor(weight, "weight")
    C = require_ext()
    if weight.dim() != 2:
        raise ValueError(f"Expected 2D tensor, got {weight.dim()}D")
    w = weight.detach()
    if per_channel:
        out = C.quantize_pack(w, threshold_factor, want_packed=False, want_tern=True)
        return out["tern"], out["scale"].to(w.dtype)
    flat = w.contiguous().reshape(1, -1)        # one global scale = one long row
    out = C.quantize_pack(flat, threshold_factor, want_packed=False, want_tern=True)
    return out["tern"].reshape(w.shape), out["scale"].to(w.dtype).reshape(())


def ternary_quantize_ste(weight: Tensor, threshold_factor: float = 0.05, per_channel: bool = True) -> Tuple[Tensor, Tensor]:
    """Quantize with a straight-through estimator (bittorch/quant/ternary.py:153-195):
    forward value = ternary codes, gradient flows to ``weight`` as identity; scale detached."""
    w_tern, scale = ternary_quantize(weight, threshold_factor, per_channel)
    return w_tern.detach() - weight.detach() + weight, scale.detach()


def dequantize_ternary(w_tern: Tensor, scale: Tensor) -> Tensor:
    """``w_tern * scale[:, None]`` (bittorch/quant/ternary.py:198-209)."""
    return w_tern * scale.unsqueeze(1)


@dataclass
class TernaryQuantConfig:
    """Configuration holder (bittorch/quant/ternary.py:16-45)."""

    threshold_factor: float = 0.05
    per_channel: bool = True

    def __post_init__(self) -> None:
        if self.threshold_factor < 0:
            raise ValueError(f"threshold_factor must be non-negative, got {self.threshold_factor}")


class TernaryQuantizer:
    """Class wrapper over the functions above (bittorch/quant/ternary.py:48-97)."""

    def __init__(self, config: TernaryQuantConfig | None = None) -> None:
        self._config = config if config is not None else TernaryQuantConfig()

    @property
    def config(self) -> TernaryQuantConfig:
        return self._config

    def quantize(self, weight: Tensor) -> Tuple[Tensor, Tensor]:
        return ternary_quantize(weight, self._config.threshold_factor, self._config.per_channel)

    def quantize_ste(self, weight: Tensor) -> Tuple[Tensor, Tensor]:
        return ternary_quantize_ste(weight, self._config.threshold_factor, self._config.per_channel)

    def dequantize(self, w_tern: Tensor, scale: Tensor) -> Tensor:
        return dequantize_ternary(w_tern, scale)
