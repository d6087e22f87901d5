"""TernaryLinear — drop-in for ``bittorch.nn.TernaryLinear`` (bittorch/nn/ternary_linear.py).

Same constructor, attributes, backend names and error messages.  ``backend="cuda"`` and
``backend="auto"`` run the B200 kernels and never fall back: ``auto`` with CPU tensors or
without the built library raises.  ``backend="python"`` is the explicitly requested eager
arithmetic of the reference (:196-213 there), written in torch ops; it is the only path
that accepts CPU tensors.
"""

from __future__ import annotations

import warnings
from typing import Literal, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

BackendType = Literal["auto", "cuda", "python"]


def _cuda_kernel_available() -> bool:
    """True when the CUDA library is built (bittorch/nn/ternary_linear.py:20-26)."""
    try:
        from .. import _C
        return hasattr(_C, "ternary_linear_forward")
    except ImportError:
        return False


def _eager_ternarize(weight: Tensor, threshold_factor: float, per_channel: bool):
    """Torch-op arithmetic of bittorch/quant/ternary.py:122-150, for backend="python" only."""
    mag = weight.abs()
    if per_channel:
        scale = mag.max(dim=1, keepdim=True).values.clamp(min=1e-8)
    else:
        scale = mag.max().unsqueeze(0).clamp(min=1e-8)
    tern = torch.where(mag > threshold_factor * scale, torch.sign(weight), torch.zeros_like(weight))
    return tern, (scale.squeeze(1) if per_channel else scale.squeeze(0))


class TernaryLinear(nn.Module):
    """Linear layer whose weights are ternarized ({-1,0,+1} x per-channel scale) on every
    forward, with straight-through gradients to full-precision master weights.

    Args mirror bittorch/nn/ternary_linear.py:91-101: ``in_features, out_features, bias,
    threshold_factor, per_channel, quantize, backend, use_cuda_kernel`` (deprecated).
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, threshold_factor: float = 0.05,
                 per_channel: bool = True, quantize: bool = True, backend: BackendType = "auto",
                 use_cuda_kernel: Optional[bool] = None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.threshold_factor = threshold_factor
        self.per_channel = per_channel
        self.quantize = quantize
        if use_cuda_kernel is not None:
            warnings.warn("use_cuda_kernel is deprecated, use backend='auto'|'cuda'|'python' instead",
                          DeprecationWarning, stacklevel=2)
            self.backend = "auto" if use_cuda_kernel else "python"
        else:
            if backend not in ("auto", "cuda", "python"):
                raise ValueError(f"backend must be 'auto', 'cuda', or 'python', got {backend!r}")
            self.backend = backend
        self.use_cuda_kernel = self.backend != "python"
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        from .ternary_linear_cuda import PackedWeightCache
        self._cache = PackedWeightCache()
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Kaiming-uniform(a=sqrt 5) weights, U(+-1/sqrt(fan_in)) bias, like nn.Linear."""
        nn.init.kaiming_uniform_(self.weight, a=5**0.5)
        if self.bias is not None:
            fan_in = self.in_features
            bound = 1 / (fan_in**0.5) if fan_in > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)

    def _should_use_cuda_kernel(self, x: Tensor) -> bool:
        if self.backend == "python":
            return False
        on_cuda = x.is_cuda and self.weight.is_cuda
        available = _cuda_kernel_available()
        if self.backend == "cuda":
            if not on_cuda:
                raise RuntimeError("backend='cuda' requires input and weights on CUDA device")
            if not available:
                raise RuntimeError("backend='cuda' requires CUDA extension to be built. "
                                   "Rebuild with CUDA support or use backend='python'")
            return True
        # backend == "auto": the CUDA kernels or an error, never a silent eager fallback
        if not on_cuda:
            raise RuntimeError("bittorch_b200 has no CPU path: backend='auto' requires input and weights on CUDA "
                               "device (use backend='python' for the eager arithmetic)")
        if not available:
            raise RuntimeError("backend='auto' requires CUDA extension to be built "
                               "(python -m bittorch_b200._build) or use backend='python'")
        return True

    def forward(self, x: Tensor) -> Tensor:
        """x: (*, in_features) -> (*, out_features)."""
        if not self.quantize:
            return F.linear(x, self.weight, self.bias)   # debug mode == nn.Linear
        if self._should_use_cuda_kernel(x):
            from .ternary_linear_cuda import TernaryLinearCUDAFunction, usable_cache
            return TernaryLinearCUDAFunction.apply(x, self.weight, self.bias, self.threshold_factor,
                                                   self.per_channel, usable_cache(self._cache))
        tern, scale = _eager_ternarize(self.weight, self.threshold_factor, self.per_channel)
        w_q = tern.detach() - self.weight.detach() + self.weight          # straight-through estimator
        w_effective = (w_q * scale.detach().unsqueeze(1)).to(x.dtype)
        bias = self.bias.to(x.dtype) if self.bias is not None else None
        return F.linear(x, w_effective, bias)

    def invalidate_cache(self) -> None:
        """Forget the packed copy of the weight that inference-mode forwards reuse: the next forward re-quantizes.
        Needed only after an in-place write through ``weight.data`` that changes so few elements that the sampled
        content check can miss it (``nn/ternary_linear_cuda.py``: ``content_fingerprint``)."""
        self._cache.invalidate()

    def _load_from_state_dict(self, *args, **kwargs):
        self._cache.invalidate()
        return super()._load_from_state_dict(*args, **kwargs)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"threshold_factor={self.threshold_factor}, per_channel={self.per_channel}, "
                f"quantize={self.quantize}, backend={self.backend!r}")

    def get_quantized_weight(self) -> tuple[Tensor, Tensor]:
        """(w_tern, scale) of the current master weights (bittorch/nn/ternary_linear.py:227-242):
        ``w_tern`` is a tensor of -1/0/+1 in the weight's dtype, ``scale`` is per channel."""
        with torch.no_grad():
            if self.backend == "python":
                return _eager_ternarize(self.weight, self.threshold_factor, self.per_channel)
            from ..quant.ternary import ternary_quantize
            return ternary_quantize(self.weight, self.threshold_factor, self.per_channel)
