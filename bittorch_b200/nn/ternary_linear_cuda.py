"""Autograd function and module for the CUDA ternary linear forward.

Counterpart of the reference's ``bittorch/nn/ternary_linear_cuda.py``.  Forward: one
fused quantize+pack kernel over the master weight, then the packed integer path
(per-token int8 activations; GEMV for small batches, tcgen05 GEMM above) or, with
``BITTORCH_B200_ACT=float``, the reference's fp32-accumulate arithmetic.  Backward is the
reference's straight-through estimator with torch matmuls (:73-111 there); it keeps the
2-bit weights instead of an fp32 effective weight and rebuilds the latter on demand.
"""

from __future__ import annotations

from typing import Any, Optional

import torch
import torch.nn as nn
from torch import Tensor

from .._ext import require_ext


class PackedWeightCache:
    """Packed/tiled copies of a master weight, valid while the parameter is unchanged.

    Keyed on the parameter's storage address, in-place version counter, dtype and
    threshold: an optimizer step bumps the version and the next forward re-quantizes.
    """

    def __init__(self) -> None:
        self.key = None
        self.packed_T: Optional[Tensor] = None
        self.tiled: Optional[Tensor] = None
        self.scale: Optional[Tensor] = None   # float32 [N]

    def lookup(self, weight: Tensor, threshold_factor: float):
        key = (weight.data_ptr(), weight._version, weight.dtype, tuple(weight.shape), float(threshold_factor))
        return key, (self.key == key)


def usable_cache(cache: Optional[PackedWeightCache]) -> Optional[PackedWeightCache]:
    """The cache is consulted only for inference-style calls (grad mode off, no autocast):
    training forwards re-quantize every time, like the reference, so an update made
    through ``weight.data`` (which does not bump the version counter) is never missed
    while training, and autocast's temporary fp16 copies are never mistaken for the
    parameter."""
    if cache is None or torch.is_grad_enabled() or torch.is_autocast_enabled("cuda"):
        return None
    return cache


def _quantized(weight: Tensor, threshold_factor: float, cache: Optional[PackedWeightCache]):
    C = require_ext()
    if cache is not None:
        key, hit = cache.lookup(weight, threshold_factor)
        if hit:
            return cache.packed_T, cache.tiled, cache.scale
    out = C.quantize_pack(weight, threshold_factor, want_packed=True)
    packed_T, scale = out["packed_T"], out["scale"]
    tiled = C.retile(packed_T, weight.shape[1])
    if cache is not None:
        cache.key, cache.packed_T, cache.tiled, cache.scale = key, packed_T, tiled, scale
    return packed_T, tiled, scale


class TernaryLinearCUDAFunction(torch.autograd.Function):
    """y = x @ (ternarize(weight) * scale).T + bias with a CUDA forward
    (bittorch/nn/ternary_linear_cuda.py:23-111)."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx: Any, x: Tensor, weight: Tensor, bias: Optional[Tensor], threshold_factor: float,
                per_channel: bool, cache: Optional[PackedWeightCache] = None) -> Tensor:
        C = require_ext()
        if not per_channel:
            # The reference hands a 0-dim scale to its extension, which rejects it
            # (csrc/core/dispatch.cpp:62); only per-channel scaling is a working configuration.
            raise RuntimeError("scale must be 1D [N]")
        if not (x.is_cuda and weight.is_cuda):
            raise RuntimeError("All tensors must be CUDA")
        if x.numel() == 0:
            raise RuntimeError("X is empty")
        if x.shape[-1] != weight.shape[1]:
            raise RuntimeError("input K doesn't match weight K")
        n, k = weight.shape
        packed_T, tiled, scale = _quantized(weight.detach(), threshold_factor, cache)
        b32 = None if bias is None else bias.detach().to(torch.float32).contiguous()
        x2d = x.detach().contiguous().reshape(-1, k)
        if C.activation_mode() == "float":
            y2d = C.ternary_linear_packed_forward(x2d, packed_T, scale, b32, k)
        else:
            y2d = C.int8_linear_tiled(x2d, tiled, k, n, scale, b32)
        ctx.save_for_backward(x, packed_T, scale)
        ctx.has_bias = bias is not None
        ctx.in_features = k
        ctx.weight_dtype = weight.dtype
        return y2d.reshape(*x.shape[:-1], n)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output: Tensor):
        C = require_ext()
        x, packed_T, scale = ctx.saved_tensors
        grad_x = grad_weight = grad_bias = None
        x2d = x.reshape(-1, x.shape[-1])
        g2d = grad_output.reshape(-1, grad_output.shape[-1])
        scale_c = scale.to(g2d.dtype)
        if ctx.needs_input_grad[0]:
            w_eff = C.unpack_codes(packed_T, ctx.in_features).to(g2d.dtype) * scale_c.unsqueeze(1)
            grad_x = (g2d @ w_eff).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            # d(w_eff)/d(weight) = scale under the straight-through estimator
            grad_weight = ((g2d.T @ x2d.to(g2d.dtype)) * scale_c.unsqueeze(1)).to(ctx.weight_dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_bias = g2d.sum(dim=0)
        return grad_x, grad_weight, grad_bias, None, None, None


class TernaryLinearCUDA(nn.Module):
    """Linear layer with ternary weights that always runs the CUDA forward
    (bittorch/nn/ternary_linear_cuda.py:114-228)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, threshold_factor: float = 0.05,
                 per_channel: bool = True) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.threshold_factor = threshold_factor
        self.per_channel = per_channel
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        self._cache = PackedWeightCache()
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=5**0.5)
        if self.bias is not None:
            fan_in = self.in_features
            bound = 1 / (fan_in**0.5) if fan_in > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, x: Tensor) -> Tensor:
        if not x.is_cuda:
            raise RuntimeError("TernaryLinearCUDA requires CUDA tensors. Use TernaryLinear for CPU.")
        return TernaryLinearCUDAFunction.apply(x, self.weight, self.bias, self.threshold_factor, self.per_channel,
                                               usable_cache(self._cache))

    def get_quantized_weight(self):
        from ..quant.ternary import ternary_quantize

        with torch.no_grad():
            return ternary_quantize(self.weight, self.threshold_factor, self.per_channel)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"threshold_factor={self.threshold_factor}, per_channel={self.per_channel}")
