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


def content_fingerprint(*tensors: Tensor) -> tuple:
    """A few numbers computed from about a thousand evenly spaced elements of each tensor, read back to the host
    (one small device-to-host copy, which synchronises the stream).

    The caches of this package key on a tensor's address and in-place version counter; a write through ``.data``
    (``p.data.copy_(w)``, the usual way of loading weights by hand) changes neither, so the key is completed with
    this content check.  It sees every bulk update (copies, scalings, optimizer steps); a write that touches only a
    few elements can fall between the samples - after such a write call ``invalidate_cache()`` on the module.
    """
    parts = []
    for t in tensors:
        flat = t.detach().reshape(-1)
        step = max(1, flat.numel() // 1024)
        sample = flat[::step][:1024].to(torch.float64)
        weights = torch.arange(1, sample.numel() + 1, dtype=torch.float64, device=sample.device)
        parts += [sample.sum(), (sample * weights).sum()]      # the second sum also sees permutations
    return tuple(torch.stack(parts).tolist())


def capturing() -> bool:
    """True while the current CUDA stream is being captured into a graph (no host read-back possible)."""
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


class PackedWeightCache:
    """Packed/tiled copies of a master weight, valid while the parameter is unchanged.

    Keyed on the parameter's storage address, in-place version counter, dtype and threshold (an optimizer step
    bumps the version and the next forward re-quantizes) plus ``content_fingerprint`` of the weight, which catches
    writes through ``.data`` that the version counter misses.  The fingerprint costs a host synchronisation per
    forward; it is skipped during CUDA-graph capture (captured weights must not change anyway) and can be switched
    off with ``verify = False`` once a model's weights are final.
    """

    verify = True

    def __init__(self) -> None:
        self.key = None
        self.fingerprint = None
        self.packed_T: Optional[Tensor] = None
        self.tiled: Optional[Tensor] = None
        self.scale: Optional[Tensor] = None   # float32 [N]

    def invalidate(self) -> None:
        self.key = None

    def lookup(self, weight: Tensor, threshold_factor: float):
        """Returns (key, fingerprint, hit)."""
        key = (weight.data_ptr(), weight._version, weight.dtype, tuple(weight.shape), float(threshold_factor))
        check = self.verify and not capturing()
        fp = content_fingerprint(weight) if check else None
        hit = self.key == key and (not check or fp == self.fingerprint)
        return key, fp, hit


def usable_cache(cache: Optional[PackedWeightCache]) -> Optional[PackedWeightCache]:
    """The cache is consulted only for inference-style calls (grad mode off, no autocast): training forwards
    re-quantize every time, like the reference, and autocast's temporary fp16 copies are never mistaken for the
    parameter."""
    if cache is None or torch.is_grad_enabled() or torch.is_autocast_enabled("cuda"):
        return None
    return cache


def verify_weight_contents(module: nn.Module, enabled: bool) -> int:
    """Switches the per-forward content check of every ternary layer below ``module`` on or off (the fingerprint
    behind ``PackedWeightCache.verify`` and ``TernaryLinearInference.verify_buffers``).  Off, a forward compares
    addresses and version counters only and does not synchronise with the host: for models whose weights are final
    and whose eager call rate matters.  A later write through ``.data`` then needs ``invalidate_cache()``.
    Returns the number of layers switched."""
    switched = 0
    for m in module.modules():
        cache = getattr(m, "_cache", None)
        if isinstance(cache, PackedWeightCache):
            cache.verify = enabled
            switched += 1
        elif hasattr(type(m), "verify_buffers"):
            m.verify_buffers = enabled
            switched += 1
    return switched


def _quantized(weight: Tensor, threshold_factor: float, cache: Optional[PackedWeightCache]):
    """(packed_T, tiled, scale float32, fresh): ``fresh`` says that the buffers were written by kernels enqueued just
    now, so the first kernel that reads them must be launched stream-ordered."""
    C = require_ext()
    key = fp = None
    if cache is not None:
        key, fp, hit = cache.lookup(weight, threshold_factor)
        if hit:
            return cache.packed_T, cache.tiled, cache.scale, False
    if weight.dtype == torch.float64:
        # float64 masters (gradient checks): the reference's own expression in float64
        # (bittorch/quant/ternary.py:122-142), then the packer kernel
        mag = weight.abs()
        scale64 = mag.max(dim=1, keepdim=True).values.clamp(min=1e-8)
        tern = torch.where(mag > threshold_factor * scale64, torch.sign(weight), torch.zeros_like(weight))
        packed_T, scale = C.pack_codes(tern.to(torch.int8)), scale64.squeeze(1).to(torch.float32)
    else:
        out = C.quantize_pack(weight, threshold_factor, want_packed=True)
        packed_T, scale = out["packed_T"], out["scale"]
    tiled = C.retile(packed_T, weight.shape[1])
    if cache is not None:
        if fp is None and cache.verify and not capturing():
            fp = content_fingerprint(weight)
        cache.key, cache.fingerprint, cache.packed_T, cache.tiled, cache.scale = key, fp, packed_T, tiled, scale
    return packed_T, tiled, scale, True


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
        packed_T, tiled, scale, fresh = _quantized(weight.detach(), threshold_factor, cache)
        b32 = None if bias is None else bias.detach().to(torch.float32).contiguous()
        x2d = x.detach().contiguous().reshape(-1, k)
        fresh = fresh or (b32 is not None and b32.data_ptr() != bias.data_ptr())     # a float32 copy made just now
        if C.activation_mode() == "float" or x2d.dtype == torch.float64:      # float64 has no int8 path
            if C.float_linear_tiled_ok(x2d.shape[0], k, x2d.dtype):
                y2d = C.float_linear_tiled(x2d, tiled, k, n, scale, b32, fresh_weights=fresh)
            else:
                y2d = C.ternary_linear_packed_forward(x2d, packed_T, scale, b32, k)
        else:
            y2d = C.int8_linear_tiled(x2d, tiled, k, n, scale, b32, fresh_weights=fresh)
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

    def invalidate_cache(self) -> None:
        """Forget the packed copy of the weight: the next forward re-quantizes.  Needed only after an in-place
        write through ``weight.data`` that changes so few elements that the sampled content check can miss it."""
        self._cache.invalidate()

    def _load_from_state_dict(self, *args, **kwargs):
        self._cache.invalidate()
        return super()._load_from_state_dict(*args, **kwargs)

    def get_quantized_weight(self):
        from ..quant.ternary import ternary_quantize

        with torch.no_grad():
            return ternary_quantize(self.weight, self.threshold_factor, self.per_channel)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"threshold_factor={self.threshold_factor}, per_channel={self.per_channel}")
