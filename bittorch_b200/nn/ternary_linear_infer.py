"""TernaryLinearInference — packed-weight inference module
(bittorch/nn/ternary_linear_infer.py).

Buffers keep the reference's names, dtypes and shapes (``weight_packed`` uint8
[ceil(K/4), N], ``scale`` [N], ``bias`` [N]) so its checkpoints load unchanged.  The
forward runs on a privately re-tiled copy of ``weight_packed`` that is rebuilt whenever
the buffer changes and is never serialized.  ``compact()`` drops the public buffer from the
device once the tiled copy exists (one copy of the weights, 2 bits each); ``state_dict()`` then
rebuilds ``weight_packed`` from the tiled copy, byte for byte, so checkpoints do not change.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from .._ext import require_cuda_tensor, require_ext
from ..quant.ternary_packed import pack_ternary_transposed


class TernaryLinearInference(nn.Module):
    """Inference-only linear layer on 2-bit packed ternary weights (no master weights,
    no autograd).  Constructor as in bittorch/nn/ternary_linear_infer.py:46-76."""

    def __init__(self, in_features: int, out_features: int, weight_packed: Tensor, scale: Tensor,
                 bias: Optional[Tensor] = None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("weight_packed", weight_packed)
        self.register_buffer("scale", scale)
        self.register_buffer("bias", bias if bias is not None else None)
        self.requires_grad_(False)
        self._derived_key = None
        self._tiled: Optional[Tensor] = None
        self._scale32: Optional[Tensor] = None
        self._bias32: Optional[Tensor] = None
        self._compact = False                                  # True: weight_packed is an empty placeholder
        self._register_state_dict_hook(_packed_into_state_dict)

    # Check the buffers' contents (a sampled fingerprint, one host synchronisation per forward) next to their
    # addresses and version counters, so that a write through ``weight_packed.data`` / ``scale.data`` is seen.
    # Set to False on a module (or on the class) once the weights are final and the eager call rate matters.
    verify_buffers = True

    def invalidate_cache(self) -> None:
        """Rebuild the derived buffers (tiled weights, float32 scale / bias) on the next forward."""
        self._derived_key = None

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        if self._compact:                                      # make room for the incoming public buffer
            self.weight_packed = torch.empty(((self.in_features + 3) // 4, self.out_features), dtype=torch.uint8,
                                             device=self.scale.device)
            self._compact = False
            self._tiled = None
        self.invalidate_cache()
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def compact(self, tiled: Optional[Tensor] = None) -> "TernaryLinearInference":
        """Keep ONE device copy of the weights: the tiled buffer the kernels read.  The public ``weight_packed``
        buffer is released (the attribute becomes an empty placeholder); ``state_dict()`` and ``public_packed()``
        rebuild it from the tiled copy with ``bt_untile_packed``, bit for bit.  ``tiled``: adopt this buffer (e.g. a
        view into a larger one shared with sibling layers) instead of re-tiling.  Undone by ``load_state_dict``."""
        if not self._compact:
            if tiled is None:
                tiled = self._derived()[0]
            self._tiled = tiled
            self.weight_packed = torch.empty(0, dtype=torch.uint8, device=self.scale.device)
            self._compact = True
            self._derived_key = None
        return self

    def public_packed(self) -> Tensor:
        """The wire-format buffer uint8 [ceil(K/4), N], whether or not the module still holds it."""
        if not self._compact:
            return self.weight_packed
        return require_ext().untile(self._tiled, self.in_features, self.out_features)

    def _derived(self):
        """(tiled weights, float32 scale, float32 bias, fresh): rebuilt when a buffer was replaced or written;
        ``fresh`` says they were written by kernels enqueued just now."""
        from .ternary_linear_cuda import capturing, content_fingerprint

        wp, sc, b = self.weight_packed, self.scale, self.bias
        watched = (sc,) if self._compact else (wp, sc)          # a compact module has no public buffer to watch
        key = tuple(v for t in watched for v in (t.data_ptr(), t._version)) + (
            None if b is None else (b.data_ptr(), b._version),)
        if self.verify_buffers and not capturing():
            key += content_fingerprint(*watched, *(() if b is None else (b,)))
        elif self._derived_key is not None:
            key += self._derived_key[len(key):]                # keep comparing addresses and versions only
        fresh = key != self._derived_key
        if fresh:
            C = require_ext()
            if not self._compact:
                self._tiled = C.retile(wp, self.in_features)
            self._scale32 = sc.to(torch.float32).contiguous()
            self._bias32 = None if b is None else b.to(torch.float32).contiguous()
            self._derived_key = key
        return self._tiled, self._scale32, self._bias32, fresh

    def forward(self, x: Tensor) -> Tensor:
        """x: (*, in_features) CUDA tensor -> (*, out_features), dtype of x."""
        require_cuda_tensor(x, "input")
        C = require_ext()
        if x.shape[-1] != self.in_features:
            raise RuntimeError("input K doesn't match in_features")
        if x.numel() == 0:
            raise RuntimeError("X is empty")
        x2d = x.contiguous().reshape(-1, self.in_features)
        if C.activation_mode() == "float" or x.dtype == torch.float64:
            if C.float_linear_tiled_ok(x2d.shape[0], self.in_features, x.dtype):      # exact, through the integer kernels
                tiled, s32, b32, fresh = self._derived()
                y = C.float_linear_tiled(x2d, tiled, self.in_features, self.out_features, s32, b32, fresh_weights=fresh)
                return y.reshape(*x.shape[:-1], self.out_features)
            return C.ternary_linear_packed_forward(x, self.public_packed(), self.scale, self.bias, self.in_features)
        tiled, s32, b32, fresh = self._derived()
        y = C.int8_linear_tiled(x2d, tiled, self.in_features, self.out_features, s32, b32, fresh_weights=fresh)
        return y.reshape(*x.shape[:-1], self.out_features)

    def forward_quantized(self, xq: Tensor, sx: Tensor, xsum: Optional[Tensor], out_dtype: torch.dtype) -> Tensor:
        """The layer on activations that are already int8 rows [M, in_features] with per-row scales (and row sums),
        as ``act_quant_i8`` or the fused elementwise kernels (``add_rmsnorm_quant``, ``silu_mul_quant``) emit them
        -> [M, out_features] in ``out_dtype``.  Same arithmetic as ``forward`` on the integer path."""
        C = require_ext()
        if xq.dim() != 2 or xq.shape[1] != self.in_features or xq.dtype != torch.int8:
            raise RuntimeError("xq must be int8 [M, in_features]")
        tiled, s32, b32, fresh = self._derived()
        m, k, n = xq.shape[0], self.in_features, self.out_features
        if m <= C.DECODE_MAX_M:
            return C.gemv_tiled_i8(xq, sx, tiled, k, n, s32, b32, out_dtype, fresh_weights=fresh)
        if k % 16 == 0:
            return C.gemm_tiled_i8(xq, sx, tiled, k, n, s32, b32, out_dtype, xsum=xsum)
        y = torch.empty((m, n), dtype=out_dtype, device=xq.device)        # ragged K: the decode kernel, 16 rows at a time
        for m0 in range(0, m, C.GEMV_MAX_M):
            m1 = min(m, m0 + C.GEMV_MAX_M)
            C.gemv_tiled_i8(xq[m0:m1], sx[m0:m1], tiled, k, n, s32, b32, out_dtype, out=y[m0:m1], fresh_weights=fresh)
        return y

    def extra_repr(self) -> str:
        packed_bytes = self.packed_size_bytes
        reduction = (self.out_features * self.in_features * 4) / (packed_bytes + self.scale.numel() * 2)
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"packed_bytes={packed_bytes}, reduction={reduction:.1f}x")

    @classmethod
    def from_unpacked(cls, w_tern: Tensor, scale: Tensor, bias: Optional[Tensor] = None) -> "TernaryLinearInference":
        """Build from ternary weights [N,K] (values -1/0/+1) and per-channel scales
        (bittorch/nn/ternary_linear_infer.py:120-152)."""
        out_features, in_features = w_tern.shape
        weight_packed, _ = pack_ternary_transposed(w_tern)
        return cls(in_features, out_features, weight_packed, scale, bias)

    @property
    def packed_size_bytes(self) -> int:
        return ((self.in_features + 3) // 4) * self.out_features

    @property
    def effective_bits_per_weight(self) -> float:
        total_bits = self.packed_size_bytes * 8 + self.scale.numel() * 16
        return total_bits / (self.out_features * self.in_features)


def _packed_into_state_dict(module, state_dict, prefix, local_metadata):
    """state_dict hook: a compact module serializes the public buffer rebuilt from its tiled copy."""
    if module._compact:
        state_dict[prefix + "weight_packed"] = module.public_packed()
    return state_dict


def create_ternary_linear_inference(in_features: int, out_features: int, weight: Tensor, bias: Optional[Tensor] = None,
                                    threshold_factor: float = 0.05) -> TernaryLinearInference:
    """Quantize + pack full-precision weights [N,K] in one fused kernel and wrap them
    (bittorch/nn/ternary_linear_infer.py:163-193)."""
    from ..quant.ternary_packed import quantize_pack_transposed

    packed_T, scale, _ = quantize_pack_transposed(weight, threshold_factor)
    return TernaryLinearInference(in_features, out_features, packed_T, scale, bias)
