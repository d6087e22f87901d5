"""2-bit packing of ternary weights on the GPU.

Same functions and byte format as the reference's ``bittorch/quant/ternary_packed.py``
(00 = 0, 01 = +1, 10 = -1; weight j of a group of four in bits 2j+1:2j; K padded to a
multiple of four), computed by ``bt_pack_codes[_rows]`` / ``bt_unpack_codes[_rows]`` /
``bt_quantize_pack``.  Tensors must be CUDA tensors.
"""

from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from .._ext import require_cuda_tensor, require_ext


def _codes_i8(w_tern: Tensor) -> Tensor:
    if w_tern.dim() != 2:
        raise ValueError(f"Expected 2D tensor, got {w_tern.dim()}D")
    require_cuda_tensor(w_tern, "w_tern")
    return w_tern if w_tern.dtype == torch.int8 else w_tern.to(torch.int8)


def pack_ternary_transposed(w_tern: Tensor) -> Tuple[Tensor, int]:
    """[N,K] ternary -> (uint8 [ceil(K/4), N], K) (bittorch/quant/ternary_packed.py:174-206)."""
    codes = _codes_i8(w_tern)
    return require_ext().pack_codes(codes), int(w_tern.shape[1])


def pack_ternary(w_tern: Tensor) -> Tuple[Tensor, int]:
    """[N,K] ternary -> (uint8 [N, ceil(K/4)], K) (bittorch/quant/ternary_packed.py:22-75)."""
    codes = _codes_i8(w_tern)
    return require_ext().pack_codes_rows(codes), int(w_tern.shape[1])


def unpack_ternary_transposed(packed_T: Tensor, in_features: int) -> Tensor:
    """uint8 [ceil(K/4), N] -> int8 [N,K]; pattern 11 decodes to 0 (ternary_packed.py:209-223)."""
    if packed_T.dim() != 2:
        raise ValueError(f"Expected 2D tensor, got {packed_T.dim()}D")
    require_cuda_tensor(packed_T, "packed_T")
    return require_ext().unpack_codes(packed_T, int(in_features))


def unpack_ternary(packed: Tensor, in_features: int) -> Tensor:
    """uint8 [N, ceil(K/4)] -> int8 [N,K] (bittorch/quant/ternary_packed.py:78-120)."""
    if packed.dim() != 2:
        raise ValueError(f"Expected 2D tensor, got {packed.dim()}D")
    require_cuda_tensor(packed, "packed")
    return require_ext().unpack_codes_rows(packed, int(in_features))


def pack_ternary_with_scale(w_tern: Tensor, scale: Tensor) -> Tuple[Tensor, Tensor, int]:
    """(packed [N, ceil(K/4)], scale as float16, K) (bittorch/quant/ternary_packed.py:123-141)."""
    packed, k = pack_ternary(w_tern)
    return packed, scale.to(torch.float16), k


def quantize_pack_transposed(weight: Tensor, threshold_factor: float = 0.05) -> Tuple[Tensor, Tensor, int]:
    """Fused ``ternary_quantize`` + ``pack_ternary_transposed`` in one pass over the master
    weight: (uint8 [ceil(K/4), N], scale in weight dtype [N], K).  No reference counterpart
    as a single call; results are bit-identical to calling the two reference functions."""
    require_cuda_tensor(weight, "weight")
    out = require_ext().quantize_pack(weight, threshold_factor, want_packed=True)
    return out["packed_T"], out["scale"].to(weight.dtype), int(weight.shape[1])


def get_packed_size(out_features: int, in_features: int) -> int:
    """Bytes of the packed weights (bittorch/quant/ternary_packed.py:144-155)."""
    return out_features * ((in_features + 3) // 4)


def get_memory_reduction(out_features: int, in_features: int) -> float:
    """fp32 bytes / (packed bytes + fp16 scale bytes) (bittorch/quant/ternary_packed.py:158-171)."""
    return (out_features * in_features * 4) / (get_packed_size(out_features, in_features) + out_features * 2)
