"""Ternary quantization and 2-bit packing (GPU kernels)."""

from .ternary import (
    TernaryQuantConfig,
    TernaryQuantizer,
    dequantize_ternary,
    ternary_quantize,
    ternary_quantize_ste,
)
from .ternary_packed import (
    get_memory_reduction,
    get_packed_size,
    pack_ternary,
    pack_ternary_transposed,
    pack_ternary_with_scale,
    quantize_pack_transposed,
    unpack_ternary,
    unpack_ternary_transposed,
)

__all__ = [
    "TernaryQuantConfig",
    "TernaryQuantizer",
    "ternary_quantize",
    "ternary_quantize_ste",
    "dequantize_ternary",
    "pack_ternary",
    "unpack_ternary",
    "pack_ternary_with_scale",
    "pack_ternary_transposed",
    "unpack_ternary_transposed",
    "quantize_pack_transposed",
    "get_packed_size",
    "get_memory_reduction",
]
