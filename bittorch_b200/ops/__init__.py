"""Functional operations of the ternary linear path."""

from .ternary_linear import ternary_linear, ternary_linear_forward_cuda
from .ternary_linear_packed import has_packed_cuda_support, ternary_linear_packed_forward
from .ternary_linear_tensor_core import ternary_linear_tensor_core_forward

__all__ = [
    "ternary_linear",
    "ternary_linear_forward_cuda",
    "ternary_linear_packed_forward",
    "ternary_linear_tensor_core_forward",
    "has_packed_cuda_support",
]
