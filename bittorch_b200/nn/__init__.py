"""Neural-network modules with ternary weights."""

from .ternary_linear import TernaryLinear
from .ternary_linear_cuda import TernaryLinearCUDA, verify_weight_contents
from .ternary_linear_infer import TernaryLinearInference, create_ternary_linear_inference

__all__ = ["TernaryLinear", "TernaryLinearCUDA", "TernaryLinearInference", "create_ternary_linear_inference",
           "verify_weight_contents"]
