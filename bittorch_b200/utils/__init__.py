"""Model conversion and checkpoint helpers."""

from .convert import (
    convert_linear_layers,
    count_ternary_params,
    fp_linear_to_ternary_infer,
    get_model_memory_bytes,
    load_ternary_checkpoint,
    save_ternary_checkpoint,
    ternary_linear_to_infer,
)

__all__ = [
    "fp_linear_to_ternary_infer",
    "ternary_linear_to_infer",
    "convert_linear_layers",
    "count_ternary_params",
    "get_model_memory_bytes",
    "save_ternary_checkpoint",
    "load_ternary_checkpoint",
]
