"""Model conversion and checkpoint helpers (bittorch/utils/convert.py), wired to the fused
quantize+pack kernel: every converted layer costs one pass over its master weight.
Layers must already live on a CUDA device.
"""

from __future__ import annotations

import copy
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from ..nn import TernaryLinear, TernaryLinearInference
from ..nn.ternary_linear_infer import create_ternary_linear_inference


def fp_linear_to_ternary_infer(linear: nn.Linear, threshold_factor: float = 0.05) -> TernaryLinearInference:
    """nn.Linear -> TernaryLinearInference (bittorch/utils/convert.py:19-49)."""
    bias = linear.bias.data if linear.bias is not None else None
    return create_ternary_linear_inference(linear.in_features, linear.out_features, linear.weight.data, bias,
                                           threshold_factor)


def ternary_linear_to_infer(ternary_linear: TernaryLinear) -> TernaryLinearInference:
    """Trained TernaryLinear -> TernaryLinearInference with the same quantized weights
    (bittorch/utils/convert.py:52-73)."""
    if not ternary_linear.per_channel:
        raise RuntimeError("scale must be 1D [N]")   # packed inference needs per-channel scales
    bias = ternary_linear.bias.data if ternary_linear.bias is not None else None
    return create_ternary_linear_inference(ternary_linear.in_features, ternary_linear.out_features,
                                           ternary_linear.weight.data, bias, ternary_linear.threshold_factor)


def convert_linear_layers(module: nn.Module, threshold_factor: float = 0.05, skip_names: Optional[list] = None,
                          inplace: bool = False) -> nn.Module:
    """Recursively replace nn.Linear / TernaryLinear children by TernaryLinearInference;
    children whose dotted name contains an entry of ``skip_names`` are left alone
    (bittorch/utils/convert.py:76-133)."""
    skip = list(skip_names or [])
    if not inplace:
        module = copy.deepcopy(module)

    def walk(parent: nn.Module, prefix: str) -> None:
        for name, child in list(parent.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            skipped = any(pat in full for pat in skip)
            if isinstance(child, nn.Linear) and not skipped:
                setattr(parent, name, fp_linear_to_ternary_infer(child, threshold_factor))
            elif isinstance(child, TernaryLinear) and not skipped:
                setattr(parent, name, ternary_linear_to_infer(child))
            else:
                walk(child, full)

    walk(module, "")
    return module


def count_ternary_params(module: nn.Module) -> Dict[str, int]:
    """Weight counts by storage type (bittorch/utils/convert.py:136-166)."""
    counts = {"fp32": 0, "fp16": 0, "packed_ternary": 0, "total": 0}
    for _, child in module.named_modules():
        if isinstance(child, TernaryLinearInference):
            n = child.out_features * child.in_features
            counts["packed_ternary"] += n
        elif isinstance(child, (nn.Linear, TernaryLinear)):
            n = child.weight.numel()
            counts["fp16" if child.weight.dtype == torch.float16 else "fp32"] += n
        else:
            continue
        counts["total"] += n
    return counts


def get_model_memory_bytes(module: nn.Module) -> Dict[str, int]:
    """Bytes by storage type (bittorch/utils/convert.py:169-207)."""
    out = {"fp32": 0, "fp16": 0, "packed_ternary": 0, "scales": 0, "total": 0}
    for _, child in module.named_modules():
        if isinstance(child, TernaryLinearInference):
            packed = child.weight_packed.numel()
            scales = child.scale.numel() * child.scale.element_size()
            out["packed_ternary"] += packed
            out["scales"] += scales
            out["total"] += packed + scales
        elif isinstance(child, (nn.Linear, TernaryLinear)):
            wbytes = child.weight.numel() * child.weight.element_size()
            out["fp16" if child.weight.dtype == torch.float16 else "fp32"] += wbytes
            out["total"] += wbytes
        else:
            continue
        if child.bias is not None:
            out["total"] += child.bias.numel() * child.bias.element_size()
    return out


def save_ternary_checkpoint(module: nn.Module, path: str, metadata: Optional[Dict[str, Any]] = None) -> None:
    """``torch.save({"state_dict", "metadata"})`` (bittorch/utils/convert.py:210-228): the wire
    format is the public packed buffer, never the private tiled copy."""
    torch.save({"state_dict": module.state_dict(), "metadata": metadata or {}}, path)


def load_ternary_checkpoint(path: str, module: nn.Module) -> Dict[str, Any]:
    """Load a checkpoint written by ``save_ternary_checkpoint`` (or by the reference) into a
    module of matching architecture; returns the metadata (bittorch/utils/convert.py:231-246)."""
    checkpoint = torch.load(path, map_location="cpu")
    module.load_state_dict(checkpoint["state_dict"])
    return checkpoint.get("metadata", {})
