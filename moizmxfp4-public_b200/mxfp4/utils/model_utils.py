"""Model-level helpers (reference: src/mxfp4/utils/model_utils.py)."""
from typing import List, Optional

import torch
import torch.nn as nn

from ..modules import MXLinear


def quantize_model_mxfp4(model: nn.Module, block_size: int = 32, exclude_layers: Optional[List[str]] = None,
                         verbose: bool = True) -> nn.Module:
    """Recursively replace every nn.Linear by a quantised MXLinear, in place
    (model_utils.py:8-73 of the reference; names containing any string of `exclude_layers` are left alone).

    Unlike the reference, the replacement layer is built directly around the existing weight: no
    float32 [out, in] parameter is allocated and randomly initialised first, and the weight is
    quantised where it lives (it must be on a CUDA device).
    """
    exclude_layers = exclude_layers or []

    def _replace_recursive(module, prefix=""):
        replaced = 0
        for name, child in module.named_children():
            full_name = f"{prefix}.{name}" if prefix else name
            if any(ex in full_name for ex in exclude_layers):
                continue
            if isinstance(child, nn.Linear):
                new_layer = MXLinear.from_linear(child, block_size=block_size)
                new_layer.quantize()
                setattr(module, name, new_layer)
                replaced += 1
            else:
                replaced += _replace_recursive(child, full_name)
        return replaced

    total = _replace_recursive(model)
    if verbose:
        print(f"Quantized {total} Linear layers.")
    return model


def get_model_size_mb(model: nn.Module) -> float:
    """Size of parameters plus buffers in MiB (model_utils.py:75-90)."""
    total = sum(p.nelement() * p.element_size() for p in model.parameters())
    total += sum(b.nelement() * b.element_size() for b in model.buffers())
    return total / (1024 * 1024)
