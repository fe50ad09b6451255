"""Model-level helpers (reference: src/mxfp4/utils/model_utils.py)."""
from typing import List, Optional

import torch
import torch.nn as nn

from ..modules import MXLinear


FUSABLE_GROUPS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))


class _FusedGroup:
    """Shared state of projections that read the same input (q|k|v, gate|up): their packed rows back to back in one
    tensor, so that one GEMM launch (and one activation quantisation) serves all of them.  The members keep their own
    buffers as views into it, so state_dict keys, shapes and bytes stay those of the unfused layers."""

    def __init__(self, packed, scales, bias, in_features, n_members):
        self.packed, self.scales, self.bias = packed, scales, bias
        self.in_features, self.n_members = in_features, n_members
        self.last_in = self.last_version = self.last_out = None
        self.served = 0

    def output(self, x):
        from ..gemm import mxlinear_forward
        if self.last_in is x and self.last_version == x._version and self.last_out is not None:
            y = self.last_out
        else:
            y = mxlinear_forward(x, self.packed, self.scales, self.bias, self.in_features)
            self.last_in, self.last_version, self.last_out, self.served = x, x._version, y, 0
        self.served += 1
        if self.served >= self.n_members:          # every member has had its slice: do not keep the tensors alive
            self.last_in = self.last_out = None
        return y


class FusedSliceLinear(nn.Module):
    """One member of a fused projection group: forward returns its columns of the group's single GEMM."""

    def __init__(self, member, group: _FusedGroup, start: int, packed_view, scales_view):
        super().__init__()
        self.in_features, self.out_features = member.in_features, packed_view.shape[0]     # rows held here (a shard's, if sharded)
        self.block_size = getattr(member, "block_size", 32)
        self.is_quantized = True
        self.tp_shard_dim = getattr(member, "tp_shard_dim", None)     # a column-parallel shard stays one
        self._group, self._start = [group], start          # in a list: not a submodule, not in state_dict
        self.register_buffer("packed_weight", packed_view)
        self.register_buffer("weight_scales", scales_view)
        self.bias = member.bias                             # Parameter or None, kept for the state_dict
        self.register_parameter("weight", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._group[0].output(x)
        return y[..., self._start:self._start + self.out_features]

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, fused=True"


def fuse_projections(model: nn.Module, groups=FUSABLE_GROUPS, verbose: bool = False) -> nn.Module:
    """Store q|k|v and gate|up projections of every block as one quantised weight each (in place).

    A parent module whose children named as one of `groups` are all quantised layers (MXLinear or column-parallel
    shards) with the same input width and block size gets them replaced by FusedSliceLinear members of one group: the
    first member called with an input runs one GEMM over the concatenated rows, the others return their slice of that
    result when they are handed the same tensor.  Concatenating rows changes no byte of any weight and no output bit
    of any row; it removes two of three (one of two) launch chains per block.  Call it after the model sits on its
    device; state_dict() keeps the unfused keys and bytes."""
    n_groups = 0
    for parent in list(model.modules()):
        for names in groups:
            members = [getattr(parent, n, None) for n in names]
            if any(m is None or isinstance(m, FusedSliceLinear) for m in members):
                continue
            if not all(getattr(m, "is_quantized", False) and getattr(m, "packed_weight", None) is not None for m in members):
                continue
            if any(getattr(m, "gather_output", False) for m in members):
                continue
            if len({(m.in_features, m.packed_weight.shape[1], m.weight_scales.shape[1], m.weight_scales.dtype, m.bias is None) for m in members}) != 1:
                continue
            packed = torch.cat([m.packed_weight for m in members], 0)
            scales = torch.cat([m.weight_scales for m in members], 0)
            bias = None if members[0].bias is None else torch.cat([m.bias.detach() for m in members], 0)
            group = _FusedGroup(packed, scales, bias, members[0].in_features, len(members))
            row = 0
            for n, m in zip(names, members):
                rows = m.packed_weight.shape[0]
                setattr(parent, n, FusedSliceLinear(m, group, row, packed[row:row + rows], scales[row:row + rows]))
                row += rows
            n_groups += 1
    if verbose:
        print(f"Fused {n_groups} projection groups.")
    return model


def quantize_model_mxfp4(model: nn.Module, block_size: int = 32, exclude_layers: Optional[List[str]] = None,
                         verbose: bool = True, fuse: bool = False) -> nn.Module:
    """Recursively replace every nn.Linear by a quantised MXLinear, in place
    (model_utils.py:8-73 of the reference; names containing any string of `exclude_layers` are left alone).

    Unlike the reference, the replacement layer is built directly around the existing weight: no
    float32 [out, in] parameter is allocated and randomly initialised first, and the weight is
    quantised where it lives (it must be on a CUDA device).
    fuse=True (an argument the reference does not have) also applies fuse_projections() to the result.
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
    if fuse:
        fuse_projections(model, verbose=verbose)
    return model


def get_model_size_mb(model: nn.Module) -> float:
    """Size of parameters plus buffers in MiB (model_utils.py:75-90)."""
    total = sum(p.nelement() * p.element_size() for p in model.parameters())
    total += sum(b.nelement() * b.element_size() for b in model.buffers())
    return total / (1024 * 1024)
