"""Tensor-parallel MXLinear layers for one 8-GPU box (one process per GPU, torch.distributed / NCCL).

The reference has no distributed code; this module adds only what sharding its MXLinear stacks needs.

Quantisation is independent per (row, 32-element block), so slicing the packed weight and its scales
along N, or along K at multiples of the block size, gives bit-identical shards to quantising the
sliced weight: sharding needs no communication and no re-quantisation.

  ColumnParallelMXLinear  weight rows (output features) split over ranks; no collective, the output
                          stays sharded (q, k, v, gate, up, lm_head).
  RowParallelMXLinear     weight columns (input features, K) split over ranks; each rank multiplies its
                          slice of the activations and one all-reduce (sum, bf16) per layer combines the
                          partial products (o, down).  The bias is added once, after the reduction.
"""
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import gemm as _gemm
from .modules import MXLinear


def _group_info(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def shard_quantized(packed: torch.Tensor, scales: torch.Tensor, dim: int, world: int, rank: int, block_size: int = 32):
    """Slice a quantised weight (packed [N, K/2], scales [N, K/block]) for `rank` of `world`.
    dim 0 splits output rows; dim 1 splits K, which must divide into whole blocks per rank."""
    N, k2 = packed.shape
    if dim == 0:
        if N % world:
            raise ValueError(f"out_features {N} not divisible by tensor-parallel size {world}")
        n = N // world
        return packed[rank * n:(rank + 1) * n].contiguous(), scales[rank * n:(rank + 1) * n].contiguous()
    K = k2 * 2
    if K % (world * block_size):
        raise ValueError(f"in_features {K} not divisible into {world} shards of whole {block_size}-element blocks")
    k = K // world
    return (packed[:, rank * k // 2:(rank + 1) * k // 2].contiguous(),
            scales[:, rank * k // block_size:(rank + 1) * k // block_size].contiguous())


class _ParallelBase(nn.Module):
    def __init__(self, in_features, out_features, group=None):
        super().__init__()
        self.in_features, self.out_features, self.group = in_features, out_features, group
        self.world, self.rank = _group_info(group)
        self.register_buffer("packed_weight", None)
        self.register_buffer("weight_scales", None)
        self.register_parameter("bias", None)
        self.is_quantized = True

    def _load(self, packed, scales, bias):
        self.packed_weight, self.weight_scales = packed, scales
        if bias is not None:
            self.bias = nn.Parameter(bias.detach().clone(), requires_grad=False)


class ColumnParallelMXLinear(_ParallelBase):
    """y_shard = x . W[rank rows]^T + b[rank rows]; optionally all-gathers the shards along the last dim."""

    def __init__(self, in_features, out_features, group=None, gather_output=False):
        super().__init__(in_features, out_features, group)
        self.gather_output = gather_output

    @classmethod
    def from_mxlinear(cls, layer: MXLinear, group=None, gather_output=False):
        assert layer.is_quantized, "quantize() the layer first"
        self = cls(layer.in_features, layer.out_features, group, gather_output)
        p, s = shard_quantized(layer.packed_weight, layer.weight_scales, 0, self.world, self.rank, layer.block_size)
        n = layer.out_features // self.world
        b = None if layer.bias is None else layer.bias.data[self.rank * n:(self.rank + 1) * n]
        self._load(p, s, b)
        return self

    def forward(self, x: torch.Tensor, reuse_act: bool = False) -> torch.Tensor:
        """reuse_act=True: the previous layer call on this stream had the same input (q/k/v, gate/up); its quantised
        activations are reused instead of being recomputed."""
        y = _gemm.mxlinear_forward(x, self.packed_weight, self.weight_scales, self.bias, self.in_features, reuse_act)
        if self.gather_output and self.world > 1:
            parts = [torch.empty_like(y) for _ in range(self.world)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y


class RowParallelMXLinear(_ParallelBase):
    """y = all_reduce_sum(x[..., rank slice of K] . W[:, rank slice]^T) + b."""

    def __init__(self, in_features, out_features, group=None, input_is_parallel=True):
        super().__init__(in_features, out_features, group)
        self.input_is_parallel = input_is_parallel

    @classmethod
    def from_mxlinear(cls, layer: MXLinear, group=None, input_is_parallel=True):
        assert layer.is_quantized, "quantize() the layer first"
        self = cls(layer.in_features, layer.out_features, group, input_is_parallel)
        p, s = shard_quantized(layer.packed_weight, layer.weight_scales, 1, self.world, self.rank, layer.block_size)
        self._load(p, s, None if layer.bias is None else layer.bias.data)
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        k = self.packed_weight.shape[-1] * 2
        if not self.input_is_parallel:
            x = x[..., self.rank * k:(self.rank + 1) * k]
        y = _gemm.mxlinear_forward(x, self.packed_weight, self.weight_scales, None, k)
        if self.world > 1:
            y = y.contiguous()
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)     # bf16 partial products, summed by NCCL
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y


class MXBlockStack(nn.Module):
    """A Llama-shaped stack of MXLinear blocks without attention: per layer
         a = q(h) + k(h) + v(h);  h = h + o(a);  g = silu(gate(h)) * up(h);  h = h + down(g)
    with an RMS normalisation in front of each half.  q/k/v/gate/up are column-parallel, o/down
    row-parallel, so a layer costs two all-reduces of [M, hidden]."""

    def __init__(self, layers):
        super().__init__()
        self.layers = nn.ModuleList(layers)

    @staticmethod
    def _norm(h):
        # one fused kernel; the composed form (float, pow, mean, rsqrt, mul, cast) was six launches and a fifth of a decode step
        return torch.nn.functional.rms_norm(h, (h.shape[-1],), eps=1e-6)

    @classmethod
    def build(cls, n_layers=32, hidden=4096, inter=11008, device="cuda", group=None, seed=0, block_size=32, fuse=True):
        """Random-init N(0, 0.02) bf16 weights, quantised and sharded for this rank.  Every rank draws the
        same full matrices from the same CPU generator (seed = layer*7 + j) and keeps its slice.
        fuse=True stores q|k|v and gate|up as one column-parallel layer each (their packed rows concatenated,
        which changes no byte of any of them): one GEMM launch instead of three / two."""
        world, rank = _group_info(group)
        layers = []
        for li in range(n_layers):
            mods = {}
            for j, (name, n, k, col) in enumerate([("q", hidden, hidden, True), ("k", hidden, hidden, True), ("v", hidden, hidden, True),
                                                   ("o", hidden, hidden, False), ("gate", inter, hidden, True), ("up", inter, hidden, True),
                                                   ("down", hidden, inter, False)]):
                g = torch.Generator().manual_seed(seed + li * 7 + j)
                if col:
                    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)[rank * n // world:(rank + 1) * n // world]
                else:
                    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)[:, rank * k // world:(rank + 1) * k // world]
                lin = MXLinear.from_linear(_as_linear(w.to(device)), block_size=block_size)
                lin.quantize()
                par = (ColumnParallelMXLinear if col else RowParallelMXLinear)(k, n, group)
                par._load(lin.packed_weight, lin.weight_scales, None)
                mods[name] = par
            if fuse:
                for fused, parts in (("qkv", ("q", "k", "v")), ("gateup", ("gate", "up"))):
                    par = ColumnParallelMXLinear(mods[parts[0]].in_features, sum(mods[p].out_features for p in parts), group)
                    par._load(torch.cat([mods[p].packed_weight for p in parts], 0), torch.cat([mods[p].weight_scales for p in parts], 0), None)
                    for p in parts:
                        del mods[p]
                    mods[fused] = par
            layers.append(nn.ModuleDict(mods))
        return cls(layers)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        for L in self.layers:
            x = self._norm(h)
            if "qkv" in L:
                q, k, v = L["qkv"](x).chunk(3, dim=-1)
                a = q + k + v
            else:
                a = L["q"](x) + L["k"](x, reuse_act=True) + L["v"](x, reuse_act=True)
            h = h + L["o"](a)
            x = self._norm(h)
            if "gateup" in L:
                gate, up = L["gateup"](x).chunk(2, dim=-1)
                g = torch.nn.functional.silu(gate) * up
            else:
                g = torch.nn.functional.silu(L["gate"](x)) * L["up"](x, reuse_act=True)
            h = h + L["down"](g)
        return h


def _as_linear(w: torch.Tensor) -> nn.Linear:
    lin = nn.Linear(w.shape[1], w.shape[0], bias=False, device="meta")
    lin.weight = nn.Parameter(w, requires_grad=False)
    return lin


def parallelize_llama(model: nn.Module, group=None):
    """Replace the quantised MXLinear projections of an HF-style Llama (after quantize_model_mxfp4) by
    their tensor-parallel shards: q/k/v/gate/up column-parallel, o/down row-parallel, lm_head
    column-parallel with gathered logits.  Attention head counts per rank are the caller's business."""
    col = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
    row = ("o_proj", "down_proj")

    def walk(mod):
        for name, child in list(mod.named_children()):
            if isinstance(child, MXLinear) and child.is_quantized:
                if name in col:
                    setattr(mod, name, ColumnParallelMXLinear.from_mxlinear(child, group))
                elif name in row:
                    setattr(mod, name, RowParallelMXLinear.from_mxlinear(child, group))
                elif name == "lm_head":
                    setattr(mod, name, ColumnParallelMXLinear.from_mxlinear(child, group, gather_output=True))
            else:
                walk(child)
    walk(model)
    return model
