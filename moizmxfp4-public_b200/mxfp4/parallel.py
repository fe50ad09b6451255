"""Tensor-parallel MXLinear layers for one 8-GPU box (one process per GPU, torch.distributed / NCCL).

The reference has no distributed code; this module adds only what sharding its MXLinear stacks needs.

Quantisation is independent per (row, 32-element block), so slicing the packed weight and its scales
along N, or along K at multiples of the block size, gives bit-identical shards to quantising the
sliced weight: sharding needs no communication and no re-quantisation.

  ColumnParallelMXLinear  weight rows (output features) split over ranks; no collective, the output
                          stays sharded (q, k, v, gate, up, lm_head).
  RowParallelMXLinear     weight columns (input features, K) split over ranks; each rank multiplies its
                          slice of the activations and the partial products (o, down) are summed over the
                          ranks.  The bias is added once, after the reduction.  On CUDA the sum is one kernel
                          of this library over peer memory (mxfp4_peer_allreduce: the GEMM writes its partial
                          into a peer-visible buffer, every rank reads all of them over NVLink and adds them in
                          float32 in rank order); NCCL's all-reduce is the fallback (MXFP4_TP_PEER_REDUCE=0,
                          no symmetric memory, N not a multiple of 8) and the path on CPU (gloo).
"""
import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _capi
from . import gemm as _gemm
from .modules import MXLinear

# The peer-visible buffers come from torch's symmetric memory, whose rendezvous would otherwise also bind them to an
# NVLink multicast object where the fabric offers one.  The reduction kernel uses plain peer loads and stores only, and
# a rank that dies while its memory is bound to a multicast object can fault the other ranks' GPUs, so the binding is
# switched off (torch reads this variable when it first allocates symmetric memory).
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


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
    tp_shard_dim = 0

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


class _PeerSum:
    """Peer-visible partial buffer of one row-parallel call site and the launch of mxfp4_peer_allreduce on it.

    The buffer comes from torch's symmetric memory (every rank allocates the same size and the ranks exchange
    mappings at rendezvous, a collective: all ranks must reach it in the same order, which SPMD layers do).  It is
    sized for the largest M seen so far and re-made when a larger M arrives; do the first call at each size outside
    CUDA graph capture."""

    def __init__(self, group):
        self.group = group
        self.world, self.rank = _group_info(group)
        self.interleaved = False      # set by a model that runs another peer call site between two uses of this one
        self.rows = 0
        self.N = 0
        self.buf = self.handle = self.blocks = self.epoch = self.status = None
        self.res = self.res_handle = self.results = self.owner_count = None        # two-shot mode of the fused peer sum
        # Two-shot (every rank reduces its own rows, then fetches the others' results) moves (world-1)/world * 2.3 partials'
        # worth of bytes per rank instead of world-1, but adds a second dependent handshake (~14 us measured at two ranks):
        # at four ranks it still loses on 16 MB sums (12.3 against 11.4 ms per 2048-token prefill of the 32-layer stack), so it
        # is the default only at eight ranks (prefill of 2048 tokens 17.6 -> 11.8 ms, decode step 4.18 -> 4.05 ms).
        ts = os.environ.get("MXFP4_TP_TWO_SHOT")
        self.two_shot = (self.world >= 8) if ts is None else ts == "1"
        self.two_shot_min_bytes = 0
        self.disabled = os.environ.get("MXFP4_TP_PEER_REDUCE", "1") == "0"

    def _make(self, M, N, device):
        import torch.distributed._symmetric_memory as symm
        L = _capi.load()
        rows = max(128, -(-M // 128) * 128)
        nbytes = L.mxfp4_peer_block_bytes(rows, N)
        group = self.group if self.group is not None else dist.group.WORLD
        buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
        handle = symm.rendezvous(buf, group)
        buf.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                      # every rank's flags are zero before anyone signals
        ptrs = [int(v) for v in handle.buffer_ptrs]
        self.blocks = (ctypes.c_void_p * len(ptrs))(*ptrs)
        self.buf, self.handle, self.rows, self.N = buf, handle, rows, N
        if self.two_shot:
            # result block: the rows this rank owns (at most ceil(rows / world)) as hidden | codes | scales
            res = symm.empty(-(-rows // self.world) * L.mxfp4_act_fused_result_row_bytes(N), dtype=torch.uint8, device=device)
            res_handle = symm.rendezvous(res, group)
            rptrs = [int(v) for v in res_handle.buffer_ptrs]
            self.results = (ctypes.c_void_p * len(rptrs))(*rptrs)
            self.res, self.res_handle = res, res_handle
            self.owner_count = torch.zeros(1, dtype=torch.int32, device=device)
            torch.cuda.synchronize(device)
            dist.barrier(group=group)
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def partial_view(self, M, N, device):
        """bf16 [M, N] view of this rank's partial inside the peer-visible block, or None when the peer path is off."""
        if self.disabled or N % 8:
            return None
        if self.buf is None or M > self.rows or N != self.N:
            err = None
            try:
                self._make(M, N, device)
            except Exception as e:            # no symmetric memory on this system
                err = e
            # The choice between the peer kernel and NCCL must be the same on every rank: a rank that fell back alone
            # would sit in an all-reduce while the others wait for its flags.  Every rank reaches this point together
            # (same sequence of calls and sizes), so the ranks vote.
            ok = torch.tensor([0 if err is not None else 1], dtype=torch.int32, device=device)
            group = self.group if self.group is not None else dist.group.WORLD
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                self.disabled = True
                self.buf = self.handle = self.blocks = None
                import warnings
                warnings.warn("mxfp4: peer-memory reduction unavailable on at least one rank"
                              + (f" (here: {err})" if err is not None else "") + "; all ranks use the NCCL all-reduce")
                return None
        off = _capi.load().mxfp4_peer_partial_offset()
        return self.buf[off:off + M * N * 2].view(torch.bfloat16).view(M, N)

    def reduce(self, M, N, bias, world, rank, device):
        L = _capi.load()
        y = torch.empty(M, N, dtype=torch.bfloat16, device=device)
        b = _gemm.bias_bf16(bias, device)
        with _capi.on_device(device):
            _capi.check(L.mxfp4_peer_allreduce(self.blocks, world, rank, self.epoch.data_ptr(), None if b is None else b.data_ptr(),
                                               y.data_ptr(), N, M, N, N, self.status.data_ptr(), _capi.stream_ptr(device)),
                        "mxfp4_peer_allreduce")
        return y

    def check_status(self):
        """Synchronises and raises if a launch at this call site gave up waiting for a peer.  Such a launch fills its
        output with NaN instead of a sum, so the failure also shows in the activations; poll this once per step,
        outside CUDA graph capture."""
        if self.status is not None and int(self.status.item()) != 0:
            self.status.zero_()
            raise _capi.MXFP4BackendError("mxfp4 peer reduction: a rank did not arrive within the wait bound")


class RowParallelMXLinear(_ParallelBase):
    """y = all_reduce_sum(x[..., rank slice of K] . W[:, rank slice]^T) + b."""
    tp_shard_dim = 1

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
        if self.world > 1 and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] == k:
            # GEMM straight into the peer-visible buffer, then one kernel sums all ranks' partials over NVLink
            if getattr(self, "_peer", None) is None:
                self._peer = _PeerSum(self.group)
            x2 = x.reshape(-1, k)
            M, N = x2.shape[0], self.out_features
            part = self._peer.partial_view(M, N, x.device) if M > 0 else None
            if part is not None:
                _gemm.quant_matmul_2d(x2, self.packed_weight, self.weight_scales, None, out=part)
                y = self._peer.reduce(M, N, self.bias, self.world, self.rank, x.device)
                return y.reshape(*x.shape[:-1], N)
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
    def build(cls, n_layers=32, hidden=4096, inter=11008, device="cuda", group=None, seed=0, block_size=32, fuse=True, init="cpu"):
        """Random-init N(0, 0.02) bf16 weights, quantised and sharded for this rank.  Every rank draws the
        same full matrices from the same generator (seed = layer*7 + j) and keeps its slice: init="cpu" uses torch's
        CPU generator (the same numbers on every machine: what the parity tests rebuild), init="cuda" the device's
        (the same numbers on every rank of a job, and seconds instead of minutes for 6.5 G elements).
        fuse=True stores q|k|v and gate|up as one column-parallel layer each (their packed rows concatenated,
        which changes no byte of any of them): one GEMM launch instead of three / two."""
        world, rank = _group_info(group)
        layers = []
        for li in range(n_layers):
            mods = {}
            for j, (name, n, k, col) in enumerate([("q", hidden, hidden, True), ("k", hidden, hidden, True), ("v", hidden, hidden, True),
                                                   ("o", hidden, hidden, False), ("gate", inter, hidden, True), ("up", inter, hidden, True),
                                                   ("down", hidden, inter, False)]):
                if init == "cuda":
                    g = torch.Generator(device=device).manual_seed(seed + li * 7 + j)
                    full = (torch.randn(n, k, generator=g, device=device) * 0.02).to(torch.bfloat16)
                else:
                    g = torch.Generator().manual_seed(seed + li * 7 + j)
                    full = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
                if col:
                    w = full[rank * n // world:(rank + 1) * n // world]
                else:
                    w = full[:, rank * k // world:(rank + 1) * k // world]
                w = w.to(device).contiguous()
                del full
                lin = MXLinear.from_linear(_as_linear(w), block_size=block_size)
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

    def forward(self, h: torch.Tensor, fused: Optional[bool] = None) -> torch.Tensor:
        """fused=True (the default on CUDA for stacks built with fuse=True): every gap between two GEMMs is one
        mxfp4_act_fused launch (residual add + RMS norm, q+k+v, silu*mul, each ending in the next GEMM's MXFP4 activation
        format, K-split partial sums and -- under tensor parallelism -- the row-parallel sum over peer memory folded in):
        eight launches per layer.  fused=False runs the same arithmetic as separate PyTorch operations and layer calls."""
        if fused is None:
            fused = h.is_cuda and h.dtype == torch.bfloat16 and h.dim() == 2 and len(self.layers) > 0 and "qkv" in self.layers[0] \
                and os.environ.get("MXFP4_STACK_FUSED", "1") != "0" and _gemm.get_gemm_mode() != "w4a16"
        if fused:
            return self._forward_fused(h)
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


def _stack_forward_fused(self, h: torch.Tensor) -> torch.Tensor:
    dev = h.device
    chain = getattr(self, "_chain", None)
    if chain is None or chain.dev != dev:
        chain = self._chain = _gemm.FusedChain(dev)
    M, hidden = h.shape
    hid = h.clone()                                  # the residual stream, updated in place by the RMSNORM steps
    world = self.layers[0]["o"].world
    peer_prev = None                                 # peer buffers holding the previous row-parallel layer's partial products

    def row_parallel(layer, peer_ok=True):
        """GEMM of a row-parallel layer: into the chain's buffer (one rank) or into this rank's peer-visible partial."""
        if world == 1:
            chain.gemm(layer.packed_weight, layer.weight_scales)
            return None
        if getattr(layer, "_peer", None) is None:
            layer._peer = _PeerSum(layer.group)
        layer._peer.interleaved = True               # o and down alternate: a site is never used twice in a row
        part = layer._peer.partial_view(M, layer.out_features, dev)
        if part is None:
            raise _capi.MXFP4BackendError("mxfp4: the fused stack needs the peer-memory reduction (symmetric memory); "
                                          "call forward(h, fused=False) for the NCCL path")
        chain.gemm(layer.packed_weight, layer.weight_scales, out=part)
        return layer._peer

    for L in self.layers:
        # h = h + (previous down); x = rmsnorm(h)
        chain.act(_capi.ACT_RMSNORM, M, hidden, residual=hid, hidden_out=hid, peer=peer_prev)
        n = chain.gemm(L["qkv"].packed_weight, L["qkv"].weight_scales)
        chain.act(_capi.ACT_SUM3, M, n // 3)                                   # a = q + k + v
        peer_o = row_parallel(L["o"])
        chain.act(_capi.ACT_RMSNORM, M, hidden, residual=hid, hidden_out=hid, peer=peer_o)    # h = h + o(a); x = rmsnorm(h)
        n = chain.gemm(L["gateup"].packed_weight, L["gateup"].weight_scales)
        chain.act(_capi.ACT_SILU_MUL, M, n // 2)                               # g = silu(gate) * up
        peer_prev = row_parallel(L["down"])
    chain.act(_capi.ACT_RMSNORM, M, hidden, residual=hid, hidden_out=hid, peer=peer_prev, quantize=False)   # h = h + down(g)
    return hid


MXBlockStack._forward_fused = _stack_forward_fused


def _as_linear(w: torch.Tensor) -> nn.Linear:
    lin = nn.Linear(w.shape[1], w.shape[0], bias=False, device="meta")
    lin.weight = nn.Parameter(w, requires_grad=False)
    return lin


def parallelize_llama(model: nn.Module, group=None, fuse: bool = True):
    """Replace the quantised MXLinear projections of an HF-style Llama (after quantize_model_mxfp4) by
    their tensor-parallel shards: q/k/v/gate/up column-parallel, o/down row-parallel, lm_head
    column-parallel with gathered logits; with fuse=True the q|k|v and gate|up shards of every block are then
    stored as one weight each (mxfp4.utils.model_utils.fuse_projections).

    Attention needs no change in models that derive the number of heads from the projection width
    (`.view(..., -1, head_dim)`, as Hugging Face's LlamaAttention does): every rank then simply attends over
    heads/world query heads and kv_heads/world key/value heads, which must both be divisible by the world size."""
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
    if fuse:
        from .utils.model_utils import fuse_projections
        fuse_projections(model)
    return model


def gather_state_dict(model: nn.Module, group=None, dst: Optional[int] = None):
    """state_dict of a tensor-parallel model in the reference's layout: every sharded packed weight, scale tensor and
    bias re-assembled from the ranks' shards (column-parallel: rows; row-parallel: columns of K), all other entries as
    they are.  The result loads into an unsharded quantised model (new.quantize(); new.load_state_dict(sd), the
    reference's flow in tests/test_modules.py:80-112) and is byte-identical to the state_dict the model had before
    parallelize_llama.  Collective: every rank must call it; every rank gets the result unless `dst` names one."""
    world, rank = _group_info(group)
    sharded = {name: mod.tp_shard_dim for name, mod in model.named_modules() if getattr(mod, "tp_shard_dim", None) is not None}
    out = {}
    for key, t in model.state_dict().items():
        mod_name, _, leaf = key.rpartition(".")
        if mod_name not in sharded or world == 1:
            out[key] = t
            continue
        dim = sharded[mod_name]
        if leaf == "bias" and dim == 1:
            out[key] = t                                   # a row-parallel bias is replicated
            continue
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=group)
        out[key] = torch.cat(parts, dim=0 if leaf == "bias" else dim)
    if dst is not None and rank != dst:
        return None
    return out
