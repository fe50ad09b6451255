"""Batched greedy decoding of a Hugging-Face-shaped Llama whose linear layers were quantised with
quantize_model_mxfp4 (the reference's README scenario: Llama-2-7B, batch 128; src/mxfp4/utils/model_utils.py:8-73 swaps
the layers, the model's own PyTorch code runs them).

The reference owns only the linear layers of such a model; everything between them is the model's code.  This runner
keeps that split but runs the part the library owns as one fused chain per layer (mxfp4.gemm.FusedChain): the RMS norms
(with their learned weights), the residual adds and silu*mul end directly in MXFP4 activations, the row-parallel sums of
tensor parallelism run inside those same kernels over peer memory, q|k|v and gate|up are one GEMM each.  Attention itself
(rotary embedding, KV cache, softmax(QK^T)V) is torch's scaled_dot_product_attention on a preallocated cache: it is not part
of this library.  A decode step has fixed shapes and is replayed from a CUDA graph.

Tensor parallelism: q/k/v/gate/up are split by output rows (whole heads per rank), o and down by input columns; every
rank holds the KV cache of its own heads.  The only exchange is the row-parallel sum, which runs inside mxfp4_act_fused:
a decode step contains no NCCL call.
"""
from typing import Optional

import torch
import torch.nn.functional as F

from . import _capi
from . import gemm as _gemm
from .parallel import _PeerSum, _group_info, shard_quantized


class LlamaMXDecoder:
    def __init__(self, model, max_batch: int, max_len: int, group=None):
        """`model`: transformers LlamaForCausalLM (or the same module layout) after quantize_model_mxfp4, on a CUDA
        device; the quantised buffers are sliced for this rank, nothing is re-quantised."""
        cfg = model.config
        self.world, self.rank = _group_info(group)
        self.group = group
        base = model.model
        self.dev = base.embed_tokens.weight.device
        self.hidden = cfg.hidden_size
        self.n_heads, self.n_kv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        if self.n_heads % self.world or self.n_kv % self.world:
            raise ValueError(f"{self.n_heads} heads / {self.n_kv} KV heads do not divide over {self.world} ranks")
        self.h_l, self.kv_l = self.n_heads // self.world, self.n_kv // self.world
        self.eps = cfg.rms_norm_eps
        self.B, self.S = max_batch, max_len
        w, r = self.world, self.rank

        def rows(layer):                      # column-parallel: output rows of this rank
            return shard_quantized(layer.packed_weight, layer.weight_scales, 0, w, r)

        def cols(layer):                      # row-parallel: input columns of this rank
            return shard_quantized(layer.packed_weight, layer.weight_scales, 1, w, r)

        self.layers = []
        for L in base.layers:
            a, m = L.self_attn, L.mlp
            for lin in (a.q_proj, a.k_proj, a.v_proj, a.o_proj, m.gate_proj, m.up_proj, m.down_proj):
                if not getattr(lin, "is_quantized", False) or lin.bias is not None:
                    raise ValueError("LlamaMXDecoder needs bias-free projections quantised by quantize_model_mxfp4")
            q, k, v, g, u = rows(a.q_proj), rows(a.k_proj), rows(a.v_proj), rows(m.gate_proj), rows(m.up_proj)
            o, d = cols(a.o_proj), cols(m.down_proj)
            self.layers.append(dict(
                qkv=(torch.cat([q[0], k[0], v[0]], 0), torch.cat([q[1], k[1], v[1]], 0)),
                gateup=(torch.cat([g[0], u[0]], 0), torch.cat([g[1], u[1]], 0)),
                o=o, down=d,
                g1=L.input_layernorm.weight.detach().to(torch.bfloat16).contiguous(),
                g2=L.post_attention_layernorm.weight.detach().to(torch.bfloat16).contiguous()))
        self.g_final = base.norm.weight.detach().to(torch.bfloat16).contiguous()
        self.embed = base.embed_tokens.weight.detach()
        head = model.lm_head
        if not getattr(head, "is_quantized", False):
            raise ValueError("LlamaMXDecoder needs a quantised lm_head")
        self.vocab = head.packed_weight.shape[0]
        # the vocabulary projection stays whole on every rank: its input (the residual stream) is replicated, so every
        # rank gets the full logits and picks the same token without any exchange (70 MB of weights per step at 7B size)
        self.head = (head.packed_weight, head.weight_scales)
        # rotary tables as the model computes them (float32 angles, cast to the activations' dtype)
        inv_freq = base.rotary_emb.inv_freq.to(self.dev).float()
        scaling = float(getattr(base.rotary_emb, "attention_scaling", 1.0))
        ang = torch.arange(max_len, device=self.dev).float()[:, None] * inv_freq[None, :]
        emb = torch.cat([ang, ang], -1)
        self.cos, self.sin = (emb.cos() * scaling).to(torch.bfloat16), (emb.sin() * scaling).to(torch.bfloat16)
        kv_shape = (max_batch, self.kv_l, max_len, self.head_dim)
        self.k_cache = [torch.zeros(kv_shape, dtype=torch.bfloat16, device=self.dev) for _ in self.layers]
        self.v_cache = [torch.zeros(kv_shape, dtype=torch.bfloat16, device=self.dev) for _ in self.layers]
        self.chain = _gemm.FusedChain(self.dev)
        # two peer-visible partial buffers serve all layers: the o and down sums alternate, so a buffer is never used
        # twice in a row and the "everybody has finished reading" handshake can be skipped
        self.peers = None
        if w > 1:
            self.peers = (_PeerSum(group), _PeerSum(group))
            for p in self.peers:
                p.interleaved = True
        self.pos = torch.zeros(1, dtype=torch.int64, device=self.dev)
        self.ids = torch.zeros(max_batch, dtype=torch.int64, device=self.dev)
        self.graph = None

    # ------------------------------------------------------------------------------------------------
    def _row_parallel(self, weight, which, M):
        """GEMM of a row-parallel layer into the chain's buffer (one rank) or this rank's peer-visible partial."""
        if self.world == 1:
            self.chain.gemm(*weight)
            return None
        peer = self.peers[which]
        part = peer.partial_view(M, self.hidden, self.dev)
        if part is None:
            raise _capi.MXFP4BackendError("mxfp4: the decoder's tensor parallelism needs the peer-memory reduction (symmetric memory)")
        self.chain.gemm(*weight, out=part)
        return peer

    def _rope(self, x, cos, sin):
        half = x.shape[-1] // 2
        rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
        return x * cos + rot * sin

    def _forward(self, ids, T, pos0=None, batch0=0):
        """Logits of the LAST position of every sequence: ids [B, T]; T > 1 is a prefill from position 0 (written into
        cache rows batch0..batch0+B), T == 1 a decode step at the device-side position self.pos for the whole batch."""
        c = self.chain
        c.src = None                                  # the first step of a pass has no GEMM in front
        B = ids.shape[0]
        M = B * T
        hid = self.embed.index_select(0, ids.reshape(-1)).to(torch.bfloat16)       # [M, hidden]: the residual stream
        if T > 1:
            cos, sin = self.cos[:T][None, None], self.sin[:T][None, None]
        else:
            cos, sin = self.cos.index_select(0, self.pos)[None, None], self.sin.index_select(0, self.pos)[None, None]
            mask = (torch.arange(self.S, device=self.dev) <= self.pos)[None, None, None, :]
        nq, nkv, D = self.h_l * self.head_dim, self.kv_l * self.head_dim, self.head_dim
        qkv = torch.empty(M, nq + 2 * nkv, dtype=torch.bfloat16, device=self.dev)
        peer_prev = None
        for li, L in enumerate(self.layers):
            c.act(_capi.ACT_RMSNORM, M, self.hidden, residual=hid, hidden_out=hid, gamma=L["g1"], eps=self.eps, peer=peer_prev)
            c.gemm(*L["qkv"], out=qkv)
            q = qkv[:, :nq].view(B, T, self.h_l, D).transpose(1, 2)
            k = qkv[:, nq:nq + nkv].view(B, T, self.kv_l, D).transpose(1, 2)
            v = qkv[:, nq + nkv:].view(B, T, self.kv_l, D).transpose(1, 2)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            if T > 1:
                self.k_cache[li][batch0:batch0 + B, :, :T] = k
                self.v_cache[li][batch0:batch0 + B, :, :T] = v
                att = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.h_l != self.kv_l)
            else:
                kc, vc = self.k_cache[li][:B], self.v_cache[li][:B]      # the batch may be smaller than the cache
                kc.index_copy_(2, self.pos, k)
                vc.index_copy_(2, self.pos, v)
                att = F.scaled_dot_product_attention(q, kc, vc, attn_mask=mask, enable_gqa=self.h_l != self.kv_l)
            c.feed(att.transpose(1, 2).reshape(M, nq))
            c.act(_capi.ACT_IDENTITY, M, nq)
            peer_o = self._row_parallel(L["o"], 0, M)
            c.act(_capi.ACT_RMSNORM, M, self.hidden, residual=hid, hidden_out=hid, gamma=L["g2"], eps=self.eps, peer=peer_o)
            n = c.gemm(*L["gateup"])
            c.act(_capi.ACT_SILU_MUL, M, n // 2)
            peer_prev = self._row_parallel(L["down"], 1, M)
        c.act(_capi.ACT_RMSNORM, M, self.hidden, residual=hid, hidden_out=hid, gamma=self.g_final, eps=self.eps, peer=peer_prev,
              quantize=(T == 1))
        if T > 1:
            # only the last position of every sequence feeds the vocabulary projection
            last = hid.view(B, T, self.hidden)[:, -1]
            x = (self.g_final * F.rms_norm(last.float(), (self.hidden,), eps=self.eps).to(torch.bfloat16)).contiguous()
            c.feed(x)
            c.act(_capi.ACT_IDENTITY, B, self.hidden)
        logits = torch.empty(B, self.vocab, dtype=torch.bfloat16, device=self.dev)
        c.gemm(*self.head, out=logits)
        return logits

    def _next_tokens(self, logits):
        return logits.float().argmax(dim=-1)

    @torch.no_grad()
    def prefill(self, prompt_ids: torch.Tensor, chunk: int = 16):
        """Fills the KV cache from the prompts [B, T] (sequence chunks bound the activation buffers) and returns the first
        generated token of every sequence."""
        B, T = prompt_ids.shape
        assert B <= self.B and T < self.S
        out = []
        for b0 in range(0, B, chunk):
            ids = prompt_ids[b0:b0 + chunk].to(self.dev)
            out.append(self._next_tokens(self._forward(ids, T, batch0=b0)))
        self.pos.fill_(T)
        if getattr(self, "nb", None) != B:
            self.graph = None                      # a captured decode step is tied to its batch size
        self.nb = B
        nxt = torch.cat(out)
        self.ids[:B].copy_(nxt)
        return nxt

    @torch.no_grad()
    def _step(self):
        nxt = self._next_tokens(self._forward(self.ids[:self.nb, None], 1))
        self.ids[:self.nb].copy_(nxt)
        self.pos.add_(1)
        return nxt

    @torch.no_grad()
    def decode(self, new_tokens: int, use_graph: bool = True):
        """Greedy decoding after prefill(): returns [B, new_tokens] (the first column is prefill's token)."""
        toks = [self.ids[:self.nb].clone()]
        if new_tokens <= 1:
            return torch.stack(toks, 1)
        if use_graph and self.graph is None:
            # one eager step allocates every buffer (and sets up the peer buffers) before the capture
            pos0, ids0 = self.pos.clone(), self.ids.clone()
            side = torch.cuda.Stream(self.dev)
            side.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(side):
                self._step()
                self.pos.copy_(pos0); self.ids.copy_(ids0)
                torch.cuda.synchronize(self.dev)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    self._graph_out = self._step()
            torch.cuda.current_stream(self.dev).wait_stream(side)
            self.pos.copy_(pos0); self.ids.copy_(ids0)
            self.graph = g
        for _ in range(new_tokens - 1):
            if use_graph:
                self.graph.replay()
                toks.append(self._graph_out.clone())
            else:
                toks.append(self._step().clone())
        return torch.stack(toks, 1)
