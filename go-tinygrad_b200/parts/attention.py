"""Grouped-query attention with a position encoding on queries and keys.

q, k, v = x Wq^T, x Wk^T, x Wv^T; rotate q and k; store k (after rotation) and
v in the cache; per query head h, softmax((q_h . K_{h // group}) * scale) V,
causal within the sequence, optionally over the last `window` keys only; then
the output projection (model/llama.go:1111-1137 projections, :1230-1233
rotation, :1253-1254 cache write, :1603-1661 attention, :1290-1297 output).

Parameters: ``hidden_size``, ``n_heads``, ``n_kv_heads``, ``head_dim``,
``window`` (None: all keys), ``scale`` (None: head_dim^-1/2), ``position`` (a
position PartSpec), ``own_kv`` (False for a layer that has no key/value
projections and reads another run's cache), and the tensor names ``q``, ``k``,
``v``, ``o``.  The three projections are fused at load into one matrix
[(n_heads + 2 n_kv_heads) * head_dim, hidden] so that one product serves them.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..cache import CacheHandle, KVRequest, Request
from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Mixer, Runtime, StepContext, build_part, emit_update, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.n_kv = int(self.param("n_kv_heads"))
        self.head_dim = int(self.param("head_dim"))
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} query heads cannot share {self.n_kv} key/value heads")
        window = self.p.get("window")
        self.window = int(window) if window else None
        scale = self.p.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.own_kv = bool(self.p.get("own_kv", True))
        self.position = build_part("position", self.param("position"))
        self.names = {k: str(self.param(k)) for k in (("q", "k", "v", "o") if self.own_kv else ("q", "o"))}
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv * self.head_dim
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.names["q"], (self.q_dim, self.hidden))]
        if self.own_kv:
            specs += [WeightSpec(self.names["k"], (self.kv_dim, self.hidden)),
                      WeightSpec(self.names["v"], (self.kv_dim, self.hidden))]
        specs.append(WeightSpec(self.names["o"], (self.hidden, self.q_dim)))
        return specs

    def children(self):
        return [self.position]

    def cache_requests(self) -> List[Request]:
        return [KVRequest(self.n_kv, self.head_dim, self.window)] if self.own_kv else []

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        parts = [tensors[self.names["q"]]]
        if self.own_kv:
            parts += [tensors[self.names["k"]], tensors[self.names["v"]]]
        self.w_qkv = rt.matrix(torch.cat([p.to(rt.dtype) for p in parts], dim=0))
        self.w_o = rt.matrix(tensors[self.names["o"]])

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        rt = ctx.rt
        kv = cache.kv
        if kv is None or kv.n_kv_heads != self.n_kv or kv.head_dim != self.head_dim:
            raise ValueError("attention was given a cache entry that does not match its heads")
        n = x.shape[0]
        qkv = rt.empty(n, self.w_qkv.shape[0])
        rotation = self.position.rotation(ctx)
        pairing, rotary_dim = self.position.pairing, self.position.rotary_dim or self.head_dim
        # the kernels that rotate inside a product or inside the attention know one
        # layout: half-split pairs over the whole head; any other goes the general way
        plain_layout = rotation is None or (pairing == "half" and rotary_dim == self.head_dim)
        store = self.n_kv if (cache.writes and self.own_kv) else 0
        # a decode step in bfloat16: the attention kernel rotates the queries and adds the new
        # token's key and value itself, and no kernel stands between it and the projection
        in_attention = (ctx.is_decode and rt.dtype == torch.bfloat16 and plain_layout
                        and ops.attention_bf16_supports(self.head_dim))
        if store and plain_layout and ops.qkv_rope_fused_supports(x, self.w_qkv, qkv, rotation, self.n_heads,
                                                                  self.n_kv, self.head_dim, kv):
            # a prompt: rotation and cache store happen in the projection's epilogue
            ops.linear_qkv_rope(x, self.w_qkv, qkv, rotation, self.n_heads, self.n_kv, kv,
                                ctx.token_seq, ctx.slots, ctx.positions)
            in_attention = False
        else:
            ops.linear(x, self.w_qkv, qkv)
            if ctx.op_hook is not None:
                ctx.trace("q", qkv[:, : self.q_dim].clone())
                if self.own_kv:
                    ctx.trace("k", qkv[:, self.q_dim: self.q_dim + self.kv_dim])
                    ctx.trace("v", qkv[:, self.q_dim + self.kv_dim:])
            if not in_attention:
                ops.rope_kv_store(qkv, rotation, self.n_heads, store, self.head_dim,
                                  kv, ctx.token_seq, ctx.slots, ctx.positions,
                                  pairing=pairing, rotary_dim=rotary_dim)
        q = qkv[:, : self.q_dim]
        if not in_attention:
            ctx.trace("q_attn", q)
        mixed = rt.empty(n, self.q_dim)
        window = self.window or 0
        if rt.dtype == torch.bfloat16 and ops.attention_bf16_supports(self.head_dim):
            if ctx.is_decode:
                new_k = qkv[:, self.q_dim: self.q_dim + self.kv_dim] if store else None
                new_v = qkv[:, self.q_dim + self.kv_dim:] if store else None
                splits, chunk, ring = ops.attention_decode_plan(n, self.n_heads, self.n_kv, self.head_dim,
                                                          ctx.max_kv_len, window, ctx.total_kv_len)
                scratch = None
                if splits > 1:
                    scratch = rt.empty(ops.attention_decode_scratch_floats(
                        n, self.n_heads, self.head_dim, splits), dtype=torch.float32)
                ops.attention_decode_bf16(q, mixed, kv, ctx.slots, ctx.positions, self.n_heads,
                                          self.scale, window, splits, scratch,
                                          unrotated=(rotation, new_k, new_v, True) if in_attention else None,
                                          chunk_pages=chunk, ring_pages=ring)
            elif ops.attention_tcgen05_supports(kv) and qkv.stride(0) % 8 == 0:
                ops.attention_prefill_tcgen05(q, mixed, kv, ctx.cu_seqlens, ctx.slots, ctx.start_pos,
                                              ctx.n_seqs, ctx.max_q_len, self.n_heads, self.scale, window)
            else:
                ops.attention_prefill_bf16(q, mixed, kv, ctx.cu_seqlens, ctx.slots, ctx.start_pos,
                                           ctx.n_seqs, ctx.max_q_len, self.n_heads, self.scale, window)
        else:
            ops.attention_simple(q, mixed, kv, ctx.token_seq, ctx.slots, ctx.positions,
                                 self.n_heads, self.scale, window)
        ctx.trace("attn", mixed)
        return emit_update(mixed, self.w_o, ctx)
