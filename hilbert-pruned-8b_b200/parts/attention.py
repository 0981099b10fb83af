"""Grouped-query causal attention over the paged key/value cache.

Per token: ``q,k,v = h Wq^T, h Wk^T, h Wv^T`` (no biases); the position encoding turns
every q head and k head; k and v go to the cache at the token's position; query head j
reads key/value head ``j // (heads/kv_heads)``; scores ``q.k / sqrt(head_dim)`` over the
keys ``0..position`` (optionally only the last ``window``), softmax in 32-bit, weighted sum
of values; ``residual += attn Wo^T`` (cleanroom-transformer/src/cpu_backend.c:77-133,242;
shapes shapes.c:23-26).  The three projections are one matrix product over the row-wise
concatenation of the weights.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .base import MIXERS, POSITION_ENCODINGS, CacheNeed, Mixer, ParamSpec


@MIXERS.register("attention")
class Attention(Mixer):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window: Optional[int] = p.get("window")
        if self.heads % self.kv_heads:
            raise ValueError("attention: heads must be a multiple of kv heads")
        self.scale = 1.0 / math.sqrt(float(self.head_dim))
        pos = p.get("position")
        self.position = ctx.shared_part(POSITION_ENCODINGS, pos) if pos is not None else None
        self.graph_safe = getattr(self.position, "graph_safe", True)      # a step is as capturable as its parts
        # whether decode steps may run the kernel that rotates, appends and attends in one launch
        # (the part decides; the kernel library only says whether it can)
        self.fuse_decode = bool(p.get("fuse_decode", True))
        self.q_width = self.heads * self.head_dim
        self.kv_width = self.kv_heads * self.head_dim
        self.w_qkv = None
        self.w_o = None

    def params(self) -> List[ParamSpec]:
        return [
            ParamSpec("q_proj.weight", (self.q_width, self.hidden)),
            ParamSpec("k_proj.weight", (self.kv_width, self.hidden)),
            ParamSpec("v_proj.weight", (self.kv_width, self.hidden)),
            ParamSpec("o_proj.weight", (self.hidden, self.q_width)),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, k, v = tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError("attention: q, k and v projections are stored in different dtypes")
        pack = self.ctx.ops.pack_weight
        self.w_qkv = pack(torch.cat([q, k, v], dim=0).contiguous())
        self.w_o = pack(tensors["o_proj.weight"].contiguous())

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o))

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.kv_heads, self.head_dim, self.window)

    folds_norms = True

    def forward(self, h, residual, step, cache, state, append: bool, prepared=None, prepare=None):
        ops, ws, T = self.ctx.ops, self.ctx.workspace, step.num_tokens
        cap = self.ctx.max_step_tokens
        width = self.q_width + 2 * self.kv_width
        qkv = ws.buffer("attention.qkv", (cap, width), self.ctx.dtype)[:T]
        if append:
            ops.linear(h, self.w_qkv, qkv, scale=prepared)
        else:
            # a layer that reads another layer's cache needs its queries only
            w_q = self.w_qkv.first_rows(self.q_width) if hasattr(self.w_qkv, "first_rows") else self.w_qkv[: self.q_width]
            ops.linear(h, w_q, qkv[:, : self.q_width], scale=prepared)
        # positions: a table of rotations that the kernels apply, or the part turns q and k itself
        table, rot = None, 0
        fusable = self.fuse_decode
        if self.position is not None:
            rotation = self.position.rotation_table(step)
            if rotation is None:
                q = qkv[:, : self.q_width].unflatten(1, (self.heads, self.head_dim))
                k = qkv[:, self.q_width: self.q_width + self.kv_width].unflatten(1, (self.kv_heads, self.head_dim))
                self.position.apply(q, k if append else None, step)
            else:
                table, rot = rotation
                fusable = fusable and self.position.fusable
        attn = ws.buffer("attention.out", (cap, self.q_width), self.ctx.dtype)[:T]
        if fusable and ops.can_fuse_decode_attention(qkv, self.heads, self.kv_heads, self.head_dim, cache, step, attn):
            # one token per sequence: rotation, append and attention are one launch
            ops.attention_decode_fused(qkv, table, rot, self.heads, self.kv_heads, self.head_dim, cache, step, attn,
                                       self.scale, self.window, append)
        else:
            ops.rope_kv_append(qkv, table, rot, self.heads, self.kv_heads, self.head_dim, cache, step, append)
            ops.attention(qkv, self.heads, self.kv_heads, self.head_dim, cache, step, attn, self.scale, self.window)
        return ops.linear(attn, self.w_o, residual, accumulate=True, prepare=prepare)
