"""SwiGLU feed-forward: ``residual += (silu(h Wg^T) * (h Wu^T)) Wd^T`` with
``silu(z) = z / (1 + exp(-z))`` (cleanroom-transformer/src/cpu_backend.c:247-251,
ops_common.h:56; shapes shapes.c:34-36).  Gate and up weights are concatenated row-wise so
that one matrix product (with the activation in its epilogue where the tensor-core kernel
applies) makes both.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def params(self) -> List[ParamSpec]:
        return [
            ParamSpec("gate_proj.weight", (self.inter, self.hidden)),
            ParamSpec("up_proj.weight", (self.inter, self.hidden)),
            ParamSpec("down_proj.weight", (self.hidden, self.inter)),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError("swiglu: gate and up projections are stored in different dtypes")
        pack = self.ctx.ops.pack_weight
        self.w_gate_up = pack(torch.cat([g, u], dim=0).contiguous(), swiglu=True)
        self.w_down = pack(tensors["down_proj.weight"].contiguous())

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    folds_norms = True

    def forward(self, h, residual, step, prepared=None, prepare=None):
        ops, ws, T = self.ctx.ops, self.ctx.workspace, step.num_tokens
        cap = self.ctx.max_step_tokens
        act = ws.buffer("swiglu.act", (cap, self.inter), self.ctx.dtype)[:T]
        ops.linear_swiglu(h, self.w_gate_up, act, ws, cap, scale=prepared)
        return ops.linear(act, self.w_down, residual, accumulate=True, prepare=prepare)
