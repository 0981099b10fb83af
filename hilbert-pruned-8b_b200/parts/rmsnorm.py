"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * (offset + w)``.

Formula and the place of ``offset`` (0 for a plain weight, 1 for a zero-centred one) follow
cleanroom-transformer/src/cpu_backend.c:56-62; the sum of squares and the scaling are done in
32-bit on the device (cuda_backend.cu:73-85), the result is written in the dtype the next
matrix product reads.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import NORMS, Norm, ParamSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.get("offset", 0.0))
        self.weight = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self.size,), kind="vector", init="ones")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        # widened once at load, exactly (model.c:259-281)
        self.weight = tensors["weight"].reshape(self.size).to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.size * 4

    def forward(self, x, out, rows=None) -> None:
        """``out[i] = norm(x[rows[i]])`` (``rows`` None: every row of ``x``)."""
        self.ctx.ops.rmsnorm(x, self.weight, self.eps, self.offset, out, rows)

    def fold_request(self, out):
        return (self.weight, self.offset, self.eps, out)
