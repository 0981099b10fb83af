"""The arrangement of norm, mixer and feed-forward in a layer.

``prenorm``: ``x += mixer(norm_a(x)); x += feed_forward(norm_b(x))`` with the residual
stream ``x`` in 32-bit (cleanroom-transformer/src/cpu_backend.c:237-252, cuda_backend.cu:628).
"""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS


@BLOCKS.register("prenorm")
class PreNormBlock:
    def __init__(self, layer_spec, ctx):
        self.spec = layer_spec
        self.ctx = ctx
        self.mixer_norm = NORMS.build(layer_spec.mixer_norm, ctx)
        self.mixer = MIXERS.build(layer_spec.mixer, ctx)
        self.feed_forward_norm = NORMS.build(layer_spec.feed_forward_norm, ctx)
        self.feed_forward = FEED_FORWARDS.build(layer_spec.feed_forward, ctx)

    def named_parts(self):
        """(name prefix below the layer's prefix, part) for every part that owns weights."""
        s = self.spec
        return [(s.mixer_norm_prefix, self.mixer_norm), (s.mixer_prefix, self.mixer),
                (s.feed_forward_norm_prefix, self.feed_forward_norm), (s.feed_forward_prefix, self.feed_forward)]

    def forward(self, x, step, cache, state, append: bool) -> None:
        ws, T = self.ctx.workspace, step.num_tokens
        h = ws.buffer("block.h", (self.ctx.max_step_tokens, x.shape[1]), self.ctx.dtype)[:T]
        self.mixer_norm.forward(x, h)
        self.mixer.forward(h, x, step, cache, state, append)
        self.feed_forward_norm.forward(x, h)
        self.feed_forward.forward(h, x, step)
