"""The arrangement of the parts of a layer.

A block is built from a ``LayerSpec``: it declares the roles it fills (``ROLES``: role name
-> the registry the part in that role comes from), builds them, and runs them in its order.
What the model needs of a block: ``named_parts()`` for the weight table, ``cache_need()``
and ``state_need()`` for the cache, and ``forward``.

``prenorm``: ``x += mixer(norm_a(x)); x += feed_forward(norm_b(x))`` with the residual
stream ``x`` in 32-bit (cleanroom-transformer/src/cpu_backend.c:237-252, cuda_backend.cu:628).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, CacheNeed, Registry, StateNeed


class Block:
    """Base of the arrangements: builds the parts that ``ROLES`` names from the layer's spec."""

    ROLES: Dict[str, Registry] = {}

    def __init__(self, layer_spec, ctx):
        self.spec = layer_spec
        self.ctx = ctx
        extra = sorted(set(layer_spec.parts) - set(self.ROLES))
        if extra:
            raise ValueError(f"block {layer_spec.block!r} has no role for the parts {extra} of layer "
                             f"{layer_spec.prefix!r} (its roles: {', '.join(self.ROLES)})")
        self.parts = {role: registry.build(layer_spec.part(role), ctx) for role, registry in self.ROLES.items()}
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in self.parts.values())

    def named_parts(self) -> List[Tuple[str, object]]:
        """(name prefix below the layer's prefix, part) for every part that may own weights."""
        return [(self.spec.part_prefix(role), part) for role, part in self.parts.items()]

    # the cache belongs to the part that mixes tokens, if the block has one
    def cache_need(self) -> Optional[CacheNeed]:
        mixer = self.parts.get("mixer")
        return mixer.cache_need() if mixer is not None else None

    def state_need(self) -> Optional[StateNeed]:
        mixer = self.parts.get("mixer")
        return mixer.state_need() if mixer is not None else None

    def forward(self, x, step, cache, state, append: bool) -> None:
        raise NotImplementedError


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    ROLES = {"mixer_norm": NORMS, "mixer": MIXERS, "feed_forward_norm": NORMS, "feed_forward": FEED_FORWARDS}

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        self.mixer_norm, self.mixer = self.parts["mixer_norm"], self.parts["mixer"]
        self.feed_forward_norm, self.feed_forward = self.parts["feed_forward_norm"], self.parts["feed_forward"]

    def forward(self, x, step, cache, state, append: bool) -> None:
        ws, T = self.ctx.workspace, step.num_tokens
        h = ws.buffer("block.h", (self.ctx.max_step_tokens, x.shape[1]), self.ctx.dtype)[:T]
        self.mixer_norm.forward(x, h)
        self.mixer.forward(h, x, step, cache, state, append)
        self.feed_forward_norm.forward(x, h)
        self.feed_forward.forward(h, x, step)
