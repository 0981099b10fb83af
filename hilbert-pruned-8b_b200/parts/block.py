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

    # A block with ``folds_norms = True`` takes two more keyword arguments and returns a value, by
    # which norms at the seam between two blocks are folded into the products around them (see
    # ``parts.base.Mixer``): ``prepared`` is what the block in front returned (None: nothing
    # prepared, the block runs its first norm), ``prepare_next`` what the next block's
    # ``fold_request`` said (None: nobody asks).  Other blocks are called without them.
    folds_norms = False

    def fold_request(self, step):
        """What the block in front has to prepare so that this block need not run its first
        norm (``Norm.fold_request`` of that norm, on the buffer this block reads), or None."""
        return None

    def forward(self, x, step, cache, state, append: bool):
        raise NotImplementedError


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    ROLES = {"mixer_norm": NORMS, "mixer": MIXERS, "feed_forward_norm": NORMS, "feed_forward": FEED_FORWARDS}

    def __init__(self, layer_spec, ctx):
        super().__init__(layer_spec, ctx)
        self.mixer_norm, self.mixer = self.parts["mixer_norm"], self.parts["mixer"]
        self.feed_forward_norm, self.feed_forward = self.parts["feed_forward_norm"], self.parts["feed_forward"]

    folds_norms = True

    def _normed(self, step, size: int):
        """The buffer the norms write and the mixer and the feed-forward read."""
        return self.ctx.workspace.buffer("block.h", (self.ctx.max_step_tokens, size), self.ctx.dtype)[:step.num_tokens]

    def _may_fold(self, step, size: int) -> bool:
        ops = self.ctx.ops
        return ops is not None and hasattr(ops, "can_fold_norm") and ops.can_fold_norm(step.num_tokens, size, self.ctx.dtype)

    def fold_request(self, step):
        # the mixer must be able to apply the prepared norm's factor; the norm says how wide the residual stream is
        size = getattr(self.mixer_norm, "size", None)
        if not getattr(self.mixer, "folds_norms", False) or size is None or not self._may_fold(step, size):
            return None
        return self.mixer_norm.fold_request(self._normed(step, size))

    def forward(self, x, step, cache, state, append: bool, prepared=None, prepare_next=None):
        h = self._normed(step, x.shape[1])
        fold = self._may_fold(step, x.shape[1])
        mixer_folds, ff_folds = getattr(self.mixer, "folds_norms", False), getattr(self.feed_forward, "folds_norms", False)
        # x += mixer(norm(x)); the mixer's last product prepares the next norm if the feed-forward can use it
        if prepared is None:
            self.mixer_norm.forward(x, h)
        if mixer_folds:
            request = self.feed_forward_norm.fold_request(h) if fold and ff_folds else None
            prepared = self.mixer.forward(h, x, step, cache, state, append, prepared=prepared, prepare=request)
        else:
            self.mixer.forward(h, x, step, cache, state, append)
            prepared = None
        # x += feed_forward(norm(x)); its last product prepares the next block's first norm if that block asked
        if prepared is None:
            self.feed_forward_norm.forward(x, h)
        if ff_folds:
            return self.feed_forward.forward(h, x, step, prepared=prepared, prepare=prepare_next if fold else None)
        self.feed_forward.forward(h, x, step)
        return None
