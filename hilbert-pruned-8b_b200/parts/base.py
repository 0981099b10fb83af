"""Interfaces and registries of the parts a decoder layer is put together from.

Kinds of part: mixer (attention, or anything else that mixes tokens of a sequence),
feed-forward, norm, position encoding, block (the arrangement of the four in a layer),
embedding and head.  Each kind has one registry from a name to a class; a configuration
chooses parts by name, layer by layer.  No part knows which model it is in: sizes and
constants arrive as parameters of its ``PartSpec``.

What a part must provide:

* ``params()``: its weight tensors as ``ParamSpec`` rows (name local to the part, shape,
  kind).  The loader, the random-weights mode and the byte accounting all read this one
  table, as the reference does with its shape table
  (cleanroom-transformer/src/shapes.c:12-39, model.c:246-257).
* ``bind(tensors)``: receives the loaded tensors by local name and may fuse them.
* mixers: ``cache_need()`` (keys and values per token, or None), ``state_need()``
  (fixed-size state per sequence, or None) and
  ``forward(h, residual, step, cache, state, append)`` which ADDS the mixer's output to the
  32-bit ``residual`` in place.
* feed-forwards: ``forward(h, residual, step)``, adding likewise.
* norms: ``forward(x, out, rows=None)``.
* position encodings: ``rotation_table(step)`` when the encoding is a rotation of pairs of
  head dimensions by position-dependent angles (the kernels then turn queries and keys
  themselves), else ``apply(q, k, step)`` which turns them in place; see ``PositionEncoding``.
* blocks (``parts/block.py``): ``ROLES``, ``named_parts()``, ``cache_need()``, ``state_need()``,
  ``forward(x, step, cache, state, append)``.
* optional, ``folds_norms = True`` on mixers, feed-forwards and blocks: the norms between two
  matrix products may be folded into them for steps of few tokens; see ``Mixer`` and
  ``Norm.fold_request`` below and ``Block`` in ``parts/block.py``.
* ``graph_safe`` (class attribute, default True): whether ``forward`` only enqueues work on
  the current stream, so that a decode step can be captured in a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..config.spec import PartSpec


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"        # "matrix" | "vector" | "int_table"
    init: str = "normal"        # random-weights mode: "normal" | "ones" | "zeros"
    absolute: bool = False      # name is not below the decoder's prefix (lm_head.weight)
    optional: bool = False      # may be absent (and is then not an error)


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values a mixer keeps per token: ``window`` None keeps all of them."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state a mixer keeps per sequence (zeroed when a sequence starts)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class BuildContext:
    """What parts need to build themselves: device, activation dtype, kernels, scratch."""

    device: torch.device
    dtype: torch.dtype                      # torch.bfloat16 or torch.float32
    ops: Any                                # the kernel library (kernels.ops)
    workspace: Any                          # engine.workspace.Workspace
    max_step_tokens: int
    _shared: Dict[str, Any] = None          # parts shared between layers, by spec

    def shared_part(self, registry: "Registry", spec: PartSpec) -> Any:
        if self._shared is None:
            self._shared = {}
        key = registry.kind + ":" + repr(spec)
        if key not in self._shared:
            self._shared[key] = registry.build(spec, self)
        return self._shared[key]


class Part:
    # False for a part whose forward reads device values on the host or allocates: the engine
    # then runs its decode steps eagerly instead of replaying a captured CUDA graph
    graph_safe = True

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx

    def params(self) -> List[ParamSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads from this part (for roofline accounting)."""
        return 0


class Mixer(Part):
    """Reads the normed input ``h``, adds its result to the 32-bit ``residual``.

    A part with ``folds_norms = True`` also takes two keyword arguments, by which a block folds
    the norms around it into its matrix products for steps of few tokens (no norm kernel):
    ``prepared`` (a ``kernels.ops.PreparedNorm``: ``h`` holds the norm's input times the norm's
    weight WITHOUT the per-token factor, which the part's first product applies to its rows),
    and ``prepare`` (what ``Norm.fold_request`` returned for the norm that reads ``residual``
    next: the part's last product fills that norm's buffer).  ``forward`` then returns the
    ``PreparedNorm`` for the next reader, or None when it prepared nothing (the block runs the
    norm).  Parts without the attribute are called without the two arguments."""

    folds_norms = False

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, h, residual, step, cache, state, append: bool):
        raise NotImplementedError


class FeedForward(Part):
    """As ``Mixer``: reads ``h``, adds to ``residual``; ``folds_norms`` as there."""

    folds_norms = False

    def forward(self, h, residual, step):
        raise NotImplementedError


class Norm(Part):
    out_dtype: torch.dtype

    def forward(self, x, out, rows=None) -> None:
        raise NotImplementedError

    def fold_request(self, out):
        """What the product that writes this norm's input needs in order to prepare it
        (``Ops.linear(..., prepare=...)``): ``(weight, offset, eps, out)`` for a norm of the form
        ``x * rsqrt(mean(x^2) + eps) * (offset + weight)``; None: the norm cannot be folded."""
        return None


class PositionEncoding(Part):
    """How a mixer's queries and keys learn their positions.  A mixer uses one of two forms:

    * ``rotation_table(step)`` returns ``(table, rotary_dim)``: ``table[t, i] = (cos a, sin a)``
      in 32-bit, ``[tokens, rotary_dim / 2, 2]``, for the step's token ``t`` and the pair
      ``(i, i + rotary_dim / 2)`` of every head; the attention kernels turn queries and keys by
      it (dimensions from ``rotary_dim`` on stay).  ``fusable`` says whether a kernel that does
      more than turning (decode attention that also appends and attends) may take the table;
      a part sets it False to keep the rotation a step of its own.
    * ``rotation_table`` returns None: the encoding is something else, and ``apply(q, k, step)``
      changes ``q [tokens, heads, head_dim]`` and ``k [tokens, kv_heads, head_dim]`` (views of
      the step's projections) in place before the keys are cached; no kernel rotates.

    ``prepare(step)`` may compute what all layers of a step share into ``step.shared``."""

    fusable = True

    def prepare(self, step) -> None:
        pass

    def rotation_table(self, step):
        return None

    def apply(self, q, k, step) -> None:
        raise NotImplementedError(f"{type(self).__name__} gives neither a rotation table nor apply()")


class Registry:
    def __init__(self, kind: str):
        self.kind = kind
        self._classes: Dict[str, Callable[..., Any]] = {}

    def register(self, name: str) -> Callable[[Any], Any]:
        def deco(cls):
            self._classes[name] = cls
            return cls
        return deco

    def unregister(self, name: str) -> None:
        self._classes.pop(name, None)

    def names(self) -> List[str]:
        return sorted(self._classes)

    def get(self, name: str) -> Callable[..., Any]:
        if name not in self._classes:
            raise KeyError(f"no {self.kind} named {name!r} is registered ({', '.join(self.names())})")
        return self._classes[name]

    def build(self, spec: PartSpec, ctx: BuildContext) -> Any:
        return self.get(spec.kind)(spec, ctx)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
