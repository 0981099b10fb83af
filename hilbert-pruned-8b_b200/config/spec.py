"""Architecture-neutral description of a decoder: what the generic model builder consumes.

A configuration class (one per architecture) turns its ``config.json`` into a ``ModelSpec``.
Nothing below this level knows which architecture it serves: a ``ModelSpec`` is a list of
layers, each naming its block (the arrangement) and the block's parts (mixer, feed-forward,
norms, ...) with their sizes and constants, plus the order in which the layers run.

The reference keeps a per-layer type array and per-kind counters for the same purpose
(cleanroom-transformer/src/transformer.h:275,289-290,307-318); here the per-layer choice is
a full part description, so that two layers of one model may differ in every part.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered ``kind`` and its parameters (sizes, constants)."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: the registered ``block`` (the arrangement) and the parts it arranges.

    ``parts`` maps a role name to the part in that role; which roles exist is the block's
    business (the pre-norm block asks for ``mixer``, ``feed_forward``, ``mixer_norm`` and
    ``feed_forward_norm``; a block of another shape names its own and this class does not
    change).  ``prefix`` is the tensor-name prefix of the layer's weights (``layers.3.``),
    ``part_prefixes[role]`` the prefix of a part's tensors below it (``self_attn.``); the
    names below that (``q_proj.weight``) are the part's own.  The architecture's
    configuration supplies all of them: none is a default of this file.
    """

    prefix: str
    parts: Dict[str, PartSpec]
    part_prefixes: Dict[str, str]
    block: str = "prenorm"

    def part(self, role: str) -> PartSpec:
        if role not in self.parts:
            raise KeyError(f"layer {self.prefix!r} ({self.block}) has no part in the role {role!r} "
                           f"({', '.join(sorted(self.parts))})")
        return self.parts[role]

    def part_prefix(self, role: str) -> str:
        return self.part_prefixes.get(role, role + ".")

    def with_part(self, role: str, spec: PartSpec, prefix: Optional[str] = None) -> "LayerSpec":
        """A copy with the part in ``role`` replaced (or added) and, if given, its tensor prefix."""
        parts = {**self.parts, role: spec}
        prefixes = dict(self.part_prefixes) if prefix is None else {**self.part_prefixes, role: prefix}
        return LayerSpec(self.prefix, parts, prefixes, self.block)

    def with_block(self, block: str) -> "LayerSpec":
        return LayerSpec(self.prefix, dict(self.parts), dict(self.part_prefixes), block)

    # the two roles most layers have, by name (a block without one of them raises KeyError)
    @property
    def mixer(self) -> PartSpec:
        return self.part("mixer")

    @property
    def feed_forward(self) -> PartSpec:
        return self.part("feed_forward")


@dataclass(frozen=True)
class PlanEntry:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (whose weights run); a layer may appear in the
    plan more than once.  Cache storage and per-sequence state belong to the plan entry, so
    a layer that runs twice keeps two sets of keys and values.  ``cache_of`` is the index of
    an EARLIER plan entry whose cache this entry reads instead of keeping its own: it then
    appends nothing.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: List[LayerSpec]
    plan: List[PlanEntry]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    # candidate prefixes of the decoder's tensors, tried in order: the first under which the
    # embedding table exists is the checkpoint's, else the last
    weight_prefixes: List[str]
    # tensor-name prefixes of the parts outside the layers, below the decoder's prefix
    embedding_prefix: str
    final_norm_prefix: str
    head_prefix: str
    stop_token_ids: List[int] = field(default_factory=list)
    # the longest sequence the checkpoint was made for (None: not stated); the generation loop
    # ends a request there, the step function does not read it
    max_position: Optional[int] = None

    def validate(self) -> None:
        n = len(self.layers)
        if not self.plan:
            raise ValueError("model spec: empty layer plan")
        for i, e in enumerate(self.plan):
            if not 0 <= e.layer < n:
                raise ValueError(f"model spec: plan entry {i} names layer {e.layer} outside 0..{n - 1}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(
                        f"model spec: plan entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if self.plan[e.cache_of].cache_of is not None:
                    raise ValueError(
                        f"model spec: plan entry {i} reads the cache of entry {e.cache_of}, which keeps none of its own")
