"""Architecture-neutral description of a decoder: what the generic model builder consumes.

A configuration class (one per architecture) turns its ``config.json`` into a ``ModelSpec``.
Nothing below this level knows which architecture it serves: a ``ModelSpec`` is a list of
layers, each naming its mixer, feed-forward and norms with their sizes and constants, plus
the order in which the layers run.

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
    """One decoder layer.

    ``prefix`` is the tensor-name prefix of the layer's weights (``layers.3.``); the part
    names below it (``self_attn.q_proj.weight``) are the parts' own.
    """

    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: str = "prenorm"
    # tensor-name prefixes of the parts below the layer's prefix (model.c:416-428)
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."


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
    # candidate prefixes of the decoder's tensors, tried in order (model.c:394-395)
    weight_prefixes: List[str] = field(default_factory=lambda: ["model.language_model.", "model."])
    stop_token_ids: List[int] = field(default_factory=list)
    max_position: Optional[int] = None
    embedding_prefix: str = "embed_tokens."
    final_norm_prefix: str = "norm."
    head_prefix: str = "lm_head."

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
