"""Typed configuration of the Llama 3 dense decoder, read from config.json keys.

Keys, defaults and error conditions follow the reference's parser
(cleanroom-transformer/src/model.c:19-58 rope and integer rules, :109-175 Llama branch).
Keys the reference never reads but a generation library needs (``max_position_embeddings``,
``eos_token_id``, ``bos_token_id``, ``torch_dtype``) are optional additions.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, PlanEntry


def _is_number(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _need_int(cfg: Dict[str, Any], key: str) -> int:
    # model.c:19-25: a number, integral, 1..1e9
    v = cfg.get(key)
    if not _is_number(v) or v < 1 or v > 1e9 or v != math.floor(v):
        raise ConfigError(f"config: missing or bad {key}")
    return int(v)


def _flag(cfg: Dict[str, Any], key: str, default: bool) -> bool:
    # model.c:27-31: anything but a JSON boolean keeps the default
    v = cfg.get(key)
    return v if isinstance(v, bool) else default


@dataclass(frozen=True)
class Llama3RopeScaling:
    """The four numbers of ``rope_type: llama3`` (model.c:47-55)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: float


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    vocab_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[Llama3RopeScaling] = None
    partial_rotary_factor: float = 1.0
    tie_word_embeddings: bool = False
    max_position_embeddings: Optional[int] = None
    eos_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None

    architecture = "LlamaForCausalLM"
    model_type = "llama"

    # ------------------------------------------------------------------ derived
    @property
    def rotary_dim(self) -> int:
        # model.c:156: (uint32)(head_dim * partial) & ~1
        return int(self.head_dim * self.partial_rotary_factor) & ~1

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, root: Dict[str, Any]) -> "LlamaConfig":
        if not isinstance(root, dict):
            raise ConfigError("config: config.json is not an object")
        tc = root.get("text_config")
        cfg = tc if isinstance(tc, dict) else root  # model.c:128-129
        act = cfg.get("hidden_act")
        if act is not None and act != "silu":
            raise ConfigError("config: only silu activations are supported")  # model.c:138-142
        hidden = _need_int(cfg, "hidden_size")
        layers = _need_int(cfg, "num_hidden_layers")
        inter = _need_int(cfg, "intermediate_size")
        vocab = _need_int(cfg, "vocab_size")
        heads = _need_int(cfg, "num_attention_heads")
        kv_heads = _need_int(cfg, "num_key_value_heads")
        if cfg.get("head_dim") is not None:  # model.c:147-151 (null allowed)
            head_dim = _need_int(cfg, "head_dim")
        else:
            head_dim = hidden // heads
        eps = cfg.get("rms_norm_eps")
        eps = float(eps) if _is_number(eps) else 1e-6  # model.c:152-154

        # rope: rope_parameters (newer) or rope_scaling (older); theta may sit at top level
        rope = cfg.get("rope_parameters")
        if not isinstance(rope, dict):
            rope = cfg.get("rope_scaling")
        if not isinstance(rope, dict):
            rope = None
        theta = 10000.0
        partial = 1.0
        if rope is not None and _is_number(rope.get("rope_theta")):
            theta = float(rope["rope_theta"])
        elif _is_number(cfg.get("rope_theta")):
            theta = float(cfg["rope_theta"])
        if rope is not None and _is_number(rope.get("partial_rotary_factor")):
            partial = float(rope["partial_rotary_factor"])
        elif _is_number(cfg.get("partial_rotary_factor")):
            partial = float(cfg["partial_rotary_factor"])
        scaling = None
        rtype = None
        if rope is not None:
            rtype = rope.get("rope_type", rope.get("type"))
        if rtype is not None and rtype != "default":
            if rtype == "llama3":
                keys = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
                if not all(_is_number(rope.get(k)) for k in keys):
                    raise ConfigError("config: incomplete llama3 rope scaling")
                scaling = Llama3RopeScaling(*(float(rope[k]) for k in keys))
            else:
                raise ConfigError(f"config: rope_type {rtype if isinstance(rtype, str) else '?'} is not supported")

        tied = _flag(cfg, "tie_word_embeddings", _flag(root, "tie_word_embeddings", False))  # model.c:157
        if _flag(cfg, "attention_bias", False) or _flag(cfg, "mlp_bias", False):
            raise ConfigError("config: Llama checkpoints with attention or MLP biases are not supported")

        max_pos = cfg.get("max_position_embeddings")
        max_pos = int(max_pos) if _is_number(max_pos) and max_pos >= 1 else None
        eos = cfg.get("eos_token_id", root.get("eos_token_id"))
        if _is_number(eos):
            eos_ids = [int(eos)]
        elif isinstance(eos, list):
            eos_ids = [int(e) for e in eos if _is_number(e)]
        else:
            eos_ids = []
        bos = cfg.get("bos_token_id", root.get("bos_token_id"))
        dtype = cfg.get("torch_dtype", cfg.get("dtype", root.get("torch_dtype")))

        out = cls(hidden_size=hidden, num_hidden_layers=layers, intermediate_size=inter, vocab_size=vocab,
                  num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=eps,
                  rope_theta=theta, rope_scaling=scaling, partial_rotary_factor=partial,
                  tie_word_embeddings=tied, max_position_embeddings=max_pos, eos_token_ids=eos_ids,
                  bos_token_id=int(bos) if _is_number(bos) else None,
                  torch_dtype=dtype if isinstance(dtype, str) else None)
        out.validate()
        return out

    def validate(self) -> None:
        # model.c:158-161
        if (self.num_hidden_layers > 256 or self.num_attention_heads % self.num_key_value_heads
                or self.rotary_dim > self.head_dim or self.rotary_dim == 0):
            raise ConfigError("config: unsupported head layout")
        for e in self.eos_token_ids:
            if not 0 <= e < self.vocab_size:
                raise ConfigError(f"config: eos_token_id {e} is outside the vocabulary")

    @classmethod
    def from_json_file(cls, path: str) -> "LlamaConfig":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_act": "silu",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            d["rope_scaling"] = {
                "rope_type": "llama3", "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": int(s.original_max_position_embeddings),
            }
        else:
            d["rope_scaling"] = None
        if self.partial_rotary_factor != 1.0:
            d["partial_rotary_factor"] = self.partial_rotary_factor
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.torch_dtype is not None:
            d["torch_dtype"] = self.torch_dtype
        return d

    # ------------------------------------------------------------------ model description
    def model_spec(self) -> ModelSpec:
        """The decoder as a list of parts: every layer is RMSNorm -> grouped-query causal
        attention with rotary positions -> RMSNorm -> SwiGLU, residual around each half
        (cleanroom-transformer/src/cpu_backend.c:237-252)."""
        rope_params: Dict[str, Any] = {
            "head_dim": self.head_dim, "rotary_dim": self.rotary_dim, "theta": self.rope_theta}
        if self.rope_scaling is not None:
            s = self.rope_scaling
            rope_params["llama3"] = {
                "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings}
        rope = PartSpec("rotary", rope_params)
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps, "offset": 0.0})
        mixer = PartSpec("attention", {
            "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "window": None, "position": rope})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        # tensor names below ``layers.{i}.`` (model.c:416-428)
        prefixes = {"mixer": "self_attn.", "feed_forward": "mlp.", "mixer_norm": "input_layernorm.",
                    "feed_forward_norm": "post_attention_layernorm."}
        layers = [LayerSpec(prefix=f"layers.{i}.", block="prenorm", part_prefixes=dict(prefixes),
                            parts={"mixer": mixer, "feed_forward": ffn, "mixer_norm": norm, "feed_forward_norm": norm})
                  for i in range(self.num_hidden_layers)]
        plan = [PlanEntry(i) for i in range(self.num_hidden_layers)]
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            layers=layers, plan=plan,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            final_norm=norm,
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                      "tied": self.tie_word_embeddings}),
            # model.c:394-406: the decoder's tensors sit below one of two prefixes; the head has none
            weight_prefixes=["model.language_model.", "model."], embedding_prefix="embed_tokens.",
            final_norm_prefix="norm.", head_prefix="lm_head.",
            stop_token_ids=list(self.eos_token_ids), max_position=self.max_position_embeddings)
        spec.validate()
        return spec
