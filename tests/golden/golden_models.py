"""The two tiny models of the golden comparison, with weights from an integer hash.

Every weight is ``k / 128 * scale`` with an 8-bit integer k from a 32-bit mixing function of
(tensor number, element index): exactly representable in bfloat16 and the same on every
machine, so the stored reference logits stay valid without storing any weights.
"""
import json
import os

import numpy as np
import torch

GOLDEN_MODELS = {
    "golden_a": {
        "config": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
                   "hidden_size": 64, "num_hidden_layers": 2, "intermediate_size": 176, "vocab_size": 256,
                   "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rms_norm_eps": 1e-5,
                   "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": True,
                   "max_position_embeddings": 128},
        "seed": 11, "n_tokens": 40, "prefix_lengths": [1, 7, 16, 40],
    },
    "golden_b": {
        "config": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
                   "hidden_size": 160, "num_hidden_layers": 3, "intermediate_size": 416, "vocab_size": 384,
                   "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 32, "rms_norm_eps": 1e-6,
                   "rope_theta": 500000.0,
                   "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                    "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
                   "tie_word_embeddings": False, "max_position_embeddings": 256},
        "seed": 23, "n_tokens": 64, "prefix_lengths": [1, 5, 33, 64],
    },
}


def _mix(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint64)
    x = (x ^ (x >> np.uint64(16))) * np.uint64(0x45D9F3B) & np.uint64(0xFFFFFFFF)
    x = (x ^ (x >> np.uint64(16))) * np.uint64(0x45D9F3B) & np.uint64(0xFFFFFFFF)
    return (x ^ (x >> np.uint64(16))) & np.uint64(0xFFFFFFFF)


def hashed(shape, tensor_no: int, seed: int, scale: float, centre: float = 0.0) -> torch.Tensor:
    n = int(np.prod(shape))
    idx = np.arange(n, dtype=np.uint64) + np.uint64((tensor_no * 0x9E3779B1 + seed * 0x85EBCA6B) & 0xFFFFFFFF)
    k = (_mix(idx) & np.uint64(0xFF)).astype(np.int64) - 128
    vals = centre + k.astype(np.float64) / 128.0 * scale
    return torch.from_numpy(vals.reshape(shape)).to(torch.float32).to(torch.bfloat16)


def golden_names(cfg: dict):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    names = [("model.embed_tokens.weight", (V, H), "m")]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        names += [(p + "input_layernorm.weight", (H,), "n"), (p + "post_attention_layernorm.weight", (H,), "n"),
                  (p + "self_attn.q_proj.weight", (nh * hd, H), "m"), (p + "self_attn.k_proj.weight", (nkv * hd, H), "m"),
                  (p + "self_attn.v_proj.weight", (nkv * hd, H), "m"), (p + "self_attn.o_proj.weight", (H, nh * hd), "m"),
                  (p + "mlp.gate_proj.weight", (I, H), "m"), (p + "mlp.up_proj.weight", (I, H), "m"),
                  (p + "mlp.down_proj.weight", (H, I), "m")]
    names.append(("model.norm.weight", (H,), "n"))
    if not cfg["tie_word_embeddings"]:
        names.append(("lm_head.weight", (V, H), "m"))
    return names


def write_golden_model(model_dir: str, spec: dict) -> None:
    from safetensors.torch import save_file
    os.makedirs(model_dir, exist_ok=True)
    cfg = spec["config"]
    tensors = {}
    for no, (name, shape, kind) in enumerate(golden_names(cfg)):
        if kind == "n":
            tensors[name] = hashed(shape, no, spec["seed"], 0.25, centre=1.0)
        else:
            # about 1/sqrt(fan_in) in size, a power of two so that the values stay exact
            scale = 2.0 ** round(np.log2(1.7 / np.sqrt(shape[1])))
            tensors[name] = hashed(shape, no, spec["seed"], scale)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(tensors, os.path.join(model_dir, "model.safetensors"))


def golden_tokens(spec: dict):
    n, vocab = spec["n_tokens"], spec["config"]["vocab_size"]
    h = _mix(np.arange(n, dtype=np.uint64) + np.uint64(spec["seed"] * 7919))
    return [int(x) for x in (h % np.uint64(vocab))]
