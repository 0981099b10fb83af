import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", hidden_size=64, num_hidden_layers=2,
    intermediate_size=176, vocab_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None, tie_word_embeddings=True, max_position_embeddings=128,
    eos_token_id=7)
TINY_B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", hidden_size=160, num_hidden_layers=3,
    intermediate_size=416, vocab_size=384, num_attention_heads=5, num_key_value_heads=1, head_dim=32,
    rms_norm_eps=1e-6, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=32),
    tie_word_embeddings=False, max_position_embeddings=256, eos_token_id=[3, 5])
# Head sizes 64 and 128 take the tensor-core attention kernels; odd group sizes and widths.
TINY_C = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", hidden_size=96, num_hidden_layers=2,
    intermediate_size=208, vocab_size=300, num_attention_heads=3, num_key_value_heads=1, head_dim=64,
    rms_norm_eps=1e-5, rope_theta=10000.0,
    rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=2.0,
                      original_max_position_embeddings=16),
    tie_word_embeddings=False, max_position_embeddings=512)
TINY_D = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", hidden_size=72, num_hidden_layers=2,
    intermediate_size=120, vocab_size=270, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
    rms_norm_eps=1e-6, rope_theta=500000.0, rope_scaling=None, tie_word_embeddings=True,
    max_position_embeddings=512)
# weights: (seed, std, norm_std, fan_in_scale).  "paper" follows the stated N(0, 0.02); "strong"
# scales by fan-in so that every layer moves the logits and a fault in one shows.
WEIGHTS = {"paper_a": (0, 0.02, 0.0, None), "paper_b": (2, 0.02, 0.01, None),
           "strong_a": (10, 0.02, 0.05, 1.0), "strong_b": (12, 0.02, 0.05, 1.0),
           "strong_c": (14, 0.02, 0.05, 1.0), "strong_d": (16, 0.02, 0.05, 1.0)}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (made once, in a temporary place)."""
    import hilbert_pruned_8b_b200 as hb
    out = {}
    for name, cfg in (("a", TINY_A), ("b", TINY_B), ("c", TINY_C), ("d", TINY_D)):
        for kind in ("paper", "strong"):
            if f"{kind}_{name}" not in WEIGHTS:
                continue
            seed, std, norm_std, fan = WEIGHTS[f"{kind}_{name}"]
            d = str(tmp_path_factory.mktemp(f"model_{kind}_{name}"))
            hb.weights.write_random_model(d, hb.LlamaConfig.from_dict(cfg), seed, std=std, norm_std=norm_std,
                                          fan_in_scale=fan)
            out[f"{kind}_{name}"] = d
    return out


def require_gpu():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
