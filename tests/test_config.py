"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

import hilbert_pruned_8b_b200 as hb
from conftest import TINY_A, TINY_B
from hilbert_pruned_8b_b200.config import (ConfigError, LlamaConfig, config_class_for, load_config,
                                           register_architecture, unregister_architecture)


def test_tiny_configs_parse_and_differ():
    a, b = LlamaConfig.from_dict(TINY_A), LlamaConfig.from_dict(TINY_B)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 2, 4, 2, 16)
    assert (b.hidden_size, b.num_hidden_layers, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (160, 3, 5, 1, 32)
    assert a.rope_scaling is None and b.rope_scaling.factor == 8.0 and b.rope_scaling.original_max_position_embeddings == 32
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.eos_token_ids == [7] and b.eos_token_ids == [3, 5]
    assert a.rms_norm_eps == 1e-5 and b.rms_norm_eps == 1e-6


def test_defaults_follow_the_reference():
    cfg = dict(model_type="llama", hidden_size=64, num_hidden_layers=1, intermediate_size=32, vocab_size=10,
               num_attention_heads=4, num_key_value_heads=4)
    c = LlamaConfig.from_dict(cfg)
    assert c.head_dim == 16 and c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert not c.tie_word_embeddings and c.rotary_dim == 16
    c = LlamaConfig.from_dict(dict(cfg, head_dim=None, rope_parameters={"rope_theta": 5e5, "rope_type": "default"}))
    assert c.head_dim == 16 and c.rope_theta == 5e5 and c.rope_scaling is None
    c = LlamaConfig.from_dict(dict(cfg, head_dim=24, partial_rotary_factor=0.5))
    assert c.head_dim == 24 and c.rotary_dim == 12
    c = LlamaConfig.from_dict({"text_config": cfg, "tie_word_embeddings": True})
    assert c.tie_word_embeddings


@pytest.mark.parametrize("change,message", [
    ({"hidden_size": None}, "missing or bad hidden_size"),
    ({"num_key_value_heads": None}, "missing or bad num_key_value_heads"),
    ({"vocab_size": 2.5}, "missing or bad vocab_size"),
    ({"num_hidden_layers": 0}, "missing or bad num_hidden_layers"),
    ({"hidden_act": "gelu"}, "only silu"),
    ({"num_key_value_heads": 3}, "unsupported head layout"),
    ({"num_hidden_layers": 300}, "unsupported head layout"),
    ({"attention_bias": True}, "biases are not supported"),
    ({"mlp_bias": True}, "biases are not supported"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type yarn is not supported"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "incomplete llama3 rope scaling"),
    ({"eos_token_id": 100000}, "outside the vocabulary"),
])
def test_bad_configs_are_refused(change, message):
    cfg = copy.deepcopy(TINY_A)
    for k, v in change.items():
        if v is None:
            cfg.pop(k)
        else:
            cfg[k] = v
    with pytest.raises(ConfigError, match=message):
        LlamaConfig.from_dict(cfg)


def test_registry_by_architecture_then_model_type(tmp_path):
    assert config_class_for(TINY_A) is LlamaConfig
    assert config_class_for({"model_type": "llama"}) is LlamaConfig
    with pytest.raises(ConfigError, match="architecture MistralForCausalLM is not supported"):
        config_class_for({"architectures": ["MistralForCausalLM"], "model_type": "llama"})
    with pytest.raises(ConfigError, match="model_type qwen3_5 is not supported"):
        config_class_for({"model_type": "qwen3_5"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(str(tmp_path)) == LlamaConfig.from_dict(TINY_B)
    with pytest.raises(ConfigError, match="cannot open"):
        load_config(str(tmp_path / "nowhere"))


def test_a_new_architecture_registers_without_touching_the_library():
    class ToyConfig:
        architecture = "ToyForCausalLM"
        model_type = "toy"

        @classmethod
        def from_dict(cls, root):
            return cls()

    register_architecture(ToyConfig)
    try:
        assert config_class_for({"architectures": ["ToyForCausalLM"]}) is ToyConfig
        assert config_class_for({"model_type": "toy"}) is ToyConfig
    finally:
        unregister_architecture(ToyConfig)
    with pytest.raises(ConfigError):
        config_class_for({"model_type": "toy"})


def test_round_trip_and_model_spec():
    for cfg in (TINY_A, TINY_B):
        c = LlamaConfig.from_dict(cfg)
        assert LlamaConfig.from_dict(c.to_dict()) == c
        spec = c.model_spec()
        assert len(spec.layers) == c.num_hidden_layers and [e.layer for e in spec.plan] == list(range(c.num_hidden_layers))
        m = spec.layers[0].mixer
        assert m.kind == "attention" and m.params["num_kv_heads"] == c.num_key_value_heads
        assert m.params["position"].params["theta"] == c.rope_theta
        assert spec.layers[0].part("mixer_norm").params["eps"] == c.rms_norm_eps
        assert spec.stop_token_ids == c.eos_token_ids


def test_no_size_stands_in_code():
    """A model spec is a function of config.json alone: two configs, every size different."""
    a, b = LlamaConfig.from_dict(TINY_A).model_spec(), LlamaConfig.from_dict(TINY_B).model_spec()
    pa, pb = a.layers[0].mixer.params, b.layers[0].mixer.params
    for key in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"):
        assert pa[key] != pb[key]
    assert a.layers[0].feed_forward.params["intermediate_size"] != b.layers[0].feed_forward.params["intermediate_size"]
    assert a.vocab_size != b.vocab_size and a.head.params["tied"] != b.head.params["tied"]


def test_plan_validation():
    from hilbert_pruned_8b_b200.config.spec import PlanEntry
    import dataclasses
    spec = LlamaConfig.from_dict(TINY_A).model_spec()
    ok = dataclasses.replace(spec, plan=[PlanEntry(0), PlanEntry(1), PlanEntry(0), PlanEntry(1, cache_of=1)])
    ok.validate()
    for bad in ([PlanEntry(5)], [PlanEntry(0, cache_of=0)], [PlanEntry(0), PlanEntry(1, cache_of=2)],
                [PlanEntry(0), PlanEntry(1, cache_of=0), PlanEntry(0, cache_of=1)], []):
        with pytest.raises(ValueError):
            dataclasses.replace(spec, plan=bad).validate()
