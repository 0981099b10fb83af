"""Weight loading by name, its one error, dtype rules, and the random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

import hilbert_pruned_8b_b200 as hb
from conftest import TINY_A, TINY_B
from hilbert_pruned_8b_b200.engine.model import weight_table
from hilbert_pruned_8b_b200.weights import (SafetensorsError, SafetensorsFolder, WeightError, choose_prefix,
                                            load_tensors, random_tensors, write_random_model, write_safetensors)

CPU = torch.device("cpu")


def _table(cfg):
    return weight_table(hb.LlamaConfig.from_dict(cfg).model_spec())


def test_table_names_and_shapes_follow_the_reference():
    t = _table(TINY_B)
    assert t["model.embed_tokens.weight"].shape == (384, 160)
    assert t["model.layers.2.self_attn.q_proj.weight"].shape == (5 * 32, 160)
    assert t["model.layers.0.self_attn.k_proj.weight"].shape == (1 * 32, 160)
    assert t["model.layers.0.self_attn.o_proj.weight"].shape == (160, 5 * 32)
    assert t["model.layers.1.mlp.gate_proj.weight"].shape == (416, 160)
    assert t["model.layers.1.mlp.down_proj.weight"].shape == (160, 416)
    assert t["model.layers.1.post_attention_layernorm.weight"].shape == (160,)
    assert t["model.norm.weight"].kind == "vector" and t["lm_head.weight"].shape == (384, 160)
    assert not t["lm_head.weight"].optional
    assert _table(TINY_A)["lm_head.weight"].optional          # tied: a stored copy is not read
    assert len(t) == 1 + 3 * 9 + 2


def test_table_equals_the_shape_table_the_reference_prints():
    """The reference's own ``shapes`` command (cleanroom-transformer/src/shapes.c:12-40,
    src/main.c:528-536), run once on the two golden configurations and stored under
    tests/golden/: every per-layer matrix of its list is in the weight table under the same name
    with the same rows and columns, in every layer, and the table has no other layer matrices;
    the head sizes it derives are the model specification's."""
    import json
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "golden"))
    from golden_models import GOLDEN_MODELS
    with open(os.path.join(here, "golden", "reference_shapes.json")) as f:
        ref = json.load(f)["models"]
    for name, spec in GOLDEN_MODELS.items():
        cfg = hb.LlamaConfig.from_dict(spec["config"])
        ms = cfg.model_spec()
        table = weight_table(ms)
        r = ref[name]
        assert r["arch"] == "llama" and r["hidden"] == ms.hidden_size and len(r["layers"]) == 1
        layer = r["layers"][0]
        assert layer["type"] == "full" and layer["count"] == len(ms.layers) == spec["config"]["num_hidden_layers"]
        mixer = ms.layers[0].mixer.params
        assert (r["n_heads"], r["n_kv_heads"], r["head_dim"]) == (mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"])
        assert r["rot_dim"] == mixer["position"].params["rotary_dim"]
        matrices = {w["name"]: (w["rows"], w["cols"]) for w in layer["weights"]}
        for i in range(layer["count"]):
            prefix = f"model.layers.{i}."
            ours = {k[len(prefix):]: tuple(v.shape) for k, v in table.items() if k.startswith(prefix) and len(v.shape) == 2}
            assert ours == matrices, (name, i)
        act = layer["activations"]
        assert act["q_gate"][1] == matrices["self_attn.q_proj.weight"][0] and act["mlp_act"][1] == matrices["mlp.down_proj.weight"][1]


def test_random_model_folder_loads_and_is_seeded(tmp_path):
    cfg = hb.LlamaConfig.from_dict(TINY_A)
    d1 = write_random_model(str(tmp_path / "m1"), cfg, seed=5)
    d2 = write_random_model(str(tmp_path / "m2"), cfg, seed=5)
    d3 = write_random_model(str(tmp_path / "m3"), cfg, seed=6)
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    assert hb.load_config(d1) == cfg
    t1 = load_tensors(d1, _table(TINY_A), torch.bfloat16, CPU)
    t2 = load_tensors(d2, _table(TINY_A), torch.bfloat16, CPU)
    t3 = load_tensors(d3, _table(TINY_A), torch.bfloat16, CPU)
    name = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(t1[name], t2[name]) and not torch.equal(t1[name], t3[name])
    assert t1[name].dtype == torch.bfloat16 and abs(t1[name].float().std().item() - 0.02) < 0.002
    assert torch.all(t1["model.norm.weight"] == 1)
    assert "lm_head.weight" not in t1


def test_random_weights_are_a_function_of_seed_name_and_element():
    """A tensor's values do not depend on which other tensors are drawn, in which order, or on
    how the work is cut; the draw is a standard normal (mean, deviation, tails, Kolmogorov
    distance); the tail's own logarithm agrees with the library's."""
    import numpy as np
    from hilbert_pruned_8b_b200.weights import random_init as ri
    table = _table(TINY_B)
    all_of_it = random_tensors(table, 7, CPU, std=0.02, norm_std=0.01)
    name = "model.layers.1.mlp.down_proj.weight"
    alone = random_tensors({name: table[name]}, 7, CPU, std=0.02, norm_std=0.01)
    assert torch.equal(all_of_it[name], alone[name])
    other_prefix = random_tensors({"x." + name: table[name]}, 7, CPU)
    assert not torch.equal(other_prefix["x." + name], alone[name])
    base = ri.stream_base(7, name)
    whole = ri.standard_normals(base, 0, 100000)
    assert np.array_equal(whole[777:999], ri.standard_normals(base, 777, 222))          # element i is element i
    big = ri.normal_tensor_cpu((5000, 1000), 7, name, 1.0, 0.0, torch.float32).numpy().ravel()   # threaded chunks
    assert np.array_equal(big[:100000], whole)
    assert abs(big.mean()) < 2e-3 and abs(big.std() - 1.0) < 2e-3
    for z, want in ((1.0, 0.158655), (2.0, 0.0227501), (3.0, 0.00134990), (4.0, 3.16712e-5)):
        tol = 4.0 / (want * big.size) ** 0.5                  # four standard deviations of the count
        assert abs((big > z).mean() / want - 1) < tol and abs((big < -z).mean() / want - 1) < tol
    srt = np.sort(big[:200000].astype(np.float64))
    cdf = 0.5 * (1.0 + np.vectorize(__import__("math").erf)(srt / np.sqrt(2.0)))
    assert np.abs(cdf - (np.arange(1, srt.size + 1) - 0.5) / srt.size).max() < 0.004
    p = np.float32(2.0) ** -np.arange(1, 34, dtype=np.float32) * np.float32(1.37)
    assert np.abs(ri._log32(p) / np.log(p.astype(np.float64)) - 1).max() < 3e-7
    norm = random_tensors({"n": table["model.norm.weight"]}, 7, CPU, norm_std=0.01, dtype=torch.float32)["n"]
    assert abs(norm.mean().item() - 1.0) < 0.005 and 0.005 < norm.std().item() < 0.02


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = hb.LlamaConfig.from_dict(TINY_B)
    table = _table(TINY_B)
    tensors = random_tensors(table, 1, CPU)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(160, 161, dtype=torch.bfloat16)
    tensors["model.layers.2.input_layernorm.weight"] = torch.zeros(159, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(160, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)        # ignorable
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as ei:
        load_tensors(str(tmp_path), table, torch.bfloat16, CPU)
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert sorted(w[0] for w in e.wrong_shape) == ["model.layers.0.self_attn.q_proj.weight",
                                                   "model.layers.2.input_layernorm.weight"]
    text = str(e)
    assert "missing (2)" in text and "unexpected (1)" in text
    assert "model.layers.0.self_attn.q_proj.weight has shape [160, 161], expected [160, 160]" in text


def test_extra_tensors_are_ignored_unless_strict(tmp_path):
    """A tensor no part asks for is not a fault (the reference never looks at what it does not
    bind, cleanroom-transformer/src/model.c:391-447); strict loading refuses it by name."""
    cfg = hb.LlamaConfig.from_dict(TINY_A)
    table = _table(TINY_A)
    tensors = random_tensors(table, 1, CPU)
    tensors["mtp.layers.0.extra.weight"] = torch.zeros(3, 3, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    got = load_tensors(str(tmp_path), table, torch.bfloat16, CPU)
    assert "mtp.layers.0.extra.weight" not in got and len(got) == len(table) - 1      # the tied head is optional
    with pytest.raises(WeightError) as ei:
        load_tensors(str(tmp_path), table, torch.bfloat16, CPU, strict=True)
    assert ei.value.unexpected == ["mtp.layers.0.extra.weight"] and not ei.value.missing


def test_dtype_rules(tmp_path):
    cfg = hb.LlamaConfig.from_dict(TINY_A)
    table = _table(TINY_A)
    tensors = random_tensors(table, 1, CPU)
    exact = tensors["model.layers.0.mlp.down_proj.weight"].clone()
    tensors["model.layers.0.mlp.gate_proj.weight"] = tensors["model.layers.0.mlp.gate_proj.weight"].to(torch.float32) * 1.001
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].to(torch.float16)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].to(torch.float32).reshape(1, 64)   # extra unit dim
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    bf = load_tensors(str(tmp_path), table, torch.bfloat16, CPU)
    assert bf["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert bf["model.layers.0.mlp.gate_proj.weight"].dtype == torch.float32      # stored in 32-bit: stays so
    assert bf["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16       # float16 is converted
    assert bf["model.norm.weight"].shape == (64,)
    f32 = load_tensors(str(tmp_path), table, torch.float32, CPU)
    assert all(t.dtype == torch.float32 for t in f32.values())
    assert torch.equal(f32["model.layers.0.mlp.down_proj.weight"], exact.float())  # widened exactly


def test_container_errors(tmp_path):
    (tmp_path / "model.safetensors").write_bytes(b"\x05\x00")
    with pytest.raises(SafetensorsError, match="bad header length"):
        SafetensorsFolder(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="bad header length"):
        SafetensorsFolder(str(tmp_path))
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 64]}}).encode()
    (tmp_path / "model.safetensors").write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="bad offsets for x"):
        SafetensorsFolder(str(tmp_path))
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFolder(str(tmp_path / "nowhere"))


def test_sharded_folder_and_prefix_choice(tmp_path):
    cfg = hb.LlamaConfig.from_dict(TINY_A)
    spec = cfg.model_spec()
    table = weight_table(spec, prefix="model.language_model.")
    tensors = random_tensors(table, 3, CPU)
    names = list(tensors)
    half = len(names) // 2
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: tensors[n] for n in names[half:]})
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    f = SafetensorsFolder(str(tmp_path))
    assert choose_prefix(f.names(), spec.weight_prefixes, "embed_tokens.weight") == "model.language_model."
    f.close()
    got = load_tensors(str(tmp_path), table, torch.bfloat16, CPU)
    assert all(torch.equal(got[n], tensors[n]) for n in names)
    assert choose_prefix(["model.embed_tokens.weight"], spec.weight_prefixes, "embed_tokens.weight") == "model."
