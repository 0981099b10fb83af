"""One layer at the layer sizes of real checkpoints of the architecture (8B, 3B and 1B
shapes; the vocabulary is cut down so that the folder stays small), in 32-bit and in
bfloat16: a batch of unequal prompts in one step, then 32 tokens one by one, against
the plain implementation.  The many-token prompt step takes the CTA-pair GEMM and the
tensor-core prefill attention, the decode steps the few-token GEMM schedules and the
split-K attention, at the widths that serving uses."""
import pytest
import torch

import trace_tools as tt
from conftest import require_gpu
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

LLAMA3 = dict(rope_type="llama3", low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
SHAPES = {
    "8b": dict(hidden_size=4096, intermediate_size=14336, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               vocab_size=4099, tie_word_embeddings=False, rope_scaling=dict(LLAMA3, factor=8.0)),
    "3b": dict(hidden_size=3072, intermediate_size=8192, num_attention_heads=24, num_key_value_heads=8, head_dim=128,
               vocab_size=3001, tie_word_embeddings=True, rope_scaling=dict(LLAMA3, factor=32.0)),
    "1b": dict(hidden_size=2048, intermediate_size=8192, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
               vocab_size=2050, tie_word_embeddings=True, rope_scaling=dict(LLAMA3, factor=32.0)),
}


@pytest.fixture(scope="module")
def size_folders(tmp_path_factory):
    import hilbert_pruned_8b_b200 as hb
    out = {}
    for i, (name, sizes) in enumerate(SHAPES.items()):
        cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", num_hidden_layers=1,
                   rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192, **sizes)
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        hb.weights.write_random_model(d, hb.LlamaConfig.from_dict(cfg), seed=40 + i, std=0.02, norm_std=0.05,
                                      fan_in_scale=1.0)
        out[name] = d
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", list(SHAPES))
def test_one_layer_at_real_sizes(size_folders, shape, dtype):
    require_gpu()
    from hilbert_pruned_8b_b200.engine.step import Engine
    vocab = SHAPES[shape]["vocab_size"]
    lengths = [862, 102, 35]        # the prompts of one step: 999 tokens, the CTA-pair product
    toks = {f"r{i}": tt.random_tokens(n, vocab, 900 + i) for i, n in enumerate(lengths)}
    steps, peak = tt.trace_batches([{rid: (t, len(t) - 32) for rid, t in toks.items()}])
    eng = Engine.from_folder(size_folders[shape], dtype, max_tokens=peak)
    got = tt.run_in_process(eng, steps)
    plain = PlainLlama(size_folders[shape], round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    tt.compare(got, tt.plain_logits(plain, toks), dtype, f"{shape} sizes")
    assert min(eng.cache.pages_free()) == eng.cache.num_pages
