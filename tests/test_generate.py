"""Generation through the entry points (Python API and command line) against the plain
implementation: greedy tokens, stop tokens, batches of unequal prompts, seeded temperature
sampling that does not depend on the batch."""
import json
import os
import subprocess
import sys

import pytest
import torch

import trace_tools as tt
from conftest import TINY_A, TINY_B, TINY_C, require_gpu
from plain_llama import PlainLlama, generate_greedy, inverse_cdf, temperature_probs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _prompts(vocab, lengths, seed):
    return [tt.random_tokens(n, vocab, seed + i) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("model,cfg", [("strong_a", TINY_A), ("strong_b", TINY_B), ("strong_c", TINY_C)])
def test_greedy_generation_float32_equals_plain(model_folders, model, cfg):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    prompts = _prompts(cfg["vocab_size"], [1, 7, 16, 30, 3], 800)
    llm = hb.load(model_folders[model], dtype="float32", max_tokens=64 * 8, max_batch=3)   # two batches: slots reused
    res = llm.generate(prompts, max_new_tokens=12, stop_token_ids=[])
    plain = PlainLlama(model_folders[model])
    for r, p in zip(res, prompts):
        assert r.tokens == generate_greedy(plain, p, 12), f"prompt of {len(p)} tokens"
        assert r.finish_reason == "length" and r.prompt_tokens == len(p)
    assert llm.generator.stats.batches == 2
    assert min(llm.engine.cache.pages_free()) == llm.engine.cache.num_pages


def test_stop_tokens_end_sequences_early(model_folders):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    prompts = _prompts(TINY_B["vocab_size"], [5, 12, 33], 820)
    plain = PlainLlama(model_folders["strong_b"])
    free = [generate_greedy(plain, p, 10) for p in prompts]
    stop = [free[0][3], free[1][0]]                  # ends request 0 after 4 tokens (or earlier), request 1 at once
    llm = hb.load(model_folders["strong_b"], dtype="float32", max_tokens=1024)
    res = llm.generate(prompts, max_new_tokens=10, stop_token_ids=stop)
    for r, p in zip(res, prompts):
        want = generate_greedy(plain, p, 10, stop=stop)
        assert r.tokens == want
        assert r.finish_reason == ("stop" if want[-1] in stop else "length")
    assert res[1].tokens == [free[1][0]]
    # the model's own eos ids (config.json) are the default
    eos = llm.engine.stop_token_ids
    assert eos == [3, 5]


def test_many_requests_with_stops_and_budgets_equal_plain(model_folders):
    """70 requests in batches of up to 32: sequences stop at different times (stop tokens, budgets
    from 0 to 14), so the decode batch shrinks step by step, replayed graphs of many batch sizes
    take turns, and the loop, which runs one step ahead of the tokens it has read, has to drop
    the sequences that stopped.  Every result is the plain model's."""
    require_gpu()
    import random
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.engine.generate import GenerationRequest
    from hilbert_pruned_8b_b200.sampling import SamplingParams
    rnd = random.Random(7)
    vocab = TINY_A["vocab_size"]
    plain = PlainLlama(model_folders["strong_a"])
    reqs, want = [], []
    for i in range(70):
        prompt = tt.random_tokens(rnd.randrange(1, 40), vocab, 2000 + i)
        budget = rnd.randrange(0, 15)
        free = generate_greedy(plain, prompt, budget) if budget else []
        stop = [free[rnd.randrange(len(free))]] if free and rnd.random() < 0.5 else []
        reqs.append(GenerationRequest(prompt, max_new_tokens=budget, sampling=SamplingParams(0.0, 0), stop_token_ids=stop))
        want.append(generate_greedy(plain, prompt, budget, stop=stop) if budget else [])
    llm = hb.load(model_folders["strong_a"], dtype="float32", max_tokens=64 * 40, max_batch=32)
    res = llm.generate_requests(reqs)
    assert [r.tokens for r in res] == want
    for r, q, w in zip(res, reqs, want):
        assert r.finish_reason == ("stop" if w and w[-1] in (q.stop_token_ids or []) else "length")
    assert llm.generator.stats.batches >= 3 and llm.engine.graph_replays > 0
    assert min(llm.engine.cache.pages_free()) == llm.engine.cache.num_pages


def test_bfloat16_greedy_follows_plain_rounded_model(model_folders):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    prompts = _prompts(TINY_C["vocab_size"], [9, 40, 70], 840)
    llm = hb.load(model_folders["strong_c"], dtype="bfloat16", max_tokens=1024)
    res = llm.generate(prompts, max_new_tokens=8, stop_token_ids=[])
    plain = PlainLlama(model_folders["strong_c"], round_to=torch.bfloat16)
    for r, p in zip(res, prompts):
        # every produced token must be (nearly) the best under the plain model given the same prefix
        toks = list(p)
        for t in r.tokens:
            lg = plain.logits(toks)[-1]
            assert lg[t] >= lg.max() - 0.02 * lg.abs().max(), "a token far from the plain model's best"
            toks.append(t)


def test_temperature_sampling_is_seeded_and_batch_independent(model_folders):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.engine.generate import GenerationRequest
    from hilbert_pruned_8b_b200.sampling import SamplingParams, uniform_from
    prompts = _prompts(TINY_B["vocab_size"], [5, 12, 33, 64], 860)
    llm = hb.load(model_folders["strong_b"], dtype="float32", max_tokens=2048)
    reqs = [GenerationRequest(p, 16, SamplingParams(0.8, seed=3), [], request_id=100 + i) for i, p in enumerate(prompts)]
    together = llm.generate_requests(reqs)
    alone = [llm.generate_requests([r])[0] for r in reqs]
    assert [r.tokens for r in together] == [r.tokens for r in alone]
    other = llm.generate_requests([GenerationRequest(prompts[0], 16, SamplingParams(0.8, seed=4), [], request_id=100)])
    assert other[0].tokens != together[0].tokens
    # each token is the inverse-CDF draw of the plain model's distribution with the same uniform
    plain = PlainLlama(model_folders["strong_b"])
    toks = list(prompts[1])
    for step, t in enumerate(together[1].tokens):
        p = temperature_probs(plain.logits(toks)[-1], 0.8)
        u = uniform_from(3, 101, step)
        c = torch.cumsum(p, 0)
        lo = float(c[t - 1]) if t > 0 else 0.0
        assert lo - 1e-5 <= u <= float(c[t]) + 1e-5
        assert t == inverse_cdf(p, u) or min(abs(u - lo), abs(u - float(c[t]))) < 1e-5
        toks.append(t)


def test_command_line_generate_and_logits(model_folders, tmp_path):
    require_gpu()
    folder = model_folders["strong_a"]
    prompts = _prompts(TINY_A["vocab_size"], [4, 11], 880)
    rows = tmp_path / "rows.jsonl"
    rows.write_text("".join(json.dumps({"id": f"x{i}", "tokens": p}) + "\n" for i, p in enumerate(prompts)))
    out = tmp_path / "out.jsonl"
    exe = [sys.executable, os.path.join(ROOT, "bin", "hilbert-b200")]
    cmd = exe + ["generate", "--model", folder, "--dtype", "float32", "--max-tokens", "256", "--input", str(rows),
                 "--output", str(out), "--max-new-tokens", "6", "--stop-ids", ""]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    got = [json.loads(line) for line in out.read_text().splitlines()]
    plain = PlainLlama(folder)
    assert [g["id"] for g in got] == ["x0", "x1"]
    assert [g["tokens"] for g in got] == [generate_greedy(plain, p, 6) for p in prompts]
    again = subprocess.run(cmd, capture_output=True, text=True)
    assert again.returncode != 0 and "Output must be new" in again.stderr
    res = subprocess.run(exe + ["logits", "--model", folder, "--dtype", "float32", "--tokens", " ".join(map(str, prompts[1])),
                                "--ids", "0 5 255", "--split", "4"], check=True, capture_output=True, text=True)
    vals = torch.tensor([float(x) for x in res.stdout.split()], dtype=torch.float64)
    ref = plain.logits(prompts[1])[-1][[0, 5, 255]]
    assert ((vals - ref).abs() / ref.abs().clamp(min=1)).max() < 1e-4
    bad = subprocess.run(exe + ["logits", "--model", folder, "--tokens", "1 999"], capture_output=True, text=True)
    assert bad.returncode == 1 and "token 999 out of range" in bad.stderr
