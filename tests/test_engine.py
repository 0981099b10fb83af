"""The engine against the plain implementation, in 32-bit and in bfloat16: whole requests,
the last 32 tokens one by one, batches of unequal lengths with slot reuse, long decoding
and the first tokens of a sequence."""
import pytest
import torch

import trace_tools as tt
from conftest import TINY_A, TINY_B, TINY_C, TINY_D, require_gpu
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
MODELS = ["strong_a", "strong_b", "strong_c", "strong_d", "paper_a", "paper_b"]
STRONG = ["strong_a", "strong_b", "strong_c", "strong_d"]
VOCAB = {"a": TINY_A["vocab_size"], "b": TINY_B["vocab_size"], "c": TINY_C["vocab_size"], "d": TINY_D["vocab_size"]}


def _plain(folder, dtype):
    return PlainLlama(folder, round_to=torch.bfloat16 if dtype == "bfloat16" else None)


def _engine(folder, dtype, max_tokens, **kw):
    from hilbert_pruned_8b_b200.engine.step import Engine
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, **kw)


def _requests(model, lengths, seed):
    v = VOCAB[model[-1]]
    return {f"r{i}": tt.random_tokens(n, v, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("model", MODELS)
def test_whole_requests(model_folders, model, dtype):
    require_gpu()
    reqs = _requests(model, [1, 7, 40, 70], seed=100)
    steps, peak = tt.trace_whole(reqs)
    eng = _engine(model_folders[model], dtype, peak)
    got = tt.run_in_process(eng, steps)
    tt.compare(got, tt.plain_logits(_plain(model_folders[model], dtype), reqs), dtype, "whole")
    assert min(eng.cache.pages_free()) == eng.cache.num_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("model", STRONG)
def test_last_tokens_one_by_one(model_folders, model, dtype):
    require_gpu()
    reqs = _requests(model, [33, 70, 100], seed=200)
    steps, peak = tt.trace_tail(reqs, tail=32)
    eng = _engine(model_folders[model], dtype, peak)
    got = tt.run_in_process(eng, steps)
    tt.compare(got, tt.plain_logits(_plain(model_folders[model], dtype), reqs), dtype, "tail")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("model", STRONG)
def test_unequal_batches_with_slot_reuse(model_folders, model, dtype):
    require_gpu()
    v = VOCAB[model[-1]]
    # (total tokens, prompt length): shorter requests end earlier; three batches in a row
    shapes = [[(9, 1), (15, 7), (24, 16)], [(21, 5), (28, 12), (49, 33), (80, 64)], [(70, 66), (3, 3), (66, 2)]]
    batches, reqs = [], {}
    for b, group in enumerate(shapes):
        batch = {}
        for i, (n, p) in enumerate(group):
            rid = f"b{b}r{i}"
            reqs[rid] = tt.random_tokens(n, v, 300 + 10 * b + i)
            batch[rid] = (reqs[rid], p)
        batches.append(batch)
    steps, peak = tt.trace_batches(batches)
    eng = _engine(model_folders[model], dtype, peak)
    got = tt.run_in_process(eng, steps)
    tt.compare(got, tt.plain_logits(_plain(model_folders[model], dtype), reqs), dtype, "batches")
    assert min(eng.cache.pages_free()) == eng.cache.num_pages and eng.cache.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("model", ["strong_b", "strong_c"])
def test_long_decoding_across_pages(model_folders, model, dtype):
    require_gpu()
    reqs = _requests(model, [200], seed=400)
    steps, peak = tt.trace_tail(reqs, tail=190)
    eng = _engine(model_folders[model], dtype, peak)
    got = tt.run_in_process(eng, steps)
    tt.compare(got, tt.plain_logits(_plain(model_folders[model], dtype), reqs), dtype, "long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("model", STRONG)
def test_first_tokens(model_folders, model, dtype):
    require_gpu()
    reqs = _requests(model, [4, 2], seed=500)
    steps, peak = tt.trace_tail(reqs, tail=3)     # one token, then one by one
    eng = _engine(model_folders[model], dtype, peak)
    got = tt.run_in_process(eng, steps)
    tt.compare(got, tt.plain_logits(_plain(model_folders[model], dtype), reqs), dtype, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_step_cut_into_chunks(model_folders, dtype):
    """A step larger than the step capacity is cut; the logits are those of the uncut step."""
    require_gpu()
    model = "strong_a"
    reqs = _requests(model, [50, 21, 90], seed=600)
    batch = {rid: (t, len(t)) for rid, t in reqs.items()}
    steps, peak = tt.trace_batches([batch])
    eng = _engine(model_folders[model], dtype, peak, max_step_tokens=32)
    got = tt.run_in_process(eng, steps)
    tt.compare(got, tt.plain_logits(_plain(model_folders[model], dtype), reqs), dtype, "chunked")


@pytest.mark.parametrize("model", ["strong_c", "strong_d"])
@pytest.mark.parametrize("fuse,inside", [(False, False), (False, True), (True, True)])
def test_other_arrangements_of_decode_attention_in_the_engine(model_folders, model, fuse, inside):
    """Decode attention behind a rotation kernel instead of rotating and appending itself, and
    with the last split combining instead of a combination kernel: the same logits."""
    require_gpu()
    reqs = _requests(model, [70, 33, 130], seed=650)
    steps, peak = tt.trace_batches([{rid: (t, 5 + 20 * i) for i, (rid, t) in enumerate(reqs.items())}])
    eng = _engine(model_folders[model], "bfloat16", peak)
    eng.ctx.ops.fuse_decode_attention = fuse
    eng.ctx.ops.combine_in_attention = inside
    got = tt.run_in_process(eng, steps)
    tt.compare(got, tt.plain_logits(_plain(model_folders[model], "bfloat16"), reqs), "bfloat16", f"decode attention fuse={fuse} inside={inside}")


@pytest.mark.parametrize("model", ["strong_b", "strong_d"])
def test_norms_folded_into_the_products_of_few_token_steps(model_folders, model):
    """Steps of up to 32 tokens fold every norm between two products into them (the product that
    adds to the residual prepares the next norm's input, the product that reads it applies the
    per-token factor): only the first layer's first norm and the final norm run as kernels.  The
    logits are the plain model's either way, in steps of few tokens, in prompts, and when the two
    alternate (a prompt of 70 tokens, then single tokens; three sequences of unequal lengths)."""
    require_gpu()
    reqs = _requests(model, [70, 12, 130], seed=660)
    steps, peak = tt.trace_batches([{rid: (t, 3 + 9 * i) for i, (rid, t) in enumerate(reqs.items())}])
    want = tt.plain_logits(_plain(model_folders[model], "bfloat16"), reqs)
    layers = {"strong_b": TINY_B, "strong_d": TINY_D}[model]["num_hidden_layers"]
    for fold in (True, False):
        eng = _engine(model_folders[model], "bfloat16", peak)
        ops = eng.ctx.ops
        ops.fold_norms = fold
        ops.call_log = []
        got = tt.run_in_process(eng, steps)
        log, ops.call_log = ops.call_log, None
        tt.compare(got, want, "bfloat16", f"norms folded={fold}")
        assert ("hb_gemm_tc_fold" in log) == fold
        if fold:
            # The prompts' step runs every norm; a decode step (up to three tokens) the first layer's first
            # one and the final one.  (Replayed graphs do not pass through the log: it holds the prompts'
            # step and the decode steps that were captured, one per batch size and page-table width.)
            decode_steps = sum(1 for s in steps if all(len(e["tokens"]) == 1 for e in s["entries"]))
            assert decode_steps > 20
            logged_decode = log.count("hb_gemm_tc_fold") // (2 * (2 * layers - 1))
            assert logged_decode >= 1 and log.count("hb_gemm_tc_fold") == logged_decode * 2 * (2 * layers - 1)
            assert log.count("hb_rmsnorm") == (2 * layers + 1) * (len(steps) - decode_steps) + 2 * logged_decode


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("model", ["strong_c", "strong_d"])
def test_hundreds_of_keys_through_the_tensor_core_attention(model_folders, model, dtype):
    """A 600-token prompt, then 40 tokens one by one, next to a short request: ten pages of keys
    per sequence, prefill blocks that start inside pages, decode splits over many pages."""
    require_gpu()
    reqs = _requests(model, [640, 90], seed=660)
    steps, peak = tt.trace_batches([{"r0": (reqs["r0"], 600), "r1": (reqs["r1"], 50)}])
    eng = _engine(model_folders[model], dtype, peak, max_step_tokens=1024)
    got = tt.run_in_process(eng, steps)
    tt.compare(got, tt.plain_logits(_plain(model_folders[model], dtype), reqs), dtype, "hundreds of keys")
