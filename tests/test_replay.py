"""bin/trace_run as a program: the same requests whole, with the last 32 tokens one by one,
and in batches of unequal lengths, in 32-bit and in bfloat16, against the plain implementation."""
import pytest
import torch

import trace_tools as tt
from conftest import TINY_A, TINY_B, TINY_C, require_gpu
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu
VOCAB = {"a": TINY_A["vocab_size"], "b": TINY_B["vocab_size"], "c": TINY_C["vocab_size"]}


def _requests(model, lengths, seed):
    return {f"r{i}": tt.random_tokens(n, VOCAB[model[-1]], seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("model", ["strong_a", "strong_b", "strong_c"])
def test_trace_run_every_way_of_cutting(model_folders, tmp_path, model, dtype):
    require_gpu()
    folder = model_folders[model]
    reqs = _requests(model, [40, 75, 33, 9], seed=700)
    plain = PlainLlama(folder, round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    ref = tt.plain_logits(plain, reqs)
    vocab = VOCAB[model[-1]]

    steps, peak = tt.trace_whole(reqs)
    got = tt.run_program(folder, dtype, steps, peak, str(tmp_path / "whole"), vocab)
    assert len(got) == sum(len(t) for t in reqs.values())
    tt.compare(got, ref, dtype, "trace_run whole")

    steps, peak = tt.trace_tail(reqs, tail=32)
    got = tt.run_program(folder, dtype, steps, peak, str(tmp_path / "tail"), vocab)
    tt.compare(got, ref, dtype, "trace_run tail")

    ids = list(reqs)
    batches = [{ids[0]: (reqs[ids[0]], 8), ids[1]: (reqs[ids[1]], 64), ids[3]: (reqs[ids[3]], 1)},
               {ids[2]: (reqs[ids[2]], 33), ids[0] + "x": (reqs[ids[0]], 17)}]
    ref2 = dict(ref)
    for p in range(len(reqs[ids[0]])):
        ref2[(ids[0] + "x", p)] = ref[(ids[0], p)]
    steps, peak = tt.trace_batches(batches)
    got = tt.run_program(folder, dtype, steps, peak, str(tmp_path / "batches"), vocab)
    tt.compare(got, ref2, dtype, "trace_run batches")


def test_trace_run_writes_nothing_for_steps_that_want_nothing(model_folders, tmp_path):
    require_gpu()
    import os
    toks = tt.random_tokens(20, VOCAB["a"], 1)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:10], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[10:], "want": [9]}], "end": ["q"]}]
    got = tt.run_program(model_folders["strong_a"], "float32", steps, 64, str(tmp_path / "o"), VOCAB["a"])
    assert sorted(os.listdir(tmp_path / "o")) == ["1.f32"] and list(got) == [("q", 19)]
    ref = PlainLlama(model_folders["strong_a"]).logits(toks)[19]
    tt.compare(got, {("q", 19): ref}, "float32", "split prefill")
