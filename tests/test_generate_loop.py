"""The generation loop's decisions with a fake engine and sampler (no GPU): batching,
admission, stop tokens, budgets, early endings, slot reuse."""
import pytest
import torch

from hilbert_pruned_8b_b200.cache import CacheManager
from hilbert_pruned_8b_b200.engine.generate import (GenerationRequest, Generator, finish_reason, plan_batch)
from hilbert_pruned_8b_b200.parts.base import CacheNeed
from hilbert_pruned_8b_b200.sampling import SamplingParams, option_scores, uniform_from

VOCAB = 50


class FakeEngine:
    """Next token = (sum of the sequence's tokens so far) % VOCAB; keeps the real cache bookkeeping."""

    def __init__(self, max_tokens=1024):
        self.cache = CacheManager({0: CacheNeed(1, 16)}, {}, max_tokens, torch.device("cpu"), torch.float32,
                                  allocate=False)
        self.stop_token_ids = [0]
        self.sums = {}
        self.steps = []          # (kind, [sequence ids]) per step
        self.peak_pages = 0

    def open_sequence(self):
        s = self.cache.open()
        self.sums[s.seq_id] = 0
        return s

    def close_sequence(self, seq):
        self.cache.close(seq)

    def step(self, entries):
        self.cache.reserve([(e.seq, e.seq.length + len(e.tokens)) for e in entries])
        rows = []
        for e in entries:
            self.sums[e.seq.seq_id] += sum(e.tokens)
            self.cache.commit(e.seq, e.seq.length + len(e.tokens))
            for _ in e.want:
                row = torch.zeros(VOCAB)
                row[self.sums[e.seq.seq_id] % VOCAB] = 1.0
                rows.append(row)
        self.steps.append(("prefill" if any(len(e.tokens) > 1 or e.seq.length == len(e.tokens) for e in entries)
                           else "decode", [e.seq.seq_id for e in entries]))
        self.peak_pages = max(self.peak_pages, self.cache.num_pages - min(self.cache.pages_free()))
        return torch.stack(rows)


class AheadEngine(FakeEngine):
    """The fake engine with the interface of a step that takes its tokens from a tensor the
    host has not read (the generation loop then runs one step ahead)."""
    takes_device_tokens = True

    def __init__(self, max_tokens=1024):
        super().__init__(max_tokens)
        self.ahead_steps = 0

    def step(self, entries, device_tokens=None):
        if device_tokens is not None:
            assert all(list(e.tokens) == [0] for e in entries) and device_tokens.numel() == len(entries)
            from hilbert_pruned_8b_b200.engine.batch import StepEntry
            entries = [StepEntry(e.seq, [int(t)], e.want) for e, t in zip(entries, device_tokens.tolist())]
            self.ahead_steps += 1
        return super().step(entries)


class FakeSampler:
    def __init__(self):
        self.calls = []

    def sample(self, logits, temperatures, seeds, request_ids, steps):
        self.calls.append((list(temperatures), list(seeds), list(request_ids), list(steps)))
        return logits.argmax(dim=-1)


def expected(prompt, n, stop):
    toks, out = list(prompt), []
    for _ in range(n):
        t = sum(toks) % VOCAB
        out.append(t)
        toks.append(t)
        if t in stop:
            return out, "stop"
    return out, "length"


def test_plan_batch():
    assert plan_batch([2, 2, 2, 2], pages_free=5, max_batch=8) == 2
    assert plan_batch([1, 1, 1, 1], pages_free=50, max_batch=3) == 3
    assert plan_batch([], 5, 3) == 0
    with pytest.raises(ValueError, match="needs 9 cache pages"):
        plan_batch([9, 1], pages_free=5, max_batch=8)


def test_finish_reason():
    assert finish_reason(7, 1, 5, 10, 100, [7]) == "stop"
    assert finish_reason(8, 5, 5, 10, 100, [7]) == "length"
    assert finish_reason(8, 2, 5, 100, 100, [7]) == "context"
    assert finish_reason(8, 2, 5, 99, 100, [7]) is None
    assert finish_reason(7, 5, 5, 100, 100, [7]) == "stop"       # a stop token wins


def test_unequal_prompts_stop_tokens_and_early_endings():
    eng, smp = FakeEngine(), FakeSampler()
    gen = Generator(eng, smp, max_batch=4)
    prompts = [[1, 2, 3], [10], [4, 4, 4, 4, 4, 4, 4], [49, 1], [5, 6]]
    reqs = [GenerationRequest(p, max_new_tokens=n, stop_token_ids=[0])
            for p, n in zip(prompts, [6, 3, 9, 4, 0])]
    res = gen.generate(reqs)
    assert [r.request_id for r in res] == [0, 1, 2, 3, 4]
    for r, q in zip(res, reqs):
        want, why = expected(q.prompt, q.max_new_tokens, [0])
        assert r.tokens == want and r.finish_reason == why and r.prompt_tokens == len(q.prompt)
    assert res[3].finish_reason == "stop" and res[3].tokens == [0]      # 49 + 1 = 50 -> token 0 at once
    assert res[4].tokens == [] and res[4].finish_reason == "length"
    # two batches (4 + 1, the last has no budget and runs no step): the first starts together
    assert eng.steps[0][0] == "prefill" and len(eng.steps[0][1]) == 4
    sizes = [len(ids) for kind, ids in eng.steps if kind == "decode"]
    assert sizes == sorted(sizes, reverse=True) and sizes[0] == 3 and sizes[-1] == 1   # sequences leave, none joins
    assert min(eng.cache.pages_free()) == eng.cache.num_pages and eng.cache.slots.num_held == 0
    # the sampler sees per-request seeds, ids and the step number
    assert smp.calls[0][2] == [0, 1, 2, 3] and smp.calls[0][3] == [0, 0, 0, 0] and smp.calls[1][3][0] == 1


def test_batches_follow_one_another_and_reuse_slots():
    eng, smp = FakeEngine(max_tokens=64 * 4), FakeSampler()
    gen = Generator(eng, smp, max_batch=8)
    reqs = [GenerationRequest([i + 1] * 40, max_new_tokens=30, stop_token_ids=[]) for i in range(7)]
    res = gen.generate(reqs)                    # each needs 2 pages: two fit at a time
    assert len(res) == 7 and all(len(r.tokens) == 30 for r in res)
    assert gen.stats.batches == 4 and eng.peak_pages <= 4
    prefills = [ids for kind, ids in eng.steps if kind == "prefill"]
    assert [len(p) for p in prefills] == [2, 2, 2, 1]
    assert eng.cache.slots.num_held == 0 and min(eng.cache.pages_free()) == 4


def test_context_limit_and_bad_requests():
    eng = FakeEngine(max_tokens=64)
    gen = Generator(eng, FakeSampler())
    res = gen.generate([GenerationRequest([3] * 60, max_new_tokens=50, stop_token_ids=[])])
    assert res[0].finish_reason == "context" and len(res[0].tokens) == 5   # 60 + 4 fed = 64, the 5th cannot be fed
    with pytest.raises(ValueError, match="empty prompt"):
        gen.generate([GenerationRequest([])])
    with pytest.raises(ValueError, match="prompt tokens"):
        gen.generate([GenerationRequest([1] * 65)])
    assert eng.cache.slots.num_held == 0


def test_a_request_ends_at_its_own_limit_while_the_pool_has_pages():
    """The context of a request is the engine's limit for ONE sequence (and the model's stated
    maximum position), not the size of the page pool: admission counts pages up to that limit."""
    eng = FakeEngine(max_tokens=64 * 16)
    eng.generation_limit = 100
    gen = Generator(eng, FakeSampler(), max_batch=8)
    reqs = [GenerationRequest([3] * 90, max_new_tokens=50, stop_token_ids=[]),
            GenerationRequest([4] * 10, max_new_tokens=20, stop_token_ids=[])]
    res = gen.generate(reqs)
    assert res[0].finish_reason == "context" and len(res[0].tokens) == 11     # 90 + 10 fed = 100, the 11th cannot be fed
    assert res[1].finish_reason == "length" and len(res[1].tokens) == 20
    assert eng.peak_pages <= 2 + 1 and min(eng.cache.pages_free()) == 16       # costs were counted up to the limit
    with pytest.raises(ValueError, match="prompt tokens, context is 100"):
        gen.generate([GenerationRequest([1] * 101)])
    ahead = AheadEngine(max_tokens=64 * 16)
    ahead.generation_limit = 100
    res2 = Generator(ahead, FakeSampler(), max_batch=8).generate(reqs)
    assert [(r.tokens, r.finish_reason) for r in res2] == [(r.tokens, r.finish_reason) for r in res]


class NotingEngine(AheadEngine):
    """An engine with device status words (here host memory): the loop copies them beside each
    step's tokens and stops the call when one is set."""

    def __init__(self, fail_at_step):
        super().__init__(256)
        self.words = torch.zeros(4, dtype=torch.int32)
        self.fail_at_step, self.decode_steps = fail_at_step, 0
        self.raised = None

    def status_tensor(self):
        return self.words

    def step(self, entries, device_tokens=None):
        out = super().step(entries, device_tokens)
        if all(len(e.tokens) == 1 for e in entries):
            self.decode_steps += 1
            if self.decode_steps == self.fail_at_step:
                self.words[1] = 3            # what a sampler notes for non-finite logits in row 2
        return out

    def raise_on_status(self, words):
        self.raised = list(words)
        self.words.zero_()
        raise RuntimeError(f"status {list(words)}")


def test_a_status_word_set_on_the_device_stops_generation(monkeypatch):
    """The loop reads the status words with the step's tokens; a non-zero word raises through
    the engine, the sequences are closed and every page comes back."""
    import hilbert_pruned_8b_b200.engine.generate as g

    eng = NotingEngine(fail_at_step=3)
    gen = Generator(eng, FakeSampler(), max_batch=4)
    # the fake sampler's tokens are host tensors: take the path of device tensors by hand
    calls = {"n": 0}
    real = Generator._launch_sampling

    def launch(self, logits, order, live, step_no, toks=None):
        rec = real(self, logits, order, live, step_no, toks)
        rec["status"] = eng.status_tensor().clone()
        calls["n"] += 1
        return rec

    monkeypatch.setattr(g.Generator, "_launch_sampling", launch)
    reqs = [GenerationRequest([3, 4, 5], max_new_tokens=30, stop_token_ids=[]),
            GenerationRequest([7], max_new_tokens=30, stop_token_ids=[])]
    with pytest.raises(RuntimeError, match="status"):
        gen.generate(reqs)
    assert eng.raised == [0, 3, 0, 0] and calls["n"] >= 3
    assert eng.cache.slots.num_held == 0 and min(eng.cache.pages_free()) == eng.cache.num_pages
    # the next call starts clean
    eng.fail_at_step = -1
    assert len(gen.generate(reqs)) == 2


def test_default_stop_ids_come_from_the_model():
    eng = FakeEngine()
    eng.stop_token_ids = [6]
    res = Generator(eng, FakeSampler()).generate([GenerationRequest([1, 2, 3], max_new_tokens=10)])
    assert res[0].tokens == [6] and res[0].finish_reason == "stop"


def test_sampling_helpers():
    assert 0.0 <= uniform_from(1, 2, 3) < 1.0
    assert uniform_from(1, 2, 3) == uniform_from(1, 2, 3) != uniform_from(1, 2, 4)
    us = [uniform_from(9, r, s) for r in range(40) for s in range(40)]
    assert 0.45 < sum(us) / len(us) < 0.55
    p = option_scores([1.0, 2.0, 3.0])
    assert abs(sum(p) - 1) < 1e-12 and p[2] > p[1] > p[0]
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_running_one_step_ahead_changes_no_result(seed):
    """With an engine that takes a step's tokens from the device the loop launches step k+1
    before it has read step k's tokens.  Results (tokens, finish reasons) are those of the
    plain loop, for stop tokens, budgets, the context's end and batch after batch; every page
    comes back."""
    import random
    rnd = random.Random(seed)
    reqs = []
    for i in range(rnd.randrange(3, 9)):
        prompt = [rnd.randrange(1, VOCAB) for _ in range(rnd.randrange(1, 40))]
        reqs.append(GenerationRequest(prompt, max_new_tokens=rnd.randrange(0, 30), sampling=SamplingParams(0.0, 0),
                                      stop_token_ids=rnd.sample(range(VOCAB), rnd.randrange(0, 6))))
    plain_engine, ahead_engine = FakeEngine(max_tokens=256), AheadEngine(max_tokens=256)
    plain = Generator(plain_engine, FakeSampler(), max_batch=4).generate(reqs)
    ahead = Generator(ahead_engine, FakeSampler(), max_batch=4).generate(reqs)
    assert [(r.request_id, r.tokens, r.finish_reason) for r in plain] == [(r.request_id, r.tokens, r.finish_reason) for r in ahead]
    for r, q in zip(ahead, reqs):
        want, why = expected(q.prompt, q.max_new_tokens, q.stop_token_ids)
        if r.finish_reason != "context":
            assert (r.tokens, r.finish_reason) == (want, why if want else "length")
    assert ahead_engine.ahead_steps > 0
    assert min(ahead_engine.cache.pages_free()) == ahead_engine.cache.num_pages


def test_running_ahead_stops_at_the_context_end_as_the_plain_loop_does():
    reqs = [GenerationRequest([3, 4, 5], max_new_tokens=500, sampling=SamplingParams(0.0, 0), stop_token_ids=[])]
    a = Generator(FakeEngine(max_tokens=64), FakeSampler(), max_batch=2).generate(reqs)
    b = Generator(AheadEngine(max_tokens=64), FakeSampler(), max_batch=2).generate(reqs)
    assert a[0].finish_reason == b[0].finish_reason == "context" and a[0].tokens == b[0].tokens
