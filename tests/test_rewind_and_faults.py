"""Rewinding a sequence on the GPU (the reference's snapshot / restore), each sequence's own
context limit, and the faults that must not pass silently: a status word a kernel set, logits
that are not finite, a page number outside the cache.  Every fault here is made on the HOST (a
word written into the status tensor, a NaN written into a weight, a wrong number written into a
page table that the kernels clamp by design); nothing makes a kernel wait, trap or touch memory
it does not own."""
import io
import json

import pytest
import torch

import trace_tools as tt
from conftest import TINY_A, TINY_B, TINY_C, require_gpu
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
VOCAB = {"a": TINY_A["vocab_size"], "b": TINY_B["vocab_size"], "c": TINY_C["vocab_size"]}


def _plain(folder, dtype):
    return PlainLlama(folder, round_to=torch.bfloat16 if dtype == "bfloat16" else None)


# ----------------------------------------------------------------------------------- rewind
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("model", ["strong_a", "strong_b", "strong_c"])
def test_rewind_then_another_suffix(model_folders, model, dtype):
    """full = prefix + snapshot + suffix + restore + another suffix (the reference's obligation,
    cleanroom-transformer/src/cuda_backend.cu:1429-1441, main.c:363-370), with what a paged cache
    adds: the pages the rewind gives back are taken by ANOTHER sequence before the rewound one
    grows again, single-token steps run through captured graphs and the ring of kept page-table
    rows on both sides of the rewind, and a second sequence shares every decode step."""
    require_gpu()
    from hilbert_pruned_8b_b200.engine.batch import StepEntry
    from hilbert_pruned_8b_b200.engine.step import Engine
    v = VOCAB[model[-1]]
    P = 37
    prefix = tt.random_tokens(P, v, 700)
    first = prefix + tt.random_tokens(70, v, 701)            # grows into a second and third page
    second = prefix + tt.random_tokens(55, v, 702)
    third = prefix + tt.random_tokens(6, v, 703)
    other = tt.random_tokens(140, v, 704)
    plain = _plain(model_folders[model], dtype)
    ref = {"first": plain.logits(first), "second": plain.logits(second), "third": plain.logits(third),
           "other": plain.logits(other)}
    eng = Engine.from_folder(model_folders[model], dtype, max_tokens=64 * 6)
    got = {}

    def feed(entries):
        """entries: (name, sequence, tokens, first position); logits at every fed position."""
        lg = eng.step_chunked([StepEntry(s, toks, list(range(len(toks)))) for _, s, toks, _ in entries])
        lg = lg.detach().cpu().double()
        row = 0
        for name, _, toks, pos0 in entries:
            for i in range(len(toks)):
                got[(name, pos0 + i)] = lg[row].clone()
                row += 1

    a, b = eng.open_sequence(), eng.open_sequence()
    feed([("first", a, prefix, 0), ("other", b, other[:20], 0)])
    snap = eng.snapshot(a)
    feed([("first", a, first[P:P + 60], P)])                                     # a holds 97 tokens: two pages
    for t in range(P + 60, len(first)):                                          # single tokens, b beside it
        feed([("first", a, [first[t]], t), ("other", b, [other[20 + t - P - 60]], 20 + t - P - 60)])
    assert a.length == len(first) and len(a.pages[0]) == 2
    pages_before = list(a.pages[0])
    eng.restore(a, snap)
    assert a.length == P and len(a.pages[0]) == 1 and min(eng.cache.pages_free()) == 6 - 2
    fed_b = 20 + len(first) - P - 60
    feed([("other", b, other[fed_b:fed_b + 70], fed_b)])                         # b takes the page a gave back
    fed_b += 70
    assert pages_before[1] in b.pages[0]
    # the second suffix: a chunk, then single tokens through the graphs captured before the rewind
    feed([("second", a, second[P:P + 40], P)])
    for t in range(P + 40, len(second)):
        feed([("second", a, [second[t]], t), ("other", b, [other[fed_b]], fed_b)])
        fed_b += 1
    assert a.pages[0][1] != pages_before[1]
    # rewind again, and single tokens at once
    eng.restore(a, snap)
    for t in range(P, len(third)):
        feed([("third", a, [third[t]], t), ("other", b, [other[fed_b]], fed_b)])
        fed_b += 1
    eng.close_sequence(a)
    eng.close_sequence(b)
    assert min(eng.cache.pages_free()) == eng.cache.num_pages and eng.cache.slots.num_held == 0
    want = {k: ref[k[0]][k[1]] for k in got}
    tt.compare(got, want, dtype, "rewind")
    assert {k[0] for k in got} == {"first", "second", "third", "other"} and eng.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logits_with_split_runs_the_rest_twice(model_folders, dtype):
    """``LLM.logits(split=N)`` is the reference's ``logits --split N``: prefix, snapshot, rest,
    restore, rest again; the answer is the unsplit one."""
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    llm = hb.load(model_folders["strong_b"], dtype=dtype, max_tokens=256)
    toks = tt.random_tokens(90, VOCAB["b"], 710)
    whole = llm.logits(toks).cpu().double()
    ref = _plain(model_folders["strong_b"], dtype).logits(toks)[-1]
    tt.compare({("w", 0): whole}, {("w", 0): ref}, dtype, "logits")
    for split in (1, 45, 64, 89):
        again = llm.logits(toks, split=split).cpu().double()
        tt.compare({("s", split): again}, {("s", split): ref}, dtype, f"logits --split {split}")
    ids = [5, 0, 383]
    assert torch.equal(llm.logits(toks, ids=ids, split=45).cpu(), llm.logits(toks, split=45).cpu()[ids])
    assert min(llm.engine.cache.pages_free()) == llm.engine.cache.num_pages


# ------------------------------------------------------------------- each sequence's own limit
def test_generation_stops_at_the_models_maximum_position(model_folders):
    """Tiny A states max_position_embeddings 128: a request ends with "context" there although the
    page pool holds far more; an explicit limit below it wins; the step function refuses tokens
    beyond the engine's limit, and given tokens (replay) may run past the model's stated maximum."""
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.engine.batch import StepEntry
    folder = model_folders["strong_a"]
    prompt = tt.random_tokens(100, VOCAB["a"], 720)
    llm = hb.load(folder, dtype="float32", max_tokens=1024)
    assert llm.engine.generation_limit == 128 and llm.engine.sequence_limit == 1024
    res = llm.generate([prompt, prompt[:5]], max_new_tokens=60, stop_token_ids=[])
    assert res[0].finish_reason == "context" and len(res[0].tokens) == 29        # 100 + 28 fed = 128
    assert res[1].finish_reason == "length" and len(res[1].tokens) == 60
    assert min(llm.engine.cache.pages_free()) == 16
    seq = llm.engine.open_sequence()
    llm.engine.step_chunked([StepEntry(seq, tt.random_tokens(200, VOCAB["a"], 721), [199])])   # replay may pass 128
    llm.engine.close_sequence(seq)
    tight = hb.load(folder, dtype="float32", max_tokens=1024, max_sequence_tokens=110)
    res = tight.generate([prompt], max_new_tokens=60, stop_token_ids=[])
    assert res[0].finish_reason == "context" and len(res[0].tokens) == 11
    seq = tight.engine.open_sequence()
    with pytest.raises(ValueError, match="exceed context 110"):
        tight.engine.step_chunked([StepEntry(seq, prompt + prompt[:11], [])])
    with pytest.raises(ValueError, match="exceed context 110"):                  # refused as a whole: nothing was fed
        tight.engine.step([StepEntry(seq, prompt + prompt[:11], [])])
    assert seq.length == 0
    tight.engine.close_sequence(seq)
    # a cut step is checked before its first part runs
    small = hb.load(folder, dtype="float32", max_tokens=1024, max_step_tokens=32)
    seq = small.engine.open_sequence()
    with pytest.raises(ValueError, match="token 256 out of range"):
        small.engine.step_chunked([StepEntry(seq, prompt + [256], [])])
    assert seq.length == 0 and min(small.engine.cache.pages_free()) == 16
    small.engine.close_sequence(seq)


# ------------------------------------------------------------------------------ loud failure
def test_a_status_word_stops_generate_and_is_cleared(model_folders):
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.kernels.ops import KernelError
    llm = hb.load(model_folders["strong_c"], dtype="bfloat16", max_tokens=512)
    prompts = [tt.random_tokens(n, VOCAB["c"], 730 + n) for n in (9, 30)]
    clean = [r.tokens for r in llm.generate(prompts, max_new_tokens=12, stop_token_ids=[])]
    llm.engine.status_tensor()[0] = 7                       # what a bounded wait that ran out leaves
    with pytest.raises(KernelError, match="bounded wait .code 7"):
        llm.generate(prompts, max_new_tokens=12, stop_token_ids=[])
    assert llm.engine.status_tensor().tolist() == [0, 0, 0, 0]
    assert min(llm.engine.cache.pages_free()) == llm.engine.cache.num_pages and llm.engine.cache.slots.num_held == 0
    assert [r.tokens for r in llm.generate(prompts, max_new_tokens=12, stop_token_ids=[])] == clean
    # set while decoding: the loop reads the words beside each step's tokens
    calls = {"n": 0}
    real_step = llm.engine.step

    def step(entries, **kw):
        calls["n"] += 1
        if calls["n"] == 5:
            llm.engine.status_tensor()[2] = 3
        return real_step(entries, **kw)

    llm.engine.step = step
    with pytest.raises(KernelError, match="page number outside the cache.*sequence 2"):
        llm.generate(prompts, max_new_tokens=12, stop_token_ids=[])
    llm.engine.step = real_step
    assert calls["n"] < 12 and llm.engine.cache.slots.num_held == 0


@pytest.mark.parametrize("temperature", [0.0, 0.7])
def test_non_finite_logits_stop_generation(model_folders, temperature):
    """A NaN in the final norm's weight makes every logit NaN: the sampler notes the row, the
    loop raises as the reference fails such a row (cleanroom-transformer/src/engine.c:29-31)."""
    require_gpu()
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.kernels.ops import KernelError
    llm = hb.load(model_folders["strong_b"], dtype="float32", max_tokens=512)
    prompts = [tt.random_tokens(n, VOCAB["b"], 740 + n) for n in (4, 17)]
    llm.generate(prompts, max_new_tokens=3, temperature=temperature, stop_token_ids=[])
    weight = llm.engine.model.final_norm.weight
    keep = weight[5].item()
    # the first step's logits are fine, later ones are not: the fault appears while decoding
    calls = {"n": 0}
    real_step = llm.engine.step

    def step(entries, **kw):
        calls["n"] += 1
        if calls["n"] == 4:
            weight[5] = float("nan")
        return real_step(entries, **kw)

    llm.engine.step = step
    with pytest.raises(KernelError, match="non-finite logits at row"):
        llm.generate(prompts, max_new_tokens=10, temperature=temperature, stop_token_ids=[])
    llm.engine.step = real_step
    with pytest.raises(KernelError, match="non-finite"):                          # and in the prompt step
        llm.generate(prompts, max_new_tokens=10, temperature=temperature, stop_token_ids=[])
    weight[5] = keep
    assert len(llm.generate(prompts, max_new_tokens=3, temperature=temperature, stop_token_ids=[])) == 2
    assert llm.engine.cache.slots.num_held == 0


def test_replay_and_command_line_end_with_one_line(model_folders, tmp_path, monkeypatch, capsys):
    require_gpu()
    from hilbert_pruned_8b_b200 import cli
    from hilbert_pruned_8b_b200.engine import replay
    from hilbert_pruned_8b_b200.engine.step import Engine
    folder = model_folders["strong_a"]
    real = Engine.from_folder.__func__

    def poisoned(cls, *a, **kw):
        eng = real(cls, *a, **kw)
        eng.status_tensor()[0] = 21
        return eng

    monkeypatch.setattr(Engine, "from_folder", classmethod(poisoned))
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": [1, 2, 3], "want": [2]}], "end": ["x"]}]
    monkeypatch.setattr("sys.stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    rc = replay.main(["--model", folder, "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"])
    err = capsys.readouterr().err.strip().splitlines()
    assert rc == 1 and len(err) == 1 and err[0].startswith("error: a tensor-core kernel gave up a bounded wait (code 21)")
    assert not (tmp_path / "o" / "0.f32").exists()
    rc = cli.run(["generate", "--model", folder, "--dtype", "float32", "--tokens", "1 2 3", "--max-new-tokens", "4"])
    err = [l for l in capsys.readouterr().err.strip().splitlines() if l.startswith("error:")]
    assert rc == 1 and len(err) == 1 and "bounded wait" in err[0]
    rc = cli.run(["logits", "--model", folder, "--dtype", "float32", "--tokens", "1 2 3"])
    assert rc == 1 and "bounded wait" in capsys.readouterr().err


def test_samplers_note_rows_that_are_not_finite():
    require_gpu()
    from hilbert_pruned_8b_b200.kernels.ops import KernelError, Ops
    ops = Ops(torch.device(DEV))
    torch.manual_seed(3)
    logits = torch.randn(5, 1003, device=DEV)
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    assert ops.status.tolist() == [0, 0, 0, 0] and torch.equal(out.long(), logits.argmax(dim=1))
    for bad, row, col in ((float("nan"), 3, 1002), (float("inf"), 1, 0), (float("-inf"), 4, 500)):
        poisoned = logits.clone()
        poisoned[row, col] = bad
        ops.argmax(poisoned, out)
        assert ops.status.tolist() == [0, 1 + row, 0, 0]
        with pytest.raises(KernelError, match=f"non-finite logits at row {row}"):
            ops.check_errors()
        assert ops.status.tolist() == [0, 0, 0, 0]
        t = torch.full((5,), 0.9, device=DEV)
        z = torch.zeros(5, dtype=torch.int64, device=DEV)
        ops.sample(poisoned, t, z, z, z, out)
        assert ops.status.tolist() == [0, 1 + row, 0, 0]
        ops.reset_status()
    unaligned = torch.randn(3, 1001, device=DEV)[:, 1:]                 # rows that do not start on 16 bytes
    ops.argmax(unaligned, out[:3])
    assert ops.status.tolist() == [0, 0, 0, 0]


def test_a_page_number_outside_the_cache_is_noted_not_followed():
    """A page table that names a page the cache does not have (a fault of the host's bookkeeping,
    written here by hand): the append skips the write, attention reads page 0 instead, the status
    word names the sequence, and everything stays finite."""
    require_gpu()
    import types
    from hilbert_pruned_8b_b200.cache.manager import LayerCache
    from hilbert_pruned_8b_b200.kernels.ops import KernelError, Ops
    ops = Ops(torch.device(DEV))
    nh, nkv, hd, n_pages, B = 8, 2, 64, 6, 3
    torch.manual_seed(4)
    for dtype in (torch.bfloat16, torch.float32):
        k = torch.randn(n_pages, nkv, 64, hd, device=DEV).to(dtype)
        cache = LayerCache(k, k.clone(), 0, None)
        pt = torch.tensor([[0, 1], [2, 77], [4, -1]], dtype=torch.int32, device=DEV)      # 77: outside; -1: missing
        pos = torch.tensor([70, 100, 30], dtype=torch.int32, device=DEV)
        step = types.SimpleNamespace(page_tables=[pt], positions=pos, tok_seq=torch.arange(B, dtype=torch.int32, device=DEV),
                                     num_tokens=B, num_seqs=B, max_len=128, is_decode=True, host_new=[1] * B,
                                     seq_start=torch.arange(B + 1, dtype=torch.int32, device=DEV), seq_pos0=pos)
        qkv = torch.randn(B, (nh + 2 * nkv) * hd, device=DEV).to(dtype)
        table = torch.zeros(B, hd // 2, 2, device=DEV)
        table[..., 0] = 1.0
        before = cache.k.clone()
        ops.rope_kv_append(qkv, table, hd, nh, nkv, hd, cache, step, True)
        assert ops.status.tolist() == [0, 0, 2, 0]                       # sequence 1 (the first one noted)
        ops.reset_status()
        assert torch.equal(cache.k[3], before[3]) and torch.equal(cache.k[5], before[5])   # nothing written elsewhere
        out = torch.empty(B, nh * hd, device=DEV, dtype=dtype)
        ops.attention(qkv, nh, nkv, hd, cache, step, out, 0.125, None)
        assert ops.status[2].item() == 2 and torch.isfinite(out.float()).all()
        with pytest.raises(KernelError, match="sequence 1"):
            ops.check_errors()
        if dtype == torch.bfloat16:
            ops.attention_decode_fused(qkv, table, hd, nh, nkv, hd, cache, step, out, 0.125, None, True)
            assert ops.status[2].item() == 2 and torch.isfinite(out.float()).all()
            ops.reset_status()
        good = torch.tensor([[0, 1], [2, 3], [4, 5]], dtype=torch.int32, device=DEV)
        step.page_tables = [good]
        ops.rope_kv_append(qkv, table, hd, nh, nkv, hd, cache, step, True)
        ops.attention(qkv, nh, nkv, hd, cache, step, out, 0.125, None)
        assert ops.status.tolist() == [0, 0, 0, 0]
