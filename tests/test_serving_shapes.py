"""The schedules that serving runs, against the plain implementation: two layers at the widths
of real checkpoints of the architecture (8B and 1B shapes) with the FULL vocabulary of 128256,
batches of 8, 24, 64 and 128 sequences with unequal prompts in one step, then decode steps
through the captured graphs while the shorter requests leave (batch sizes change, slots and
pages are used again), in bfloat16 and in 32-bit.  That covers what the tiny models never reach:
the token tiles 16/32/64/128 of the tensor-core product with their cluster sums and cut tiles,
the head at 1002 tiles, decode attention with one split per sequence and with whole waves.

The engine draws its weights ON THE DEVICE from a seed; the plain model reads the folder that
the CPU wrote from the same seed: the two draws are the same model bit for bit, or nothing here
passes.  The plain model does its float64 arithmetic with torch on the GPU for these sizes.
"""
import math

import pytest
import torch

import trace_tools as tt
from conftest import require_gpu
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
VOCAB = 128256
LLAMA3 = dict(rope_type="llama3", low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
SHAPES = {
    "8b": dict(hidden_size=4096, intermediate_size=14336, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               tie_word_embeddings=False, rope_scaling=dict(LLAMA3, factor=8.0)),
    "1b": dict(hidden_size=2048, intermediate_size=8192, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
               tie_word_embeddings=True, rope_scaling=dict(LLAMA3, factor=32.0)),
}
SEEDS = {"8b": 71, "1b": 72}
DRAW = dict(std=0.02, norm_std=0.05, fan_in_scale=1.0)


def _config(shape):
    import hilbert_pruned_8b_b200 as hb
    return hb.LlamaConfig.from_dict(dict(
        architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", num_hidden_layers=2, vocab_size=VOCAB,
        rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192, **SHAPES[shape]))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """name -> folder written from the CPU draw (made when first asked for)."""
    import hilbert_pruned_8b_b200 as hb
    made = {}

    def get(shape):
        if shape not in made:
            d = str(tmp_path_factory.mktemp(f"serving_{shape}"))
            hb.weights.write_random_model(d, _config(shape), seed=SEEDS[shape], **DRAW)
            made[shape] = d
        return made[shape]
    return get


def test_device_draw_equals_cpu_draw(folders):
    """Random weights are a function of (seed, tensor name, element): the tensors the kernel
    draws on the device equal, bit for bit, the folder the CPU wrote, whatever the order."""
    require_gpu()
    from hilbert_pruned_8b_b200.engine.model import weight_table
    from hilbert_pruned_8b_b200.weights import SafetensorsFolder, random_tensors
    cfg = _config("8b")
    table = weight_table(cfg.model_spec())
    names = [n for n in reversed(list(table)) if not table[n].optional]          # another order than the writer's
    dev = random_tensors({n: table[n] for n in names}, SEEDS["8b"], torch.device(DEV), dtype=torch.bfloat16, **DRAW)
    folder = SafetensorsFolder(folders("8b"))
    try:
        assert sorted(folder.names()) == sorted(names)
        for n in names:
            want = folder.tensor(n)
            assert want.dtype == torch.bfloat16 and torch.equal(dev[n].cpu().view(torch.int16), want.view(torch.int16)), n
    finally:
        folder.close()
    # in 32-bit too (no rounding to hide a last bit), on a matrix and a norm vector
    name = "model.layers.1.mlp.down_proj.weight"
    for n, kw in ((name, {}), ("model.norm.weight", {})):
        a = random_tensors({n: table[n]}, 5, torch.device(DEV), dtype=torch.float32, **DRAW)[n]
        b = random_tensors({n: table[n]}, 5, torch.device("cpu"), dtype=torch.float32, **DRAW)[n]
        assert torch.equal(a.cpu().view(torch.int32), b.view(torch.int32)), n


def _batches(sizes, seed):
    """Batches of unequal prompts; every request decodes at least 4 tokens (so the captured graph
    of the full batch is replayed), the shorter ones leave earlier."""
    g = torch.Generator().manual_seed(seed)
    batches, reqs = [], {}
    for b, size in enumerate(sizes):
        batch = {}
        for i in range(size):
            prompt = int(torch.randint(1, 41, (1,), generator=g))
            if i == 0:
                prompt = 70                              # one prompt over a page
            if i == 1:
                prompt = 600                             # and one over many: decode attention cuts its keys into several splits
            new = 4 + int(torch.randint(0, 7, (1,), generator=g))
            rid = f"b{b}r{i}"
            reqs[rid] = [int(t) for t in torch.randint(0, VOCAB, (prompt + new,), generator=g)]
            batch[rid] = (reqs[rid], prompt)
        batches.append(batch)
    return batches, reqs


def _run_and_compare(eng, plain, batches, reqs, dtype, what):
    """Runs the batches one after another through ``Engine.step_chunked`` and compares, step by
    step on the device, the logits of every prompt's last position and of every decoded position."""
    from hilbert_pruned_8b_b200.engine.batch import StepEntry
    ref = {}
    for rid, toks in reqs.items():
        prompt = next(b[rid][1] for b in batches if rid in b)
        places = list(range(prompt - 1, len(toks)))
        lg = plain.logits_at(toks, places)
        for row, p in enumerate(places):
            ref[(rid, p)] = lg[row]
    steps, _ = tt.trace_batches(batches, want_all=False)
    places = tt.wanted_places(steps)
    seqs, worst, compared, sizes = {}, 0.0, 0, set()
    for s in steps:
        entries = []
        for e in s["entries"]:
            if e["id"] not in seqs:
                seqs[e["id"]] = eng.open_sequence()
            entries.append(StepEntry(seqs[e["id"]], e["tokens"], e["want"]))
        logits = eng.step_chunked(entries)
        if all(len(e["tokens"]) == 1 for e in s["entries"]):
            sizes.add(len(entries))
        got = logits.double()
        assert torch.isfinite(got).all(), f"{what}: non-finite logits at step {s['step']}"
        for row, key in enumerate(places[s["step"]]):
            r = ref[key]
            if dtype == "float32":
                err, bound = ((got[row] - r).abs() / r.abs().clamp(min=1.0)).max().item(), 1e-4
            else:
                err, bound = (got[row] - r).abs().max().item() / max(1e-3, r.abs().max().item()), 0.02
            worst = max(worst, err)
            assert err <= bound, f"{what}: {dtype} logits differ at request {key[0]} position {key[1]} (step {s['step']}, " \
                                 f"{len(entries)} sequences): {err:.3e} > {bound}"
            compared += 1
        for rid in s["end"]:
            eng.close_sequence(seqs.pop(rid))
    assert not seqs and compared == len(ref)
    assert min(eng.cache.pages_free()) == eng.cache.num_pages and eng.cache.slots.num_held == 0
    return worst, sizes


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("shape", ["8b", "1b"])
def test_batches_of_8_24_64_128_through_the_graphs(folders, shape, dtype):
    require_gpu()
    from hilbert_pruned_8b_b200.engine.step import Engine
    batches, reqs = _batches([8, 24, 64, 128], seed=1000 + len(shape))
    peak = max(sum(tt.round64(len(t)) for t, _ in b.values()) for b in batches)
    eng = Engine.from_random(_config(shape), SEEDS[shape], dtype, max_tokens=peak, device=DEV, max_step_tokens=8192,
                             max_sequences=128, **DRAW)
    plain = PlainLlama(folders(shape), round_to=torch.bfloat16 if dtype == "bfloat16" else None, device=DEV)
    replays0 = eng.graph_replays
    worst, sizes = _run_and_compare(eng, plain, batches, reqs, dtype, f"{shape} widths")
    assert {8, 24, 64, 128} <= sizes
    assert eng.graph_replays - replays0 >= 4 * 2          # every full batch ran its captured graph more than once
    eng.check_status()


@pytest.mark.parametrize("K", [2048, 3072, 4096])
def test_head_product_at_the_full_vocabulary(K):
    """The output head's product, N = 128256 (1002 tiles of 128 rows: cut tiles first, whole
    tiles after), at the hidden widths of the 1B, 3B and 8B shapes, for 1, 8, 64 and 130 rows,
    row-major and tiled weights, against float64."""
    require_gpu()
    from hilbert_pruned_8b_b200.kernels.ops import Ops
    ops = Ops(torch.device(DEV))
    torch.manual_seed(K)
    w = (torch.randn(VOCAB, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    packed = ops.pack_weight(w)
    wd = w.double()
    for M in (1, 8, 64, 130):
        a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        ref = a.double() @ wd.t()
        out = torch.empty(M, VOCAB, device=DEV)
        ops.linear(a, w, out)
        ops.check_errors()
        err = ((out.double() - ref).abs().max() / ref.abs().max()).item()
        assert err < 2e-6 * math.sqrt(K), (M, K, err)
        tiled = torch.empty(M, VOCAB, device=DEV)
        ops.linear(a, packed, tiled)
        ops.check_errors()
        assert torch.equal(out, tiled), (M, K)
        # the largest logit and its index are what the sampler reads: the same as the reference's
        assert torch.equal(out.argmax(dim=1), ref.argmax(dim=1)) or \
            (ref.max(dim=1).values - ref.gather(1, out.argmax(dim=1, keepdim=True)).squeeze(1)).abs().max() < 1e-4
        assert int(ops._splitk_counters.abs().sum()) == 0
