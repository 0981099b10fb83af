"""Decode and prefill throughput of the Llama-3.1-8B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
    python bench.py --workload 3b|1b      # a line of its own: unequal prompts, then decoding
    python bench.py --timeline --layers 3 --skip-points    # per-kernel times inside the decode graph

Prints ONE JSON line.  A step is one decode step of a batch of 8 sequences whose caches hold
about 8192 tokens each; ``value`` is decoded tokens per second from CUDA events around the
steps; ``e2e`` is the same through the library's generation loop with host tokens in and out
(pinned host memory -> device every step, sampled tokens device -> host every step).
``prefill`` times one 2048-token prompt; ``roofline`` relates the decode step to the HBM
bandwidth it needs (every weight once + the live sequences' cache); ``points`` adds decoding
at batch 1 and 64, prefill at 512, 8192 and 32768 tokens, and steady decoding at the 3B and 1B
shapes (batch 16 and 64) with the fraction of the HBM peak each reaches.  Weights (15 GB) exceed L2 (126 MB), so every step reads them from HBM.
The caches of the decode benchmark are filled with random keys and values instead of being
prefilled; a decode step's work does not depend on their values.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Llama-3.1-8B-shaped
MODEL_8B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", hidden_size=4096,
    num_hidden_layers=32, intermediate_size=14336, vocab_size=128256, num_attention_heads=32,
    num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=False, max_position_embeddings=131072)
# BASELINE.json configs[3] and configs[4]: generation workloads at the 3B and 1B shapes
# (--workload 3b | 1b): (model, batch, prompt lengths uniform in [lo, hi], decode steps)
LLAMA3_32 = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                 original_max_position_embeddings=8192)
MODEL_3B = dict(MODEL_8B, hidden_size=3072, num_hidden_layers=28, intermediate_size=8192, num_attention_heads=24,
                rope_scaling=LLAMA3_32, tie_word_embeddings=True)
MODEL_1B = dict(MODEL_8B, hidden_size=2048, num_hidden_layers=16, intermediate_size=8192, head_dim=64,
                rope_scaling=LLAMA3_32, tie_word_embeddings=True)
WORKLOADS = {"3b": (MODEL_3B, "llama-3.2-3b-shaped", 16, 64, 1024, 128),
             "1b": (MODEL_1B, "llama-3.2-1b-shaped", 64, 16, 512, 256)}
CONTEXT = 8192
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        out = {k: float(p[k]) for k in FALLBACK_PEAKS if k in p}
        if "hbm_gbs" in out and "bf16_tflops" in out:
            out.setdefault("bf16_tflops_sustained", out["bf16_tflops"])
            return out, "measured"
    except (OSError, ValueError, KeyError, TypeError):
        pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0])), mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def fill_cache_random(llm, seed=1):
    """Random keys and values in the whole cache (stands for prefilled prompts)."""
    import torch
    g = torch.Generator(device=llm.engine.device).manual_seed(seed)
    for grp in llm.engine.cache.groups:
        for t in (grp.k, grp.v):
            flat = t.view(-1)
            step = 1 << 28
            for i in range(0, flat.numel(), step):
                part = flat[i:i + step]
                part.copy_(torch.randn(part.numel(), generator=g, device=part.device, dtype=torch.float32) * 0.5)


def open_filled(llm, batch, length):
    """`batch` sequences whose caches already hold `length` tokens."""
    seqs = []
    for _ in range(batch):
        s = llm.engine.open_sequence()
        llm.engine.cache.reserve([(s, length)])
        llm.engine.cache.commit(s, length)
        seqs.append(s)
    return seqs


def time_decode(llm, batch, steps, warmup, length, sampler=None):
    """Device time of `steps` decode steps of `batch` sequences at about `length` cached tokens."""
    import torch
    from hilbert_pruned_8b_b200.engine.batch import StepEntry
    eng = llm.engine
    seqs = open_filled(llm, batch, length - steps - warmup - 1)
    gen = torch.Generator().manual_seed(5)
    vocab = eng.vocab_size
    toks = torch.randint(0, vocab, (steps + warmup, batch), generator=gen).tolist()
    for w in range(warmup):
        eng.step([StepEntry(s, [toks[w][b]], [0]) for b, s in enumerate(seqs)], greedy=True)
    torch.cuda.synchronize()
    launches0 = eng.ctx.ops.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks = sampler
    if clocks:
        clocks.start()
    start.record()
    for k in range(steps):
        # the greedy pick is the last kernel of the step's captured graph
        eng.step([StepEntry(s, [toks[warmup + k][b]], [0]) for b, s in enumerate(seqs)], greedy=True)
    end.record()
    torch.cuda.synchronize()
    eng.check_status()                 # a kernel that noted a fault makes the number worthless: raise
    ms = start.elapsed_time(end) / steps
    clock_info = clocks.stop() if clocks else None
    launches = eng.ctx.ops.launches - launches0
    lengths = [s.length for s in seqs]
    step_bytes = eng.decode_step_bytes(lengths)
    for s in seqs:
        eng.close_sequence(s)
    return ms, launches, step_bytes, clock_info


def time_e2e(llm, batch, steps, warmup, length):
    """The generation loop's decode phase: host tokens in, host tokens out, every step."""
    import torch
    from hilbert_pruned_8b_b200.engine.generate import GenerationRequest
    from hilbert_pruned_8b_b200.sampling import SamplingParams
    eng = llm.engine
    gen = llm.generator
    seqs = open_filled(llm, batch, length - steps - warmup - 2)
    req = GenerationRequest([0], max_new_tokens=warmup, sampling=SamplingParams(0.0, 0), stop_token_ids=[])
    live = {b: {"req": req, "rid": b, "stop": [], "seq": s, "out": [], "next": (17 * b + 3) % eng.vocab_size}
            for b, s in enumerate(seqs)}
    results = [None] * batch
    # warm-up steps through the same loop (it closes nothing: budgets are per phase here)
    for st in live.values():
        st["req"] = GenerationRequest([0], max_new_tokens=10 ** 9, sampling=SamplingParams(0.0, 0), stop_token_ids=[])
    _run_steps(gen, live, results, warmup)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _run_steps(gen, live, results, steps)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    eng.check_status()
    for s in seqs:
        eng.close_sequence(s)
    h2d = _step_meta_bytes(eng, batch, length)
    return batch * steps / dt, h2d, batch * 4 + 16      # the tokens and the four status words


def _run_steps(gen, live, results, n):
    """`n` steps of Generator.decode: budgets are set so that the loop returns after n tokens."""
    from hilbert_pruned_8b_b200.engine.generate import GenerationRequest
    from hilbert_pruned_8b_b200.sampling import SamplingParams
    if n <= 0:
        return
    keep = dict(live)
    for st in live.values():
        st["req"] = GenerationRequest([0], max_new_tokens=len(st["out"]) + n, sampling=SamplingParams(0.0, 0),
                                      stop_token_ids=[])
    closed = []
    orig_close = gen.engine.close_sequence
    gen.engine.close_sequence = lambda seq: closed.append(seq)      # keep the caches for the next phase
    try:
        gen.decode(live, results)
    finally:
        gen.engine.close_sequence = orig_close
    live.update(keep)


def _step_meta_bytes(eng, batch, length):
    """Bytes of the per-step host-to-device copy (tokens, positions, page tables, ...)."""
    from hilbert_pruned_8b_b200.cache import pages_for
    per_seq = 3 + 4 + pages_for(length) * max(1, len(eng.cache.groups))
    return 4 * (batch * per_seq + 8)


def other_shape_point(name, steps, pk):
    """Steady decoding at the 3B / 1B shapes with their workloads' batch and a cache length in the
    middle of what that workload reaches: tokens/s, ms per step, GB/s and the fraction of the HBM
    peak, as flat keys for `points`."""
    import torch
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.api import LLM
    cfg_dict, label, batch, lo, hi, new_tokens = WORKLOADS[name]
    length = (lo + hi) // 2 + new_tokens // 2
    cfg = hb.LlamaConfig.from_dict(cfg_dict)
    llm = LLM.random(cfg, seed=0, dtype="bfloat16", max_tokens=batch * ((length + 127) // 64 * 64), device=0,
                     max_batch=batch, max_step_tokens=256)
    fill_cache_random(llm)
    ms, _, step_bytes, _ = time_decode(llm, batch, steps, 3, length)
    del llm
    torch.cuda.empty_cache()
    gbs = step_bytes / (ms * 1e-3) / 1e9
    key = f"decode_{name}_b{batch}"
    return {key: round(batch / (ms * 1e-3), 1), key + "_ms": round(ms, 4), key + "_gbs": round(gbs, 1),
            key + "_frac": round(gbs / pk["hbm_gbs"], 4), key + "_ctx": length}


def time_prefill(llm, tokens, repeats=3, warmup=2):
    import torch
    from hilbert_pruned_8b_b200.engine.batch import StepEntry
    eng = llm.engine
    gen = torch.Generator().manual_seed(9)
    toks = torch.randint(0, eng.vocab_size, (tokens,), generator=gen).tolist()
    times = []
    for i in range(warmup + repeats):
        s = eng.open_sequence()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step_chunked([StepEntry(s, toks, [tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
        eng.close_sequence(s)
    return statistics.median(times)


def prefill_flops(cfg, layers, tokens):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = 2 * tokens * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I)
    attn = 2 * tokens * tokens * hd * nh          # causal: QK^T and PV over half the square each
    return layers * (per_layer + attn) + 2 * H * V


def generation_workload(name, repeats, warmup):
    """A batch of unequal prompts through the Python entry point (host tokens in and out):
    all prompts in one step, then a fixed number of decode steps (no stop tokens).  One JSON
    line of its own; the default line (8B shape) is not affected."""
    import torch
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.api import LLM
    cfg_dict, label, batch, lo, hi, new_tokens = WORKLOADS[name]
    cfg = hb.LlamaConfig.from_dict(cfg_dict)
    g = torch.Generator().manual_seed(11)
    lengths = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lengths]
    max_tokens = sum((n + new_tokens + 63) // 64 * 64 for n in lengths)
    llm = LLM.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, device=0, max_batch=batch,
                     max_step_tokens=max(PREFILL_TOKENS, hi))
    llm.generator._sync = torch.cuda.synchronize     # so that the phase times split at the right place
    runs = []
    clocks = ClockSampler()
    for i in range(warmup + repeats):
        if i == warmup:
            clocks.start()
        st = llm.generator.stats = type(llm.generator.stats)()
        launches0 = llm.engine.ctx.ops.launches
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = llm.generate(prompts, max_new_tokens=new_tokens, temperature=0.0, stop_token_ids=[])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert all(len(r.tokens) == new_tokens for r in out)
        runs.append((dt, st.prefill_seconds, st.decode_seconds, st.decode_steps, llm.engine.ctx.ops.launches - launches0))
    clock_info = clocks.stop()
    dt, pre_s, dec_s, dec_steps, launches = sorted(runs[warmup:])[len(runs[warmup:]) // 2]
    dec_tokens = batch * (new_tokens - 1)            # the first token of each comes from the prompt step
    pk, pk_src = peaks()
    mean_len = [n + new_tokens // 2 for n in lengths]
    step_bytes = llm.engine.decode_step_bytes(mean_len)
    ms = dec_s / max(1, dec_steps) * 1e3
    line = {
        "metric": f"decode tok/s, batch {batch}, prompts uniform in [{lo}, {hi}], {new_tokens} new tokens ({label}, random weights)",
        "value": round(dec_tokens / dec_s, 1), "unit": "tokens/s", "n_gpus": 1, "steps": dec_steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights, random token ids", "impl": "ours",
        "config": {"model": label, "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": batch,
                   "prompt_tokens": sum(lengths), "new_tokens": new_tokens, "parallelism": "single-gpu",
                   "timing": "host clock around the generation loop's phases, device synchronised", "peaks": pk_src},
        "e2e": {"value": round(batch * new_tokens / dt, 1), "unit": "generated tokens/s, prompts included in the time",
                "seconds": round(dt, 4)},
        "gpu_launches": launches,
        "prefill": {"value": round(sum(lengths) / pre_s, 1), "tokens": sum(lengths), "ms": round(pre_s * 1e3, 3),
                    "frac": round(sum(prefill_flops_varlen(cfg_dict, lengths)) / pre_s / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(step_bytes / (ms * 1e-3) / 1e9, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)},
        "clocks": clock_info,
    }
    print(json.dumps(line))
    return 0


def prefill_flops_varlen(cfg, lengths):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    L = cfg["num_hidden_layers"]
    return [L * (2 * n * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I) + 2 * n * n * hd * nh) + 2 * H * V
            for n in lengths]


def timeline_table(llm, batch, context, steps=8):
    """Per-kernel times of decode steps inside the replayed graph (timeline build of the
    kernel library): for every kernel the time from the moment it found its predecessors
    finished to the moment its successor did, overlap between neighbours included, and how
    long before that moment its first block was already resident."""
    import torch
    from hilbert_pruned_8b_b200.engine.batch import StepEntry
    eng = llm.engine
    ops = eng.ctx.ops
    seqs = open_filled(llm, batch, context - steps - 8)

    def one(k):
        eng.step([StepEntry(s, [(7 * k + b) % 1000], [0]) for b, s in enumerate(seqs)], greedy=True)

    ops.call_log = []
    one(0)                                   # the first step runs eagerly: its calls name the kernels
    names = []
    for n in ops.call_log:
        if n == "hb_attention_decode":
            names += ["attention_decode", "attention_decode_combine"]
        elif n == "hb_attention_decode_combined":
            names.append("attention_decode")
        elif n == "hb_attention_decode_fused":      # rotation and append inside; a single split has no combine kernel
            names += ["attention_decode_fused", "attention_decode_combine"]
        elif n not in ("hb_device_info", "hb_timeline_set"):
            names.append(n[3:])
    ops.call_log = None
    for k in range(1, 5):
        one(k)
    torch.cuda.synchronize()
    ops.timeline_begin(1 << 20)
    for k in range(steps):
        one(5 + k)
    marks = [m for m in ops.timeline_end() if m[0] > 10 ** 9]      # kernel marks (events carry small codes)
    per = len(marks) // steps
    if per == len(names) - names.count("attention_decode_fused"):
        names = [n for n in names if n != "attention_decode_combine"]
    if per != len(names):
        names = [f"kernel {i}" for i in range(per)]
    rows, total = [], 0.0
    for i in range(per):
        dur = [marks[s * per + i + 1][1] - marks[s * per + i][1] for s in range(1, steps - 1)]
        lead = [marks[s * per + i][1] - marks[s * per + i][0] for s in range(1, steps - 1)]
        d, l = statistics.median(dur) / 1e3, statistics.median(lead) / 1e3
        total += d
        rows.append((i, names[i], d, l))
    print(f"decode step, batch {batch}, context {context}, {llm.config.num_hidden_layers} layers: "
          f"{per} kernels, {total:.1f} us (sum of medians over {steps - 2} replayed steps)")
    print("   #  kernel                          us    resident before its predecessors finished (us)")
    for i, n, d, l in rows:
        print(f"{i:4d}  {n:28s} {d:8.2f} {l:10.2f}")
    for s in seqs:
        eng.close_sequence(s)
    return 0


NO_DECODE = ("decode tokens/s: the reference generates nothing (no decode loop, no sampler: "
             "cleanroom-transformer/README.md:7-10; its Python package only scores answer options of text rows "
             "through transformers and needs a tokenizer and a hub revision)")


def reference_arm(a) -> int:
    """The UNMODIFIED reference on the same box, for the one part of the metric it can measure: the
    warm 2048-token prefill that its own ``selftest`` command times and prints
    (cleanroom-transformer/src/cuda_backend.cu:1449-1457).  The binary is the reference's CUDA
    build, made by its own Makefile with its stock flags (``make cuda``: sm_86 code plus
    compute_86 PTX, which the driver compiles for this GPU) under ``baseline/_ref/ct/``; the model
    folder is the 8B-shaped random model of the default arm (same seed, same bits), written to a
    temporary folder.  It has no decode loop, so ``value`` (decode tokens/s) stays unavailable."""
    import re
    import shutil
    import tempfile
    ct = os.path.join(ROOT, "baseline", "_ref", "ct")
    binary = os.path.join(ct, "build", "cleanroom-transformer-cuda")
    line = {"impl": "reference", "unavailable": NO_DECODE}
    if a.gpus != 1:
        print(json.dumps(line))
        return 0
    if not os.path.isfile(binary) and os.path.isfile(os.path.join(ct, "Makefile")):
        subprocess.run(["make", "-C", ct, "cuda", "CC=/usr/bin/gcc"], capture_output=True, text=True)
    if not os.path.isfile(binary):
        line["prefill"] = {"unavailable": "the reference's CUDA build is not installed under baseline/_ref/ct "
                                          "(copy cleanroom-transformer/ there and run `make cuda CC=/usr/bin/gcc`)"}
        print(json.dumps(line))
        return 0
    import torch
    import hilbert_pruned_8b_b200 as hb
    cfg_dict = dict(MODEL_8B)
    layers = a.layers or cfg_dict["num_hidden_layers"]
    cfg_dict["num_hidden_layers"] = layers
    folder = tempfile.mkdtemp(prefix="hilbert_b200_reference_model_")
    try:
        t0 = time.time()
        hb.weights.write_random_model(folder, hb.LlamaConfig.from_dict(cfg_dict), seed=0, device="cuda:0")
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        write_s = time.time() - t0
        env = dict(os.environ)
        env["LD_LIBRARY_PATH"] = os.pathsep.join(filter(None, [env.get("LD_LIBRARY_PATH"), "/usr/local/cuda/lib64"]))
        clocks = ClockSampler()
        clocks.start()
        t0 = time.time()
        try:
            res = subprocess.run([binary, "selftest", "--tokens", "2", "--model", folder], capture_output=True, text=True,
                                 env=env, timeout=1500)
            out, err, rc = res.stdout, res.stderr, res.returncode
        except subprocess.TimeoutExpired as e:
            out, err, rc = (e.stdout or b"").decode("utf-8", "replace") if isinstance(e.stdout, bytes) else (e.stdout or ""), \
                "selftest did not end within 1500 s", 124
        run_s = time.time() - t0
        clock_info = clocks.stop()
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    m = re.search(r"cuda prefill (\d+) tokens: ([0-9.]+) ms \(([0-9.]+) tokens/s\)", out)
    pk, pk_src = peaks()
    if m:
        tokens, ms = int(m.group(1)), float(m.group(2))
        line["prefill"] = {"value": round(tokens / (ms * 1e-3), 1), "tokens": tokens, "ms": round(ms, 3),
                           "frac": round(prefill_flops(cfg_dict, layers, tokens) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                           "timer": "the reference's own: host clock around its second (warm) prefill, device synchronised"}
    else:
        tail = (err.strip().splitlines() or out.strip().splitlines() or ["no output"])[-1]
        line["prefill"] = {"unavailable": f"the reference's selftest printed no prefill time (exit code {rc}): {tail[:300]}"}
    checks = [l.strip() for l in out.splitlines() if l.strip().endswith(("ok", "FAIL")) and "cuda vs cpu" in l]
    line.update({
        "metric": "prefill tok/s @ 2048 tokens (Llama-3.1-8B-shaped, random weights), the reference's own selftest timer",
        "unit": "tokens/s", "n_gpus": 1, "steps": 1, "warmup": 1, "dtype": "bf16 weights and GEMM inputs, float32 activations and cache",
        "data": "synthetic: random weights (the default arm's seed), the selftest's own token ids",
        "config": {"model": "llama-3.1-8b-shaped", "layers": layers, "layers_in_config": MODEL_8B["num_hidden_layers"],
                   "hidden": cfg_dict["hidden_size"], "vocab": cfg_dict["vocab_size"], "prefill_tokens": PREFILL_TOKENS,
                   "command": "cleanroom-transformer-cuda selftest --tokens 2 --model DIR", "build": "make cuda (stock flags: sm_86 + compute_86 PTX)",
                   "peaks": pk_src},
        "selftest_exit_code": rc, "selftest_checks": checks[:4], "model_write_s": round(write_s, 1), "selftest_s": round(run_s, 1),
        "clocks": clock_info})
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", choices=("8b", "3b", "1b"), default="8b",
                    help="layer sizes of the steady-decode line and of --timeline (default: the 8B shape of the contract)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each sequence's cache holds while decoding")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                    help="float32: the true 32-bit path (FP32-pipe products, general attention), a line of its own; "
                         "give --layers to keep it short")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--workload", choices=("8b", "3b", "1b"), default="8b",
                    help="8b: the default line; 3b, 1b: the generation workloads at those shapes (--steps = repeats)")
    ap.add_argument("--timeline", action="store_true",
                    help="print the per-kernel times of a decode step inside the replayed graph (builds the "
                         "timeline variant of the kernel library) instead of the JSON line")
    a = ap.parse_args()
    if a.timeline:
        os.environ["HILBERT_B200_TIMELINE"] = "1"      # before the kernel library is looked for
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {a.gpus} is not supported by this single-GPU library")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.workload != "8b":
        return generation_workload(a.workload, repeats=min(a.steps, 3), warmup=1)

    import torch
    import hilbert_pruned_8b_b200 as hb
    from hilbert_pruned_8b_b200.api import LLM

    cfg_dict = dict({"8b": MODEL_8B, "3b": MODEL_3B, "1b": MODEL_1B}[a.shape])
    shape_name = {"8b": "llama-3.1-8b-shaped", "3b": "llama-3.2-3b-shaped", "1b": "llama-3.2-1b-shaped"}[a.shape]
    context = a.context
    full_layers = cfg_dict["num_hidden_layers"]
    layers = a.layers or full_layers
    cfg_dict["num_hidden_layers"] = layers
    cfg = hb.LlamaConfig.from_dict(cfg_dict)
    pk, pk_src = peaks()
    fp32 = a.dtype == "float32"
    if fp32:
        a.skip_points = True            # the other points are about the serving precision
    max_batch = 64 if not a.skip_points else a.batch
    max_tokens = max(max_batch * ((context + 127) // 64 * 64), 64 * 1024 if not a.skip_points else 0, PREFILL_TOKENS)
    t_build = time.time()
    llm = LLM.random(cfg, seed=0, dtype=a.dtype, max_tokens=max_tokens, device=0, max_batch=max_batch,
                     max_step_tokens=PREFILL_TOKENS)
    fill_cache_random(llm)
    torch.cuda.synchronize()
    build_s = time.time() - t_build

    if a.timeline:
        return timeline_table(llm, a.batch, context)
    prefill_ms = time_prefill(llm, PREFILL_TOKENS)
    pf = prefill_flops(cfg_dict, layers, PREFILL_TOKENS)
    ms, launches, step_bytes, clocks = time_decode(llm, a.batch, a.steps, a.warmup, context, ClockSampler())
    e2e, h2d, d2h = time_e2e(llm, a.batch, a.steps, a.warmup, context)
    points = {}
    if not a.skip_points:
        for b in (1, 64):
            pms, _, pbytes, _ = time_decode(llm, b, max(4, a.steps // 2), 3, context)
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
            points[f"decode_b{b}_frac"] = round(pbytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        # prefill at other lengths (cut into steps of 2048 tokens): tokens/s
        for t in (512, 8192, 32768):
            pms = time_prefill(llm, t, repeats=2, warmup=1)
            points[f"prefill_t{t}"] = round(t / (pms * 1e-3), 1)
            points[f"prefill_t{t}_frac"] = round(prefill_flops(cfg_dict, layers, t) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        del llm
        torch.cuda.empty_cache()
        # decoding at the 3B and 1B shapes (their workloads' batch sizes)
        for name in ("3b", "1b"):
            points.update(other_shape_point(name, max(8, a.steps), pk))
    achieved = step_bytes / (ms * 1e-3) / 1e9
    value = a.batch / (ms * 1e-3)
    # the 32-bit path runs on the FP32 pipe: its prefill fraction is of that pipe's nominal peak
    # (148 SMs x 128 lanes x 2 flop x 1.965 GHz), not of the tensor cores'
    flop_peak = 148 * 128 * 2 * 1.965e9 if fp32 else pk["bf16_tflops"] * 1e12
    line = {
        "metric": f"decode tok/s @ batch {a.batch}, context {context} ({shape_name.replace('llama', 'Llama').replace('b-shaped', 'B-shaped')}, "
                  "random weights)" + (", true 32-bit path" if fp32 else ""),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32" if fp32 else "bf16", "data": "synthetic: random weights, random token ids, random cache contents",
        "impl": "ours",
        "config": {"model": shape_name, "layers": layers, "layers_in_config": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": a.batch, "seq_len": context, "prefill_tokens": PREFILL_TOKENS,
                   "parallelism": "single-gpu", "l2": "weights (15 GB) exceed L2; every step reads them from HBM",
                   "peaks": pk_src, "hbm_gbs_peak": pk["hbm_gbs"], "bf16_tflops_peak": pk["bf16_tflops"]},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(pf / (prefill_ms * 1e-3) / flop_peak, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
        "setup_s": round(build_s, 1),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
