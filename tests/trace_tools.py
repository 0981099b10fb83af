"""Builds replay traces (the step objects bin/trace_run reads), runs them in-process or
through the program, and compares the logits with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]


def round64(n):
    return (n + 63) // 64 * 64


def trace_whole(requests):
    """Each request alone and whole; logits at every position."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps, max(round64(len(t)) for t in requests.values())


def trace_tail(requests, tail=32):
    """Each request alone: the head in one step, the last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": [rid] if head == len(toks) else []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
    return steps, max(round64(len(t)) for t in requests.values())


def trace_batches(batches, want_all=True):
    """`batches`: list of {id: (tokens, prompt_len)}.  A batch's prompts start together in one
    step, then every live request feeds one token per step; a request ends when its tokens
    are used up, the shorter ones earlier.  Batches follow one another, so slots are reused.
    Logits are wanted at every position, or (`want_all` False) at each prompt's last position
    and at every position after it."""
    steps, peak = [], 0
    for batch in batches:
        peak = max(peak, sum(round64(len(t)) for t, _ in batch.values()))
        fed = {rid: p for rid, (t, p) in batch.items()}
        entries = [{"id": rid, "tokens": t[:p], "want": list(range(p)) if want_all else [p - 1]}
                   for rid, (t, p) in batch.items()]
        ends = [rid for rid, (t, p) in batch.items() if p == len(t)]
        steps.append({"step": len(steps), "entries": entries, "end": ends})
        live = [rid for rid in batch if rid not in ends]
        while live:
            entries, ends = [], []
            for rid in live:
                t = batch[rid][0]
                entries.append({"id": rid, "tokens": [t[fed[rid]]], "want": [0]})
                fed[rid] += 1
                if fed[rid] == len(t):
                    ends.append(rid)
            steps.append({"step": len(steps), "entries": entries, "end": ends})
            live = [r for r in live if r not in ends]
    return steps, peak


def wanted_places(steps):
    """For every step that wants something: [(id, absolute position), ...] in output order."""
    pos, out = {}, {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            rows += [(e["id"], base + w) for w in e["want"]]
            pos[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
        if rows:
            out[s["step"]] = rows
    return out


def run_in_process(engine, steps):
    """{(id, position): float64 logits} through Engine.step_chunked."""
    from hilbert_pruned_8b_b200.engine.batch import StepEntry
    seqs, got = {}, {}
    places = wanted_places(steps)
    for s in steps:
        entries = []
        for e in s["entries"]:
            if e["id"] not in seqs:
                seqs[e["id"]] = engine.open_sequence()
            entries.append(StepEntry(seqs[e["id"]], e["tokens"], e["want"]))
        logits = engine.step_chunked(entries)
        if logits is not None:
            lg = logits.detach().cpu().to(torch.float64)
            for row, key in enumerate(places[s["step"]]):
                got[key] = lg[row].clone()
        for rid in s["end"]:
            engine.close_sequence(seqs.pop(rid))
    assert not seqs
    return got


def run_program(model_dir, dtype, steps, max_tokens, out_dir, vocab, env=None, timeout=600):
    """{(id, position): float64 logits} through bin/trace_run, one step at a time."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == f"done {s['step']}", f"trace_run answered {line!r} to step {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    got = {}
    for step_no, rows in wanted_places(steps).items():
        a = np.fromfile(os.path.join(out_dir, f"{step_no}.f32"), dtype="<f4")
        assert a.size == len(rows) * vocab, f"step {step_no}: {a.size} floats for {len(rows)} places"
        a = torch.from_numpy(a.reshape(len(rows), vocab).astype(np.float64))
        for row, key in enumerate(rows):
            got[key] = a[row]
    return got


def plain_logits(plain, requests):
    """{(id, position): float64 logits} of whole sequences through the plain implementation."""
    ref = {}
    for rid, toks in requests.items():
        lg = plain.logits(toks)
        for p in range(len(toks)):
            ref[(rid, p)] = lg[p]
    return ref


# Tolerances (fixed; a failure means a fault, not a tolerance to widen).
#  float32: |d| <= 1e-4 * max(1, |ref|), the reference's own parity bound
#           (cleanroom-transformer/tools/parity.py:171-190).
#  bfloat16: max|d| <= 0.02 * max|ref| per position against the plain model that rounds
#           at the same places; the reference accepts 0.05 * scale for its bf16 GPU path
#           (cleanroom-transformer/src/cuda_backend.cu:1386).
def compare(got, ref, dtype, what=""):
    assert got, "nothing was compared"
    worst, worst_key = 0.0, None
    for key, g in got.items():
        r = ref[key]
        assert torch.isfinite(g).all(), f"{what}: non-finite logits at {key}"
        if dtype == "float32":
            err = ((g - r).abs() / torch.clamp(r.abs(), min=1.0)).max().item()
            bound = 1e-4
        else:
            err = (g - r).abs().max().item() / max(1e-3, r.abs().max().item())
            bound = 0.02
        if err > worst:
            worst, worst_key = err, key
        assert err <= bound, f"{what}: {dtype} logits differ at request {key[0]} position {key[1]}: {err:.3e} > {bound}"
    return worst, worst_key
