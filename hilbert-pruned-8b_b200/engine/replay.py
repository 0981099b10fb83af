"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing.  It drives the same engine, step function, cache and kernels that
generation uses.  Its ancestor in the reference is the ``logits`` command with ``--split``
(cleanroom-transformer/src/main.c:351-387).

Input: one JSON object per line,
``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}``.
For a step that wants something, ``<out>/<step>.f32`` receives the logits at the wanted
places as little-endian float32 ``[wanted, vocab]``, in the order of the entries and of
``want``.  After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

from .batch import StepEntry


def replay(engine, lines: IO[str], out_dir: str, reply: IO[str]) -> int:
    os.makedirs(out_dir, exist_ok=True)
    seqs: Dict[str, object] = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        obj = json.loads(line)
        step_no = obj["step"]
        entries = []
        for e in obj.get("entries", []):
            key = str(e["id"])
            if key not in seqs:
                seqs[key] = engine.open_sequence()
            entries.append(StepEntry(seqs[key], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = engine.step_chunked(entries)
            if logits is not None:
                a = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step_no}.f32.tmp")
                a.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step_no}.f32"))
        for key in obj.get("end", []):
            seq = seqs.pop(str(key), None)
            if seq is None:
                raise ValueError(f"trace: request {key} ends but was never started")
            engine.close_sequence(seq)
        reply.write(f"done {step_no}\n")
        reply.flush()
    return 0


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="Replay a token trace through the model and write logits.")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64); sizes the cache")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    if args.max_tokens < 1:
        ap.error("--max-tokens must be positive")
    from .step import Engine
    try:
        engine = Engine.from_folder(args.model, args.dtype, max_tokens=args.max_tokens, device=f"cuda:{args.device}")
        return replay(engine, sys.stdin, args.out, sys.stdout)
    except (ValueError, RuntimeError) as e:        # configuration, weights, a refused step, a fault a kernel noted
        print(f"error: {e}", file=sys.stderr)
        return 1
