"""Command line, in the reference's manner: ``COMMAND --model DIR [options]`` with its option
names where it has them (cleanroom-transformer/src/main.c:11-50,66-129: ``--model``,
``--device N``, ``--max-tokens N``, ``logits --tokens "1 2 3" --ids "4 5" [--split N]``,
``shapes``; src/semif_phase1/cli.py:16-37: ``--dtype``, ``--input`` rows as JSON lines,
``--output`` a new file of JSON lines).

commands:
  generate  tokens for prompts   --input rows.jsonl --output results.jsonl | --tokens "1 2 3"
                                 [--max-new-tokens N] [--temperature T] [--seed S] [--stop-ids "7 9"] [--batch N]
  logits    raw logits           --tokens "1 2 3" [--ids "4 5"] [--split N]   (N: prefix, snapshot, rest, restore, rest)
  shapes    the weight table as JSON (config only, no GPU)
  random    write a model folder --config config.json --output DIR [--seed S] [--std X] [--norm-std X]
  selftest  a tiny random model: token by token against whole prompts, on the GPU
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def _ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit("--tokens, --ids and --stop-ids need lists of integers")


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="hilbert-b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=("generate", "logits", "shapes", "random", "selftest"))
    ap.add_argument("--model", help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                    help="model precision; changing it can change the tokens")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--max-tokens", type=int, default=4096, help="context: tokens the cache holds")
    ap.add_argument("--max-sequence-tokens", type=int, default=None,
                    help="most tokens of one sequence (default: --max-tokens; generation also stops at the "
                         "model's max_position_embeddings)")
    ap.add_argument("--strict-weights", action="store_true",
                    help="tensors in the folder that the model does not read are an error")
    ap.add_argument("--input", help="JSON lines: {\"id\":..., \"tokens\":[...], \"max_new_tokens\":..., \"temperature\":..., \"seed\":...}")
    ap.add_argument("--output", help="JSON lines, one per row; must not exist yet")
    ap.add_argument("--tokens", help="one prompt as token ids")
    ap.add_argument("--ids", help="vocabulary ids to read out")
    ap.add_argument("--split", type=int, default=0)
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--stop-ids", help="stop token ids (default: the model's eos_token_id)")
    ap.add_argument("--batch", type=int, default=64, help="most requests that start together")
    ap.add_argument("--config", help="random: a config.json to take the sizes from")
    ap.add_argument("--std", type=float, default=0.02)
    ap.add_argument("--norm-std", type=float, default=0.0)
    return ap


def main(argv=None) -> int:
    ap = _parser()
    a = ap.parse_args(argv)
    if a.max_tokens < 1:
        ap.error("--max-tokens must be positive")
    if a.command == "shapes":
        from .config import load_config
        from .engine.model import weight_table
        if not a.model:
            ap.error("shapes needs --model")
        table = weight_table(load_config(a.model).model_spec())
        print(json.dumps({n: {"shape": list(p.shape), "kind": p.kind} for n, p in table.items()}, indent=1))
        return 0
    if a.command == "random":
        from .config import config_class_for
        from .weights import write_random_model
        if not a.config or not a.output:
            ap.error("random needs --config and --output")
        with open(a.config) as f:
            root = json.load(f)
        write_random_model(a.output, config_class_for(root).from_dict(root), a.seed, std=a.std, norm_std=a.norm_std)
        return 0
    from .api import LLM
    from .engine.generate import GenerationRequest
    from .sampling import SamplingParams
    if a.command == "selftest":
        from .selftest import selftest
        return selftest(a.device)
    if not a.model:
        ap.error(f"{a.command} needs --model")
    if a.command == "logits":
        if not a.tokens:
            ap.error("logits needs --tokens")
        llm = LLM.load(a.model, a.dtype, a.max_tokens, a.device, max_sequence_tokens=a.max_sequence_tokens,
                       strict_weights=a.strict_weights)
        out = llm.logits(_ids(a.tokens), _ids(a.ids) if a.ids else None, a.split)
        print(" ".join(repr(float(x)) for x in out.tolist()))
        return 0
    # generate
    stop = _ids(a.stop_ids) if a.stop_ids is not None else None
    if a.tokens:
        rows = [{"id": 0, "tokens": _ids(a.tokens)}]
    elif a.input:
        with open(a.input) as f:
            rows = [json.loads(line) for line in f if line.strip()]
        if not rows:
            ap.error("Input is empty")
    else:
        ap.error("generate needs --input or --tokens")
    dest = sys.stdout
    if a.output:
        try:
            dest = open(a.output, "x")
        except FileExistsError:
            ap.error("Output must be new")
    llm = LLM.load(a.model, a.dtype, a.max_tokens, a.device, max_batch=a.batch,
                   max_sequence_tokens=a.max_sequence_tokens, strict_weights=a.strict_weights)
    reqs = [GenerationRequest([int(t) for t in r["tokens"]], int(r.get("max_new_tokens", a.max_new_tokens)),
                              SamplingParams(float(r.get("temperature", a.temperature)), int(r.get("seed", a.seed))),
                              r.get("stop_token_ids", stop), i) for i, r in enumerate(rows)]
    results = llm.generate_requests(reqs)
    st = llm.generator.stats
    for row, res in zip(rows, results):
        dest.write(json.dumps({"id": row.get("id", res.request_id), "tokens": res.tokens,
                               "finish_reason": res.finish_reason, "prompt_tokens": res.prompt_tokens}) + "\n")
    if dest is not sys.stdout:
        dest.close()
    print(json.dumps({"batches": st.batches, "prefill_tokens": st.prefill_tokens, "prefill_s": round(st.prefill_seconds, 4),
                      "decode_tokens": st.decode_tokens, "decode_s": round(st.decode_seconds, 4)}), file=sys.stderr)
    return 0


def run(argv=None) -> int:
    """``main`` with the library's own errors printed as one line (the reference prints
    ``error: <message>`` and exits with 1)."""
    from .config import ConfigError
    from .weights import SafetensorsError, WeightError
    try:
        return main(argv)
    except (ConfigError, WeightError, SafetensorsError, ValueError, RuntimeError) as e:     # KernelError is a RuntimeError
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(run())
