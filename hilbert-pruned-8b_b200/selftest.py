"""``selftest``: a tiny random model on the GPU, each way of cutting the work against the
others, as the reference's selftest does for its one sequence (full prefill vs prefix +
rest vs all but one + one token, cleanroom-transformer/src/cuda_backend.cu:1429-1441)."""
from __future__ import annotations

import sys

import torch


def selftest(device: int = 0) -> int:
    from .config import LlamaConfig
    from .engine.batch import StepEntry
    from .engine.step import Engine
    cfg = LlamaConfig.from_dict(dict(
        model_type="llama", hidden_size=96, num_hidden_layers=2, intermediate_size=208, vocab_size=320,
        num_attention_heads=6, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5, rope_theta=10000.0))
    gen = torch.Generator().manual_seed(7)
    toks = [int(t) for t in torch.randint(0, cfg.vocab_size, (96,), generator=gen)]
    ok = True
    for dtype, bound in (("float32", 1e-4), ("bfloat16", 3e-2)):
        eng = Engine.from_random(cfg, 1, dtype, max_tokens=256, device=f"cuda:{device}", fan_in_scale=1.0)
        a = eng.open_sequence()
        whole = eng.step([StepEntry(a, toks, list(range(len(toks))))]).clone()
        b = eng.open_sequence()
        eng.step([StepEntry(b, toks[:40], [])])
        rest = eng.step([StepEntry(b, toks[40:95], list(range(55)))]).clone()
        last = eng.step([StepEntry(b, toks[95:], [0])]).clone()
        eng.close_sequence(a), eng.close_sequence(b)
        scale = whole.abs().max().item()
        e1 = (rest - whole[40:95]).abs().max().item() / scale
        e2 = (last[0] - whole[95]).abs().max().item() / scale
        good = e1 <= bound and e2 <= bound
        ok = ok and good
        print(f"selftest {dtype}: prefix+rest {e1:.2e}, one token {e2:.2e} (bound {bound:g}) {'ok' if good else 'FAIL'}",
              file=sys.stderr)
    return 0 if ok else 1
