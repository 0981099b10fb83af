"""The Python entry point: load a model folder (or draw random weights), generate, read logits.

The option names are the reference's where it has them: ``model`` (a folder), ``dtype``
(``bfloat16`` | ``float32``), ``max_tokens`` (the context the cache is sized for) and
``device`` (src/semif_phase1/cli.py:26-34; cleanroom-transformer/src/main.c:86-118).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .engine.batch import StepEntry
from .engine.generate import GenerationRequest, GenerationResult, Generator
from .engine.step import Engine
from .sampling.sampler import Sampler, SamplingParams, option_scores


class LLM:
    """A loaded model with its cache, sampler and generation loop."""

    def __init__(self, engine: Engine, max_batch: int = 64):
        self.engine = engine
        self.sampler = Sampler(engine.ctx.ops, engine.device)
        self.generator = Generator(engine, self.sampler, max_batch=max_batch,
                                   synchronize=lambda: torch.cuda.synchronize(engine.device))

    @classmethod
    def load(cls, model: str, dtype: str = "bfloat16", max_tokens: int = 4096, device: int = 0,
             max_batch: int = 64, **kw) -> "LLM":
        """Further keywords go to the engine: ``max_sequence_tokens`` (the most one sequence may
        hold; default: the whole cache), ``max_step_tokens``, ``max_sequences``, ``strict_weights``."""
        return cls(Engine.from_folder(model, dtype, max_tokens=max_tokens, device=f"cuda:{device}", **kw), max_batch)

    @classmethod
    def random(cls, config, seed: int = 0, dtype: str = "bfloat16", max_tokens: int = 4096, device: int = 0,
               max_batch: int = 64, **kw) -> "LLM":
        return cls(Engine.from_random(config, seed, dtype, max_tokens=max_tokens, device=f"cuda:{device}", **kw),
                   max_batch)

    @property
    def config(self):
        return self.engine.config

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0,
                 seed: int = 0, stop_token_ids: Optional[Sequence[int]] = None) -> List[GenerationResult]:
        """Generates for token-id prompts; results come in the order of the prompts.  Request i
        draws with ``(seed, i)``, so a result does not depend on what else is in the call."""
        params = SamplingParams(temperature=temperature, seed=seed)
        reqs = [GenerationRequest(list(p), max_new_tokens, params, stop_token_ids, i) for i, p in enumerate(prompts)]
        return self.generator.generate(reqs)

    def generate_requests(self, requests: Sequence[GenerationRequest]) -> List[GenerationResult]:
        return self.generator.generate(requests)

    def logits(self, tokens: Sequence[int], ids: Optional[Sequence[int]] = None, split: int = 0) -> torch.Tensor:
        """Logits at the last position of ``tokens`` (all of the vocabulary, or the given ids),
        as the reference's ``logits`` command reads them.  ``split`` N does what the reference's
        ``--split N`` does (cleanroom-transformer/src/main.c:363-370): the first N tokens in a
        step of their own, a snapshot, the rest, a restore, and the rest once more; the logits
        of that second run are returned, so a rewind that left anything behind would show."""
        eng = self.engine
        seq = eng.open_sequence()
        try:
            toks = [int(t) for t in tokens]
            if 0 < split < len(toks):
                eng.step_chunked([StepEntry(seq, toks[:split], [])])
                snap = eng.snapshot(seq)
                rest = toks[split:]
                eng.step_chunked([StepEntry(seq, rest, [len(rest) - 1])])
                eng.restore(seq, snap)
                toks = rest
            out = eng.step_chunked([StepEntry(seq, toks, [len(toks) - 1])])[0].clone()
        finally:
            eng.close_sequence(seq)
        if ids is not None:
            for i in ids:
                if not 0 <= int(i) < eng.vocab_size:
                    raise ValueError(f"logits: readout id {int(i)} out of range")
            out = out[torch.tensor([int(i) for i in ids], dtype=torch.long, device=out.device)]
        return out

    def option_scores(self, tokens: Sequence[int], ids: Sequence[int]) -> List[float]:
        """Probabilities over a few option ids at the last position (engine.c:8-14)."""
        return option_scores(self.logits(tokens, ids).tolist())
