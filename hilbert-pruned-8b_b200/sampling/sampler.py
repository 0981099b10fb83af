"""Greedy and temperature sampling.

The reference generates nothing and so samples nothing; what it reads out is the logits of
a few option ids with a softmax over them in double precision
(cleanroom-transformer/src/engine.c:8-14), kept here as ``option_scores``.  Greedy takes the
largest logit (lowest index on ties).  Temperature sampling draws from
``softmax(logits / T)`` by inverse CDF with a uniform number derived from
``(seed, request id, step)``, so that a request's tokens do not depend on which other
requests share its batch.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence

import torch

_MASK = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_from(seed: int, request: int, step: int) -> float:
    """The 24-bit uniform in [0, 1) that the device sampler uses for this draw."""
    z = ((seed & _MASK) * 0x9E3779B97F4A7C15 + (request & _MASK) * 0xBF58476D1CE4E5B9
         + (step & _MASK) * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & _MASK
    z = _mix64(_mix64(z))
    return (z >> 40) / 16777216.0


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0   # 0: greedy
    seed: int = 0

    def __post_init__(self):
        if not (self.temperature >= 0.0) or math.isinf(self.temperature):
            raise ValueError("sampling: temperature must be a finite number >= 0")


def option_scores(logits: Sequence[float]) -> List[float]:
    """Softmax over a handful of option logits in double precision (engine.c:8-14)."""
    m = max(logits)
    e = [math.exp(float(x) - m) for x in logits]
    s = sum(e)
    return [x / s for x in e]


class Sampler:
    """Device-side sampler over ``[rows, vocab]`` float32 logits."""

    def __init__(self, ops, device, max_rows: int = 1024):
        self.ops = ops
        self.device = torch.device(device)
        self.max_rows = max_rows
        self._out = torch.empty(max_rows, dtype=torch.int32, device=self.device)

    def _grow(self, n: int) -> None:
        if n > self.max_rows:
            self.max_rows = n
            self._out = torch.empty(n, dtype=torch.int32, device=self.device)

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        n = logits.shape[0]
        self._grow(n)
        out = self._out[:n]
        self.ops.argmax(logits, out)
        return out

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], seeds: Sequence[int],
               request_ids: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """One token per row; rows with temperature 0 are greedy.  Returns int32 on the device
        (scratch: overwritten by the next call)."""
        n = logits.shape[0]
        self._grow(n)
        out = self._out[:n]
        if all(t == 0.0 for t in temperatures):
            self.ops.argmax(logits, out)
            return out
        temp = torch.tensor(list(temperatures), dtype=torch.float32).to(self.device, non_blocking=True)
        meta = torch.tensor([[s - (1 << 64) if s >= (1 << 63) else s for s in seeds], list(request_ids), list(steps)],
                            dtype=torch.int64).to(self.device, non_blocking=True)
        self.ops.sample(logits, temp, meta[0], meta[1], meta[2], out)
        return out
