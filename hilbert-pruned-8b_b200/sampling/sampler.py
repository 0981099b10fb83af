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
    """Device-side sampler over ``[rows, vocab]`` float32 logits.  The per-row parameters of a
    temperature step travel in one copy from a small ring of pinned host buffers (a buffer is
    written again only after the copy that read it has finished), so a step allocates nothing."""

    RING = 4

    def __init__(self, ops, device, max_rows: int = 1024):
        self.ops = ops
        self.device = torch.device(device)
        self.max_rows = 0
        self._turn = 0
        self._grow(max_rows)

    def _grow(self, n: int) -> None:
        if n <= self.max_rows:
            return
        self.max_rows = n
        pin = self.device.type == "cuda"
        self._out = torch.empty(n, dtype=torch.int32, device=self.device)
        # rows of the parameter block: temperatures (float32, at the row's start), seeds, requests, steps
        self._dev = torch.empty((4, n), dtype=torch.int64, device=self.device)
        self._host = [torch.zeros((4, n), dtype=torch.int64, pin_memory=pin) for _ in range(self.RING)]
        self._host_np = [h.numpy() for h in self._host]
        self._events = [None] * self.RING

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
        import numpy as np
        n = logits.shape[0]
        self._grow(n)
        out = self._out[:n]
        if all(t == 0.0 for t in temperatures):
            self.ops.argmax(logits, out)
            return out
        r = self._turn
        self._turn = (r + 1) % self.RING
        if self._events[r] is not None:
            self._events[r].synchronize()
        a = self._host_np[r]
        a[0].view(np.float32)[:n] = np.asarray(temperatures, dtype=np.float32)      # the row's first n floats
        a[1, :n] = [s - (1 << 64) if s >= (1 << 63) else s for s in seeds]
        a[2, :n] = request_ids
        a[3, :n] = steps
        self._dev[:, :n].copy_(self._host[r][:, :n], non_blocking=True)
        if self.device.type == "cuda":
            ev = self._events[r] or torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._events[r] = ev
        temp = self._dev[0].view(torch.float32)[:n]
        self.ops.sample(logits, temp, self._dev[1, :n], self._dev[2, :n], self._dev[3, :n], out)
        return out
