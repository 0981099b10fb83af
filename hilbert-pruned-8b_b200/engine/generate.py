"""The generation loop above the step function.

Requests (token-id prompts) are served in batches that start together: a batch's prompts
run in one step (cut into several if they exceed the step capacity), then every live
sequence gets one token per step.  A sequence ends at a stop token, at its token budget or
when the context is full; it then leaves the batch and its cache pages and slot are given
back at once.  No request joins a running batch; when the batch is empty the next one
starts, reusing the slots.  The reference has no generation at all
(cleanroom-transformer/README.md:7-10): the loop, its admission rule and its stopping rules
are this library's own.

Admission: a batch takes the next requests in order while their worst-case page needs
(prompt plus token budget, rounded up to pages) fit the cache and the batch size limit,
so a running batch can never run out of cache.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from ..cache.manager import PAGE_TOKENS, pages_for
from ..sampling.sampler import SamplingParams
from .batch import StepEntry


@dataclass
class GenerationRequest:
    prompt: Sequence[int]
    max_new_tokens: int = 16
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_token_ids: Optional[Sequence[int]] = None   # None: the model's own (eos_token_id)
    request_id: Optional[int] = None                 # None: position in the call


@dataclass
class GenerationResult:
    request_id: int
    tokens: List[int]
    finish_reason: str          # "stop" | "length" | "context"
    prompt_tokens: int


@dataclass
class GenerationStats:
    batches: int = 0
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_steps: int = 0
    decode_seconds: float = 0.0


def plan_batch(costs: Sequence[int], pages_free: int, max_batch: int) -> int:
    """How many of the next requests (page costs in order) start together.  At least one
    request is taken if it fits at all; a request that can never fit raises."""
    n, used = 0, 0
    for c in costs:
        if n >= max_batch or used + c > pages_free:
            break
        used += c
        n += 1
    if n == 0 and costs:
        raise ValueError(f"generate: a request needs {costs[0]} cache pages of {PAGE_TOKENS} tokens, "
                         f"only {pages_free} exist")
    return n


def finish_reason(token: int, produced: int, budget: int, length: int, context: int,
                  stop_ids: Sequence[int]) -> Optional[str]:
    """Why a sequence ends after producing ``token`` (None: it goes on).  ``length`` is the
    number of tokens its cache holds once the new token is fed."""
    if token in stop_ids:
        return "stop"
    if produced >= budget:
        return "length"
    if length + 1 > context:
        return "context"
    return None


class Generator:
    """Drives ``engine`` (anything with open_sequence/close_sequence/step and a cache) and
    ``sampler`` (``sample(logits, temperatures, seeds, request_ids, steps) -> tokens``)."""

    def __init__(self, engine, sampler, max_batch: int = 64, synchronize=None):
        self.engine = engine
        self.sampler = sampler
        self.max_batch = max_batch
        self.stats = GenerationStats()
        self._sync = synchronize or (lambda: None)

    # a request may use the whole context: prompt + budget tokens, the last one never fed
    def _cost(self, req: GenerationRequest) -> int:
        return pages_for(min(len(req.prompt) + req.max_new_tokens, self._context()))

    def _context(self) -> int:
        """The most tokens a request's sequence may hold: the engine's limit for one sequence
        (and the checkpoint's stated maximum position), not the size of the page pool, which
        bounds what a whole batch holds and is the admission rule's business."""
        limit = getattr(self.engine, "generation_limit", None)
        return int(limit) if limit else self.engine.cache.tokens_capacity()

    def generate(self, requests: Sequence[GenerationRequest]) -> List[GenerationResult]:
        reqs = list(requests)
        for i, r in enumerate(reqs):
            if len(r.prompt) == 0:
                raise ValueError(f"generate: request {i} has an empty prompt")
            if len(r.prompt) > self._context():
                raise ValueError(f"generate: request {i} has {len(r.prompt)} prompt tokens, context is {self._context()}")
            if r.max_new_tokens < 0:
                raise ValueError(f"generate: request {i} has a negative token budget")
        results: List[Optional[GenerationResult]] = [None] * len(reqs)
        nxt = 0
        while nxt < len(reqs):
            free = min(self.engine.cache.pages_free()) if self.engine.cache.groups else 1 << 30
            n = plan_batch([self._cost(r) for r in reqs[nxt:nxt + self.max_batch]], free, self.max_batch)
            self._run_batch(reqs, list(range(nxt, nxt + n)), results)
            nxt += n
        return [r for r in results if r is not None]

    def _run_batch(self, reqs, idxs: List[int], results) -> None:
        eng = self.engine
        self.stats.batches += 1
        live: Dict[int, dict] = {}
        for i in idxs:
            r = reqs[i]
            rid = r.request_id if r.request_id is not None else i
            stop = list(r.stop_token_ids) if r.stop_token_ids is not None else list(getattr(eng, "stop_token_ids", []))
            if r.max_new_tokens == 0:
                results[i] = GenerationResult(rid, [], "length", len(r.prompt))
                continue
            live[i] = {"req": r, "rid": rid, "stop": stop, "seq": eng.open_sequence(), "out": [], "next": None}
        if not live:
            return
        try:
            # all prompts in one step; each sequence wants the logits of its last prompt token
            self._sync()
            t0 = time.perf_counter()
            order = list(live)
            entries = [StepEntry(live[i]["seq"], list(live[i]["req"].prompt), [len(live[i]["req"].prompt) - 1])
                       for i in order]
            logits = eng.step_chunked(entries) if hasattr(eng, "step_chunked") else eng.step(entries)
            toks = self._sample(logits, [live[i] for i in order], step_no=0)
            if hasattr(eng, "check_status"):
                eng.check_status()              # what the sampler noted (non-finite logits); the tokens were read anyway
            self._sync()
            self.stats.prefill_seconds += time.perf_counter() - t0
            self.stats.prefill_tokens += sum(len(live[i]["req"].prompt) for i in order)
            self._take(order, toks, live, results)
            self.decode(live, results, first_step=1)
        finally:
            for st in live.values():
                if st["seq"].open:
                    eng.close_sequence(st["seq"])

    def decode(self, live: Dict[int, dict], results, first_step: int = 1) -> None:
        """The decode phase: one token per live sequence per step until none is live.  ``live``
        maps a result index to a state with ``req``, ``rid``, ``stop``, ``seq`` (whose cache
        holds everything but the token in ``next``) and ``out``.  Every step copies the batch's
        metadata to the device and the sampled tokens back.

        With an engine that takes a step's tokens from the device (``takes_device_tokens``) the
        loop runs one step ahead: step k+1 is launched on the tokens step k left on the device
        before the host has read them, so the host's work hides behind the device's.  What
        the host does not know yet is whether a sequence stopped on a stop token at step k;
        such a sequence has then run one step for nothing, its result is not affected.  A step
        is only launched ahead when the same sequences take part as in the step before
        (nobody ends on its budget or at the context's end)."""
        eng = self.engine
        step_no = first_step
        ahead = bool(getattr(eng, "takes_device_tokens", False))
        flying = None          # a step whose sampled tokens the host has not read yet
        while live or flying is not None:
            t0 = time.perf_counter()
            if flying is not None and self._same_batch_goes_on(flying, live):
                order = flying["order"]
                entries = [StepEntry(live[i]["seq"], [0], [0]) for i in order]
                nxt = self._step_and_sample(entries, order, live, step_no, flying["tokens"])
                self._land(flying, live, results)
                flying = nxt
            else:
                if flying is not None:
                    self._land(flying, live, results)
                    flying = None
                if not live:
                    self.stats.decode_seconds += time.perf_counter() - t0
                    break
                order = list(live)
                entries = [StepEntry(live[i]["seq"], [live[i]["next"]], [0]) for i in order]
                flying = self._step_and_sample(entries, order, live, step_no, None)
                if not ahead or not flying["on_device"]:
                    self._land(flying, live, results)
                    flying = None
            self.stats.decode_steps += 1
            self.stats.decode_seconds += time.perf_counter() - t0
            step_no += 1

    def _step_and_sample(self, entries, order, live, step_no: int, device_tokens) -> dict:
        """One decode step and its sampling.  When every sequence of the step is greedy and the
        engine can take the largest logit itself (``samples_greedy``), that is part of the step
        (of its captured graph), not a launch of its own behind it."""
        eng = self.engine
        states = [live[i] for i in order]
        kw = {} if device_tokens is None else {"device_tokens": device_tokens}
        if getattr(eng, "samples_greedy", False) and all(s["req"].sampling.temperature == 0.0 for s in states):
            eng.step(entries, greedy=True, **kw)
            return self._launch_sampling(None, order, live, step_no, eng.greedy_tokens)
        return self._launch_sampling(eng.step(entries, **kw), order, live, step_no)

    def _launch_sampling(self, logits, order, live, step_no: int, toks=None) -> dict:
        """Samples a step's tokens (unless the step took them itself: ``toks``) and starts their
        copy to the host, together with the device status words if the engine has some; the
        record of a step whose tokens have not been read."""
        states = [live[i] for i in order]
        if toks is None:
            toks = self.sampler.sample(logits, [s["req"].sampling.temperature for s in states],
                                       [s["req"].sampling.seed for s in states], [s["rid"] for s in states],
                                       [step_no] * len(states))
        # the sequences' lengths as of this step: a later step may have grown them when this is read
        rec = {"order": order, "tokens": toks, "on_device": False, "host": None, "event": None, "status": None,
               "lengths": {i: live[i]["seq"].length for i in order}}
        if hasattr(toks, "is_cuda"):                   # a tensor: the next step can take it as it is
            import torch
            if toks.is_cuda:
                n = len(order)
                status = self.engine.status_tensor() if hasattr(self.engine, "status_tensor") else None
                words = 0 if status is None else status.numel()
                host = self._host_tokens(n + words)
                host[:n].copy_(toks, non_blocking=True)
                if words:
                    # what the kernels noted up to and including this step's sampling, read when
                    # the tokens are read: no wait of its own
                    host[n:].copy_(status, non_blocking=True)
                    rec["status"] = host[n:]
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(toks.device))
                rec.update(on_device=True, host=host[:n], event=ev)
            else:
                rec.update(on_device=True, host=toks.clone())
        return rec

    def _host_tokens(self, n: int):
        """One of two pinned buffers in turn (a step in flight and the one before it)."""
        import torch
        bufs = getattr(self, "_token_buffers", None)
        if bufs is None or bufs[0].numel() < n:
            bufs = self._token_buffers = [torch.empty(max(n, 72), dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._token_turn = 0
        self._token_turn ^= 1
        return bufs[self._token_turn][:n]

    def _same_batch_goes_on(self, flying: dict, live: Dict[int, dict]) -> bool:
        """Whether the step after ``flying`` can be launched before ``flying``'s tokens are read:
        every sequence of it is still live and will be, whatever token it got, unless that is
        a stop token."""
        order = flying["order"]
        if len(order) != len(live):
            return False
        context = self._context()
        for i in order:
            st = live.get(i)
            if st is None:
                return False
            if len(st["out"]) + 1 >= st["req"].max_new_tokens or st["seq"].length + 1 > context:
                return False
        return True

    def _land(self, flying: dict, live: Dict[int, dict], results) -> None:
        """Reads a step's tokens and books them (sequences that ended meanwhile are skipped)."""
        toks = flying["tokens"]
        if flying["on_device"]:
            if flying["event"] is not None:
                flying["event"].synchronize()
            if flying.get("status") is not None:
                words = flying["status"].tolist()
                if any(words):
                    # a kernel noted a fault (a wait that ran out, non-finite logits, a bad page or
                    # token number): the tokens are not to be trusted, the call ends here
                    self.engine.raise_on_status(words)
            toks = flying["host"].tolist()
        else:
            toks = [int(t) for t in (toks.tolist() if hasattr(toks, "tolist") else toks)]
        pairs = [(i, t) for i, t in zip(flying["order"], toks) if i in live]
        self.stats.decode_tokens += len(pairs)
        self._take([i for i, _ in pairs], [t for _, t in pairs], live, results, flying["lengths"])

    def _sample(self, logits, states, step_no: int) -> List[int]:
        toks = self.sampler.sample(logits, [s["req"].sampling.temperature for s in states],
                                   [s["req"].sampling.seed for s in states], [s["rid"] for s in states],
                                   [step_no] * len(states))
        return [int(t) for t in (toks.tolist() if hasattr(toks, "tolist") else toks)]

    def _take(self, order, toks, live, results, lengths=None) -> None:
        """Books each sequence's new token and retires the sequences that end with it.
        ``lengths``: the sequences' lengths when the tokens were sampled (default: now)."""
        for i, tok in zip(order, toks):
            st = live[i]
            st["out"].append(tok)
            st["next"] = tok
            length = lengths[i] if lengths is not None else st["seq"].length
            why = finish_reason(tok, len(st["out"]), st["req"].max_new_tokens, length, self._context(), st["stop"])
            if why is not None:
                results[i] = GenerationResult(st["rid"], st["out"], why, len(st["req"].prompt))
                self.engine.close_sequence(st["seq"])
                del live[i]
