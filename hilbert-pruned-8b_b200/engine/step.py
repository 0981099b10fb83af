"""The step function: a batch of sequences, their next tokens, logits at the wanted places.

``Engine.step`` runs only the tokens it is given, as one packed batch, against the cache
that earlier steps left, and returns the logits at the wanted places.  The sequences of a
step may have any lengths and bring any number of tokens each: all prompts of a batch in
one step, then one token each, is the usual use, and a long prompt may be cut into several
steps.  It is the batched generalisation of the reference's
``forward(tokens, n, ids, n_ids, logits)`` on one sequence with a position counter
(cleanroom-transformer/src/transformer.h:347-364); the checks are the reference's
(cpu_backend.c:223-228).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence as Seq

import torch

from ..cache.manager import CacheManager, Sequence
from ..config.registry import load_config
from ..parts.base import BuildContext
from ..weights.loader import choose_prefix, folder_names, load_tensors
from .batch import DecodeMeta, StepBatch, StepEntry, build_step
from .model import DecoderModel
from .workspace import Workspace

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if dtype not in _DTYPES:
        raise ValueError(f"dtype {dtype!r} is not supported (bfloat16 or float32)")
    return _DTYPES[dtype]


class Engine:
    """A model on one GPU with its cache: the object every entry point drives."""

    def __init__(self, spec, dtype="bfloat16", max_tokens: int = 4096, device="cuda:0",
                 max_step_tokens: Optional[int] = None, max_sequences: Optional[int] = None,
                 max_sequence_tokens: Optional[int] = None):
        """``max_tokens`` sizes the cache (tokens all live sequences hold together, in pages of
        64); ``max_sequence_tokens`` is the most one sequence may hold (default: the whole
        cache, as the reference's ``--max-tokens`` is both: cleanroom-transformer/src/main.c:76,
        cpu_backend.c:223-228)."""
        from ..kernels import ops  # fails loudly without a GPU toolchain or a built library
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("engine: the model runs on a CUDA device only; there is no CPU path")
        self.dtype = parse_dtype(dtype)
        self.spec = spec
        self.max_tokens = int(max_tokens)
        self.max_step_tokens = int(max_step_tokens) if max_step_tokens else min(max(self.max_tokens, 64), 8192)
        torch.cuda.set_device(self.device)
        self.workspace = Workspace(self.device)
        self.ctx = BuildContext(device=self.device, dtype=self.dtype, ops=ops.Ops(self.device), workspace=self.workspace,
                                max_step_tokens=self.max_step_tokens)
        self.model = DecoderModel(spec, self.ctx)
        self.cache: Optional[CacheManager] = None
        self._max_sequences = max_sequences
        if max_sequence_tokens is not None and max_sequence_tokens < 1:
            raise ValueError("engine: max_sequence_tokens must be positive")
        self.max_sequence_tokens = max_sequence_tokens
        self.greedy_tokens: Optional[torch.Tensor] = None      # what step(..., greedy=True) left on the device
        # decode steps (one token per sequence) are captured in CUDA graphs, one per
        # (batch size, page-table width): a step is then one small copy and one graph launch
        self.use_graphs = True
        self._graphs: Dict[tuple, object] = {}
        self._decode_meta: Dict[tuple, DecodeMeta] = {}
        self.graph_replays = 0
        self.stop_token_ids = list(spec.stop_token_ids)
        self.vocab_size = spec.vocab_size

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", max_tokens: int = 4096, device="cuda:0",
                    strict_weights: bool = False, **kw) -> "Engine":
        """``strict_weights``: tensors in the folder that no part of the model reads are an error
        (default: ignored, as the reference ignores what it does not bind)."""
        config = load_config(model_dir)
        eng = cls(config.model_spec(), dtype, max_tokens, device, **kw)
        eng.config = config
        names = folder_names(model_dir)
        prefix = choose_prefix(names, eng.spec.weight_prefixes, eng.model.first_weight_name())
        table = eng.model.weight_table(prefix)
        tensors = load_tensors(model_dir, table, eng.dtype, eng.device, strict=strict_weights)
        eng.model.bind(tensors, prefix)
        eng._make_cache()
        return eng

    @classmethod
    def from_random(cls, config, seed: int, dtype="bfloat16", max_tokens: int = 4096, device="cuda:0",
                    std: float = 0.02, norm_std: float = 0.0, fan_in_scale=None, stored_dtype=torch.bfloat16,
                    **kw) -> "Engine":
        """Random weights drawn on the device (no folder is written).  The values are a function
        of (seed, tensor name, element): the model that ``write_random_model(folder, config, seed,
        ...)`` writes from the CPU with the same arguments, bit for bit; ``stored_dtype`` is that
        folder's dtype, and a 32-bit engine widens it exactly, as it does when it loads."""
        from ..weights.random_init import random_tensors
        eng = cls(config.model_spec(), dtype, max_tokens, device, **kw)
        eng.config = config
        table = eng.model.weight_table()
        tensors = random_tensors(table, seed, eng.device, std, norm_std, stored_dtype, fan_in_scale, ops=eng.ctx.ops)
        if eng.dtype == torch.float32:
            tensors = {n: (t.to(torch.float32) if t.is_floating_point() else t) for n, t in tensors.items()}
        eng.model.bind(tensors)
        del tensors
        eng._make_cache()
        return eng

    def _make_cache(self) -> None:
        self.cache = CacheManager(self.model.cache_needs(), self.model.state_needs(), self.max_tokens, self.device,
                                  self.dtype, self._max_sequences)

    # ------------------------------------------------------------------ sequences
    def open_sequence(self) -> Sequence:
        return self.cache.open()

    def close_sequence(self, seq: Sequence) -> None:
        self.cache.close(seq)

    def snapshot(self, seq: Sequence):
        """Remembers where ``seq`` stands (``CacheManager.snapshot``)."""
        return self.cache.snapshot(seq)

    def restore(self, seq: Sequence, snapshot) -> None:
        """Rewinds ``seq`` to a snapshot of itself; the next step feeds the tokens that follow it."""
        self.cache.restore(seq, snapshot)

    # ------------------------------------------------------------------ limits
    @property
    def sequence_limit(self) -> int:
        """The most tokens one sequence may hold: what the step function enforces."""
        cap = self.cache.tokens_capacity()
        return cap if self.max_sequence_tokens is None else min(cap, self.max_sequence_tokens)

    @property
    def generation_limit(self) -> int:
        """Where the generation loop ends a request with ``"context"``: the sequence limit, and
        the longest sequence the checkpoint states it was made for (``max_position_embeddings``)
        if it states one.  The step function itself does not read that key, as the reference
        does not: given tokens may run past it."""
        lim = self.sequence_limit
        return lim if not self.spec.max_position else min(lim, int(self.spec.max_position))

    # ------------------------------------------------------------------ status
    def status_tensor(self) -> torch.Tensor:
        """The device status words the kernels note faults in (``Ops.status``)."""
        return self.ctx.ops.status

    def raise_on_status(self, words) -> None:
        self.ctx.ops.raise_on_status(words)

    def check_status(self) -> None:
        """Reads the status words (this waits for the device) and raises ``KernelError`` if a
        kernel noted a fault: a wait that ran out, non-finite logits given to a sampler, a page
        or token number out of range."""
        self.ctx.ops.check_errors()

    # ------------------------------------------------------------------ the step
    def check_entries(self, entries: List[StepEntry]) -> None:
        if not entries:
            raise ValueError("step: no sequences")
        total = 0
        seen = set()
        capacity = self.sequence_limit
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise ValueError("step: no tokens")
            if id(e.seq) in seen:
                raise ValueError(f"step: sequence {e.seq.seq_id} appears twice in one step")
            seen.add(id(e.seq))
            if not e.seq.open:
                raise ValueError(f"step: sequence {e.seq.seq_id} is closed")
            if e.seq.length + n > capacity:
                raise ValueError(f"step: {e.seq.length + n} tokens exceed context {capacity}")
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise ValueError(f"step: token {int(t)} out of range")
            total += n
        if total > self.max_step_tokens:
            raise ValueError(f"step: {total} tokens exceed the step capacity {self.max_step_tokens}")

    takes_device_tokens = True      # step(entries, device_tokens=...) exists
    samples_greedy = True           # step(entries, greedy=True) leaves the largest logits' indices in greedy_tokens

    def step(self, entries: List[StepEntry], device_tokens: Optional[torch.Tensor] = None,
             greedy: bool = False) -> Optional[torch.Tensor]:
        """Runs the entries' tokens; returns ``[wanted, vocab]`` float32 logits on the device,
        in the order of the entries and of each entry's ``want`` (None if nothing is wanted).
        The tensor is engine scratch: it is overwritten by the next step.  ``device_tokens``
        (int32 on the device, one per entry, each entry then brings one placeholder token)
        gives the tokens without the host knowing them: what a sampler just wrote.  ``greedy``:
        the step also takes the index of the largest logit of every wanted row (lowest index on
        ties) into ``self.greedy_tokens`` (int32 on the device, scratch as well); in a decode
        step that is part of the captured graph."""
        self.check_entries(entries)
        if device_tokens is not None and (device_tokens.dtype != torch.int32 or device_tokens.numel() != len(entries)
                                          or any(len(e.tokens) != 1 for e in entries)):
            raise ValueError("step: device tokens need one int32 token per entry and one placeholder token each")
        self.cache.reserve([(e.seq, e.seq.length + len(e.tokens)) for e in entries])
        self.greedy_tokens = None
        if self.use_graphs and self.model.graph_safe and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            logits, batch = self._decode_step(entries, device_tokens, greedy)
        else:
            batch = build_step(entries, self.cache, self.workspace, self.device)
            if device_tokens is not None:
                batch.tokens.copy_(device_tokens)
            logits = self.model.forward(batch, self.cache)
            if greedy and logits is not None:
                self.greedy_tokens = self._greedy(logits, batch.tag)
        for e, new_len in zip(entries, batch.host_len):
            self.cache.commit(e.seq, new_len)
        return logits

    def _greedy(self, logits: torch.Tensor, tag: str) -> torch.Tensor:
        n = logits.shape[0]
        cap = max(n, 64) if not tag else n
        out = self.workspace.buffer("step.greedy" + tag, (cap,), torch.int32)[:n]
        self.ctx.ops.argmax(logits, out)
        return out

    def _decode_step(self, entries: List[StepEntry], device_tokens: Optional[torch.Tensor] = None, greedy: bool = False):
        """A decode step through a captured graph.  The first step of a shape runs eagerly
        (it also allocates every buffer), the second captures, later ones replay."""
        from ..cache.manager import pages_for
        B = len(entries)
        need = max(pages_for(e.seq.length + 1) for e in entries)
        width = 1 << (need - 1).bit_length()
        meta_key = (B, width)
        meta = self._decode_meta.get(meta_key)
        if meta is None:
            meta = self._decode_meta[meta_key] = DecodeMeta(B, width, self.cache, self.workspace, self.device,
                                                            f"step.meta.decode.{B}.{width}")
        batch = meta.fill(entries)          # max_len is the bucket's: kernel launch shapes depend on it only
        if device_tokens is not None:
            batch.tokens.copy_(device_tokens)       # after the metadata copy, before the graph that reads it
        batch.tag = f".decode.{B}"
        key = (B, width, bool(greedy))

        def run():
            logits = self.model.forward(batch, self.cache)
            return logits, (self._greedy(logits, batch.tag) if greedy else None)

        state = self._graphs.get(key)
        if state is None:
            self._graphs[key] = "warm"
            logits, self.greedy_tokens = run()
            return logits, batch
        if state == "warm":
            ops = self.ctx.ops
            torch.cuda.synchronize(self.device)
            before = ops.launches
            graph = torch.cuda.CUDAGraph()
            self.workspace.capturing = True
            try:
                with torch.cuda.graph(graph):
                    logits, toks = run()
            finally:
                self.workspace.capturing = False
            state = (graph, logits, toks, ops.launches - before)
            ops.launches = before
            self._graphs[key] = state
        graph, logits, toks, launches = state
        graph.replay()
        self.greedy_tokens = toks
        self.ctx.ops.launches += launches
        self.graph_replays += 1
        return logits, batch

    def step_chunked(self, entries: List[StepEntry]) -> Optional[torch.Tensor]:
        """``step`` for any number of tokens: a step larger than the step capacity is cut into
        several, each sequence's tokens staying in order.  The logits come back in the order
        of the entries and of each entry's ``want``, in a tensor of their own (scratch of the
        engine when the step was not cut).  Everything is checked before the first part runs
        (token ids, each sequence's limit, the pages the whole call needs), so a call that is
        refused has fed nothing.  At the end the device status words are read: this waits for
        the device, and raises ``KernelError`` if a kernel noted a fault."""
        total = sum(len(e.tokens) for e in entries)
        if total <= self.max_step_tokens:
            logits = self.step(entries)
            self.check_status()
            return logits
        self._check_whole_call(entries)
        # row of each wanted place in the result
        rows, r = [], 0
        for e in entries:
            rows.append({int(w): r + k for k, w in enumerate(e.want)})
            if len(rows[-1]) != len(e.want):
                raise ValueError("step: a place is wanted twice")
            for w in rows[-1]:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"step: wanted place {w} is outside the {len(e.tokens)} tokens of this step")
            r += len(e.want)
        result = torch.empty((r, self.vocab_size), dtype=torch.float32, device=self.device) if r else None
        done = [0] * len(entries)
        while any(done[i] < len(e.tokens) for i, e in enumerate(entries)):
            room = self.max_step_tokens
            sub: List[StepEntry] = []
            dest: List[int] = []
            for i, e in enumerate(entries):
                left = len(e.tokens) - done[i]
                if left == 0 or room == 0:
                    continue
                n = min(left, room)
                lo = done[i]
                wants = sorted(w for w in rows[i] if lo <= w < lo + n)
                sub.append(StepEntry(e.seq, e.tokens[lo:lo + n], [w - lo for w in wants]))
                dest.extend(rows[i][w] for w in wants)
                done[i] += n
                room -= n
            logits = self.step(sub)
            if dest:
                result.index_copy_(0, torch.tensor(dest, dtype=torch.long, device=self.device), logits)
        self.check_status()
        return result

    def _check_whole_call(self, entries: List[StepEntry]) -> None:
        """The checks of ``check_entries`` over all tokens of a call that will be cut into several
        steps, and the pages the whole call needs against the pages that are free."""
        if not entries:
            raise ValueError("step: no sequences")
        seen = set()
        limit = self.sequence_limit
        for e in entries:
            if len(e.tokens) == 0:
                raise ValueError("step: no tokens")
            if id(e.seq) in seen:
                raise ValueError(f"step: sequence {e.seq.seq_id} appears twice in one step")
            seen.add(id(e.seq))
            if not e.seq.open:
                raise ValueError(f"step: sequence {e.seq.seq_id} is closed")
            if e.seq.length + len(e.tokens) > limit:
                raise ValueError(f"step: {e.seq.length + len(e.tokens)} tokens exceed context {limit}")
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise ValueError(f"step: token {int(t)} out of range")
        self.cache.check_room([(e.seq, e.seq.length + len(e.tokens)) for e in entries])

    # ------------------------------------------------------------------ accounting
    def decode_step_bytes(self, live_lengths: Seq[int]) -> int:
        """Bytes a decode step has to read: every weight it uses once and the cache of the
        live sequences."""
        kv = sum(int(l) for l in live_lengths) * self.cache.bytes_per_token()
        return self.model.step_weight_bytes() + kv
