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
                 max_step_tokens: Optional[int] = None, max_sequences: Optional[int] = None):
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

    # ------------------------------------------------------------------ the step
    def check_entries(self, entries: List[StepEntry]) -> None:
        if not entries:
            raise ValueError("step: no sequences")
        total = 0
        seen = set()
        capacity = self.cache.tokens_capacity()
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

    def step(self, entries: List[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the entries' tokens; returns ``[wanted, vocab]`` float32 logits on the device,
        in the order of the entries and of each entry's ``want`` (None if nothing is wanted).
        The tensor is engine scratch: it is overwritten by the next step.  ``device_tokens``
        (int32 on the device, one per entry, each entry then brings one placeholder token)
        gives the tokens without the host knowing them: what a sampler just wrote."""
        self.check_entries(entries)
        if device_tokens is not None and (device_tokens.dtype != torch.int32 or device_tokens.numel() != len(entries)
                                          or any(len(e.tokens) != 1 for e in entries)):
            raise ValueError("step: device tokens need one int32 token per entry and one placeholder token each")
        self.cache.reserve([(e.seq, e.seq.length + len(e.tokens)) for e in entries])
        if self.use_graphs and self.model.graph_safe and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            logits, batch = self._decode_step(entries, device_tokens)
        else:
            batch = build_step(entries, self.cache, self.workspace, self.device)
            if device_tokens is not None:
                batch.tokens.copy_(device_tokens)
            logits = self.model.forward(batch, self.cache)
        for e, new_len in zip(entries, batch.host_len):
            self.cache.commit(e.seq, new_len)
        return logits

    def _decode_step(self, entries: List[StepEntry], device_tokens: Optional[torch.Tensor] = None):
        """A decode step through a captured graph.  The first step of a shape runs eagerly
        (it also allocates every buffer), the second captures, later ones replay."""
        from ..cache.manager import pages_for
        B = len(entries)
        need = max(pages_for(e.seq.length + 1) for e in entries)
        width = 1 << (need - 1).bit_length()
        key = (B, width)
        meta = self._decode_meta.get(key)
        if meta is None:
            meta = self._decode_meta[key] = DecodeMeta(B, width, self.cache, self.workspace, self.device,
                                                       f"step.meta.decode.{B}.{width}")
        batch = meta.fill(entries)          # max_len is the bucket's: kernel launch shapes depend on it only
        if device_tokens is not None:
            batch.tokens.copy_(device_tokens)       # after the metadata copy, before the graph that reads it
        batch.tag = f".decode.{B}"
        state = self._graphs.get(key)
        if state is None:
            self._graphs[key] = "warm"
            return self.model.forward(batch, self.cache), batch
        if state == "warm":
            ops = self.ctx.ops
            torch.cuda.synchronize(self.device)
            before = ops.launches
            graph = torch.cuda.CUDAGraph()
            self.workspace.capturing = True
            try:
                with torch.cuda.graph(graph):
                    logits = self.model.forward(batch, self.cache)
            finally:
                self.workspace.capturing = False
            state = (graph, logits, ops.launches - before)
            ops.launches = before
            self._graphs[key] = state
        graph, logits, launches = state
        graph.replay()
        self.ctx.ops.launches += launches
        self.graph_replays += 1
        return logits, batch

    def step_chunked(self, entries: List[StepEntry]) -> Optional[torch.Tensor]:
        """``step`` for any number of tokens: a step larger than the step capacity is cut into
        several, each sequence's tokens staying in order.  The logits come back in the order
        of the entries and of each entry's ``want``, in a tensor of their own."""
        total = sum(len(e.tokens) for e in entries)
        if total <= self.max_step_tokens:
            logits = self.step(entries)
            return logits
        self.check_entries([StepEntry(e.seq, e.tokens[:1], ()) for e in entries])
        # row of each wanted place in the result
        rows, r = [], 0
        for e in entries:
            rows.append({int(w): r + k for k, w in enumerate(e.want)})
            if len(rows[-1]) != len(e.want):
                raise ValueError("step: a place is wanted twice")
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
        return result

    # ------------------------------------------------------------------ accounting
    def decode_step_bytes(self, live_lengths: Seq[int]) -> int:
        """Bytes a decode step has to read: every weight it uses once and the cache of the
        live sequences."""
        kv = sum(int(l) for l in live_lengths) * self.cache.bytes_per_token()
        return self.model.step_weight_bytes() + kv
