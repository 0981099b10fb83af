"""One step's batch: which tokens run, where they sit in their sequences, what is wanted.

Tokens of all sequences are packed one after another without padding.  Per token the
device holds its sequence's row in the batch and its absolute position; per sequence the
offsets of its tokens, its length before and after the step, its state slot and, per cache
group, the physical pages of its logical pages.  All of it travels in one host-to-device
copy of one int32 array.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence as Seq

import numpy as np
import torch

from ..cache.manager import PAGE_TOKENS, CacheManager, Sequence, pages_for


@dataclass
class StepEntry:
    """A sequence's share of a step: its next tokens and the places (indices into these
    tokens) whose logits are wanted."""

    seq: Sequence
    tokens: Seq[int]
    want: Seq[int] = ()


@dataclass
class StepBatch:
    num_tokens: int
    num_seqs: int
    num_wanted: int
    tokens: torch.Tensor
    positions: torch.Tensor
    tok_seq: torch.Tensor
    seq_start: torch.Tensor
    seq_pos0: torch.Tensor
    seq_len: torch.Tensor
    state_slots: torch.Tensor
    want_rows: Optional[torch.Tensor]
    page_tables: List[torch.Tensor]
    max_new: int
    max_len: int
    is_decode: bool
    host_new: List[int]
    host_len: List[int]
    host_state_slots: List[int] = field(default_factory=list)
    shared: Dict[str, Any] = field(default_factory=dict)
    tag: str = ""               # suffix of buffers whose size follows the batch (captured steps keep their own)


def _round4(n: int) -> int:
    return (n + 3) & ~3


def build_step(entries: List[StepEntry], cache: CacheManager, workspace, device, table_width: Optional[int] = None,
               meta_name: str = "step.meta") -> StepBatch:
    """Packs ``entries`` (already reserved in the cache) into device metadata.  A fixed
    ``table_width`` (pages per page-table row) and a ``meta_name`` of its own give a layout
    and addresses that stay the same from step to step, which a captured graph needs."""
    B = len(entries)
    new = [len(e.tokens) for e in entries]
    pos0 = [e.seq.length for e in entries]
    lens = [p + n for p, n in zip(pos0, new)]
    T = sum(new)
    n_want = sum(len(e.want) for e in entries)
    groups = cache.groups
    need = max(1, max(pages_for(l) for l in lens))
    if table_width is not None and table_width < need:
        raise ValueError("step: the fixed page-table width is smaller than a sequence needs")
    widths = [need if table_width is None else table_width for _ in groups]

    # layout of the packed int32 array (every segment starts on a 16-byte boundary)
    off: Dict[str, int] = {}
    cur = 0
    for name, n in (("tokens", T), ("positions", T), ("tok_seq", T), ("seq_start", B + 1), ("seq_pos0", B),
                    ("seq_len", B), ("state_slots", B), ("want", max(n_want, 1))):
        off[name] = cur
        cur = _round4(cur + n)
    for gi, w in enumerate(widths):
        off[f"pt{gi}"] = cur
        cur = _round4(cur + B * w)
    total = cur

    host = torch.empty(total, dtype=torch.int32, pin_memory=(torch.device(device).type == "cuda"))
    a = host.numpy()
    a[:] = 0
    t0 = 0
    starts = [0]
    want_rows: List[int] = []
    for b, e in enumerate(entries):
        n = new[b]
        a[off["tokens"] + t0: off["tokens"] + t0 + n] = np.asarray(e.tokens, dtype=np.int64)
        a[off["positions"] + t0: off["positions"] + t0 + n] = np.arange(pos0[b], pos0[b] + n)
        a[off["tok_seq"] + t0: off["tok_seq"] + t0 + n] = b
        for w in e.want:
            if not 0 <= w < n:
                raise ValueError(f"step: wanted place {w} is outside the {n} tokens of this step")
            want_rows.append(t0 + int(w))
        t0 += n
        starts.append(t0)
    a[off["seq_start"]: off["seq_start"] + B + 1] = starts
    a[off["seq_pos0"]: off["seq_pos0"] + B] = pos0
    a[off["seq_len"]: off["seq_len"] + B] = lens
    a[off["state_slots"]: off["state_slots"] + B] = [e.seq.state_slot for e in entries]
    if want_rows:
        a[off["want"]: off["want"] + n_want] = want_rows
    for gi, w in enumerate(widths):
        table = np.full((B, w), -1, dtype=np.int32)
        for b, e in enumerate(entries):
            pages = e.seq.pages[gi][:w]
            table[b, :len(pages)] = [(-1 if p is None else p) for p in pages]
        a[off[f"pt{gi}"]: off[f"pt{gi}"] + B * w] = table.reshape(-1)

    cap = 1 << max(10, (total - 1).bit_length())
    dev = workspace.buffer(meta_name, (cap,), torch.int32)[:total]
    dev.copy_(host, non_blocking=True)

    def seg(name: str, n: int) -> torch.Tensor:
        return dev[off[name]: off[name] + n]

    return StepBatch(
        num_tokens=T, num_seqs=B, num_wanted=n_want,
        tokens=seg("tokens", T), positions=seg("positions", T), tok_seq=seg("tok_seq", T),
        seq_start=seg("seq_start", B + 1), seq_pos0=seg("seq_pos0", B), seq_len=seg("seq_len", B),
        state_slots=seg("state_slots", B), want_rows=seg("want", n_want) if n_want else None,
        page_tables=[seg(f"pt{gi}", B * w).view(B, w) for gi, w in enumerate(widths)],
        max_new=max(new), max_len=max(lens), is_decode=all(n == 1 for n in new),
        host_new=new, host_len=lens, host_state_slots=[e.seq.state_slot for e in entries])


class DecodeMeta:
    """The metadata of decode steps (one token per sequence, its logits wanted) of a fixed
    batch size and page-table width, kept from step to step: the same layout and device
    addresses as ``build_step`` gives with that ``table_width`` and ``meta_name``, but a step
    only writes what changed since the last one (tokens, positions, lengths, and the page-table
    row of a sequence whose pages changed).  The host side is a small ring of pinned buffers:
    a buffer is written again only after the copy that read it has finished."""

    RING = 4

    def __init__(self, batch: int, width: int, cache: CacheManager, workspace, device, meta_name: str):
        B = self.B = batch
        self.width = width
        self.n_groups = len(cache.groups)
        off: Dict[str, int] = {}
        cur = 0
        for name, n in (("tokens", B), ("positions", B), ("tok_seq", B), ("seq_start", B + 1), ("seq_pos0", B),
                        ("seq_len", B), ("state_slots", B), ("want", B)):
            off[name] = cur
            cur = _round4(cur + n)
        for gi in range(self.n_groups):
            off[f"pt{gi}"] = cur
            cur = _round4(cur + B * width)
        self.off, self.total = off, cur
        pin = torch.device(device).type == "cuda"
        self.hosts = [torch.zeros(cur, dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self.arrays = [h.numpy() for h in self.hosts]
        self.events: List[Optional[torch.cuda.Event]] = [None] * self.RING
        self.seqs: List[Optional[list]] = [None] * self.RING          # the sequences a buffer was written for
        self.versions: List[Optional[list]] = [None] * self.RING      # their pages_version then
        self.turn = 0
        cap = 1 << max(10, (cur - 1).bit_length())
        dev = self.dev = workspace.buffer(meta_name, (cap,), torch.int32)[:cur]

        def seg(name: str, n: int) -> torch.Tensor:
            return dev[off[name]: off[name] + n]

        self.batch = StepBatch(
            num_tokens=B, num_seqs=B, num_wanted=B, tokens=seg("tokens", B), positions=seg("positions", B),
            tok_seq=seg("tok_seq", B), seq_start=seg("seq_start", B + 1), seq_pos0=seg("seq_pos0", B),
            seq_len=seg("seq_len", B), state_slots=seg("state_slots", B), want_rows=seg("want", B),
            page_tables=[seg(f"pt{gi}", B * width).view(B, width) for gi in range(self.n_groups)],
            max_new=1, max_len=width * PAGE_TOKENS, is_decode=True, host_new=[1] * B, host_len=[0] * B)

    def _row(self, a, gi: int, b: int, pages) -> None:
        w = self.width
        lo = self.off[f"pt{gi}"] + b * w
        a[lo: lo + w] = -1
        pages = pages[:w]
        a[lo: lo + len(pages)] = [(-1 if p is None else p) for p in pages]

    def fill(self, entries: List[StepEntry]) -> StepBatch:
        B, off = self.B, self.off
        r = self.turn
        self.turn = (r + 1) % self.RING
        if self.events[r] is not None:
            self.events[r].synchronize()              # the copy that read this buffer has finished
        a = self.arrays[r]
        seqs = [e.seq for e in entries]
        versions = [s.pages_version for s in seqs]
        old = self.seqs[r]
        if old is None or len(old) != B or any(x is not y for x, y in zip(old, seqs)):
            a[off["tok_seq"]: off["tok_seq"] + B] = np.arange(B)
            a[off["seq_start"]: off["seq_start"] + B + 1] = np.arange(B + 1)
            a[off["want"]: off["want"] + B] = np.arange(B)
            a[off["state_slots"]: off["state_slots"] + B] = [s.state_slot for s in seqs]
            for gi in range(self.n_groups):
                for b, s in enumerate(seqs):
                    self._row(a, gi, b, s.pages[gi])
        else:
            was = self.versions[r]
            for b in range(B):
                if versions[b] != was[b]:
                    for gi in range(self.n_groups):
                        self._row(a, gi, b, seqs[b].pages[gi])
        self.seqs[r], self.versions[r] = seqs, versions
        pos0 = [s.length for s in seqs]
        a[off["tokens"]: off["tokens"] + B] = [e.tokens[0] for e in entries]
        a[off["positions"]: off["positions"] + B] = pos0
        a[off["seq_pos0"]: off["seq_pos0"] + B] = pos0
        lens = [p + 1 for p in pos0]
        a[off["seq_len"]: off["seq_len"] + B] = lens
        self.dev.copy_(self.hosts[r], non_blocking=True)
        if self.dev.is_cuda:
            ev = self.events[r] or torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.dev.device))
            self.events[r] = ev
        batch = self.batch
        batch.shared = {}                  # what parts keep per step (the rotary table) is of the last step
        batch.host_len = lens
        batch.host_state_slots = [s.state_slot for s in seqs]
        return batch
