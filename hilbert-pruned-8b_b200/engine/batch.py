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
