"""The cache: keys and values per plan entry, per sequence, in pages; fixed-size state beside it.

Layout.  Time is cut into pages of ``PAGE_TOKENS`` (64) tokens.  Plan entries whose mixers
have the same need (kv heads, head size, window) form a GROUP with storage of its own:
``k, v: [entries, pages, kv_heads, PAGE_TOKENS, head_dim]`` and its own page pool.  A
sequence holds, per group, the list of physical pages of its logical pages; a group with a
window gives pages back as soon as no later token can see them.  The same page index is
used by all entries of a group, so one page table per group serves all its layers.

The reference keeps one sequence with ``[max_seq][kv_heads*head_dim]`` arrays per
full-attention layer, indexed by the layer's number within its kind, and separate
fixed-size state arrays for its other layer kind (cleanroom-transformer/src/cpu_backend.c:15-24,
310-337; transformer.h:307-318); rewinding is a position reset (cpu_backend.c:279-292).
Batches, slots and paging are this library's own.

Per-sequence state of fixed size lives in ``state[entry]: [slots, *shape]``; a sequence's
slot is zeroed when the sequence opens.  The Llama decoder has no such state: the area
exists, with zero entries.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import CacheNeed, StateNeed
from .pool import CacheFull, IndexPool

PAGE_TOKENS = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass
class LayerCache:
    """What a mixer sees of the cache: its entry's storage and the group it belongs to."""

    k: torch.Tensor            # [pages, kv_heads, PAGE_TOKENS, head_dim]
    v: torch.Tensor
    group: int
    window: Optional[int]


@dataclass
class Sequence:
    seq_id: int
    length: int = 0
    state_slot: int = -1
    # per group: physical page of each logical page (None: given back, outside the window)
    pages: List[List[Optional[int]]] = field(default_factory=list)
    open: bool = True
    pages_version: int = 0      # counts the changes of `pages`: who keeps a copy compares this


@dataclass
class Snapshot:
    """A sequence's length and fixed-size state at some moment (``CacheManager.snapshot``)."""

    seq_id: int
    length: int
    state: Dict[int, torch.Tensor]


class CacheGroup:
    def __init__(self, need: CacheNeed, entries: List[int], num_pages: int, device, dtype,
                 allocate: bool = True):
        self.need = need
        self.entries = list(entries)
        self.index_of = {e: i for i, e in enumerate(entries)}
        self.pool = IndexPool(num_pages, "page")
        shape = (len(entries), num_pages, need.num_kv_heads, PAGE_TOKENS, need.head_dim)
        self.shape = shape
        if allocate:
            # zero-filled: a page's unwritten tail is read by no kernel, but NaN garbage there
            # would still poison 0 * NaN in a tile-wide product
            self.k = torch.zeros(shape, dtype=dtype, device=device)
            self.v = torch.zeros(shape, dtype=dtype, device=device)
        else:
            self.k = self.v = None

    def bytes_per_token(self, element_size: int) -> int:
        return 2 * len(self.entries) * self.need.num_kv_heads * self.need.head_dim * element_size


class CacheManager:
    def __init__(self, cache_needs: Dict[int, CacheNeed], state_needs: Dict[int, StateNeed], max_tokens: int,
                 device, dtype: torch.dtype, max_sequences: Optional[int] = None, allocate: bool = True):
        if max_tokens < 1:
            raise ValueError("cache: max_tokens must be positive")
        self.device = device
        self.dtype = dtype
        self.max_tokens = max_tokens
        self.num_pages = pages_for(max_tokens)
        self.max_sequences = max_sequences if max_sequences is not None else min(self.num_pages, 1024)
        by_need: Dict[CacheNeed, List[int]] = {}
        for entry in sorted(cache_needs):
            by_need.setdefault(cache_needs[entry], []).append(entry)
        self.groups: List[CacheGroup] = [
            CacheGroup(need, entries, self.num_pages, device, dtype, allocate) for need, entries in by_need.items()]
        self._windowed = any(g.need.window is not None for g in self.groups)
        self._group_of_entry: Dict[int, int] = {}
        for gi, g in enumerate(self.groups):
            for e in g.entries:
                self._group_of_entry[e] = gi
        self.slots = IndexPool(self.max_sequences, "sequence slot")
        self.state: Dict[int, torch.Tensor] = {}
        self.state_needs = dict(state_needs)
        for entry, need in state_needs.items():
            if allocate:
                self.state[entry] = torch.zeros((self.max_sequences,) + tuple(need.shape), dtype=need.dtype,
                                                device=device)
        self._next_id = 0
        self._live: Dict[int, Sequence] = {}

    # ------------------------------------------------------------------ sequences
    def open(self) -> Sequence:
        (slot,) = self.slots.alloc(1)
        seq = Sequence(self._next_id, 0, slot, [[] for _ in self.groups])
        self._next_id += 1
        self._live[seq.seq_id] = seq
        for t in self.state.values():
            t[slot].zero_()
        return seq

    def close(self, seq: Sequence) -> None:
        if not seq.open or self._live.get(seq.seq_id) is not seq:
            raise ValueError(f"cache: sequence {seq.seq_id} is closed twice or was never opened")
        for g, pages in zip(self.groups, seq.pages):
            g.pool.free([p for p in pages if p is not None])
        self.slots.free([seq.state_slot])
        seq.pages = [[] for _ in self.groups]
        seq.open = False
        del self._live[seq.seq_id]

    def live_sequences(self) -> List[Sequence]:
        return list(self._live.values())

    # ------------------------------------------------------------------ pages
    def _pages_needed(self, seqs_and_lengths) -> List[int]:
        need = [0] * len(self.groups)
        for seq, new_len in seqs_and_lengths:
            for gi, g in enumerate(self.groups):
                have = len(seq.pages[gi])
                need[gi] += max(0, pages_for(new_len) - have)
        return need

    def check_room(self, seqs_and_lengths: List[Tuple[Sequence, int]]) -> None:
        """Raises ``CacheFull`` if the pages are not there for each sequence to grow to its new
        length; reserves nothing.  A group with a window may get by with fewer (it gives pages
        back as the sequence grows): for such a group this is the worst case."""
        need = self._pages_needed(seqs_and_lengths)
        for gi, g in enumerate(self.groups):
            if g.need.window is None and need[gi] > g.pool.num_free:
                raise CacheFull(
                    f"cache: the call needs {need[gi]} more pages of {PAGE_TOKENS} tokens, "
                    f"{g.pool.num_free} of {g.pool.size} are free (max_tokens {self.max_tokens})")

    def reserve(self, seqs_and_lengths: List[Tuple[Sequence, int]]) -> None:
        """Makes room for each sequence to grow to its new length; all or nothing."""
        for seq, new_len in seqs_and_lengths:
            if not seq.open:
                raise ValueError(f"cache: sequence {seq.seq_id} is closed")
            if new_len < seq.length:
                raise ValueError("cache: reserve cannot shrink a sequence (use truncate)")
        # pages a window lets go of are given back first: they may be what the step needs
        if self._windowed:
            for seq, _ in seqs_and_lengths:
                self._release_outside_window(seq, seq.length)
        need = self._pages_needed(seqs_and_lengths)
        if not any(need):
            return
        for gi, g in enumerate(self.groups):
            if need[gi] > g.pool.num_free:
                raise CacheFull(
                    f"cache: the step needs {need[gi]} more pages of {PAGE_TOKENS} tokens, "
                    f"{g.pool.num_free} of {g.pool.size} are free (max_tokens {self.max_tokens})")
        for seq, new_len in seqs_and_lengths:
            for gi, g in enumerate(self.groups):
                extra = pages_for(new_len) - len(seq.pages[gi])
                if extra > 0:
                    seq.pages[gi].extend(g.pool.alloc(extra))
                    seq.pages_version += 1

    def _release_outside_window(self, seq: Sequence, first_new_position: int) -> None:
        for gi, g in enumerate(self.groups):
            w = g.need.window
            if w is None:
                continue
            # the oldest key any coming token can see
            oldest = max(0, first_new_position - w + 1)
            dead = oldest // PAGE_TOKENS
            pages = seq.pages[gi]
            gone = [p for p in pages[:dead] if p is not None]
            if gone:
                g.pool.free(gone)
                for i in range(min(dead, len(pages))):
                    pages[i] = None
                seq.pages_version += 1

    def commit(self, seq: Sequence, new_len: int) -> None:
        seq.length = new_len

    def truncate(self, seq: Sequence, length: int) -> None:
        """Rewinds a sequence: later keys and values are forgotten, their pages given back (the
        reference's restore is a position reset, rows beyond it are overwritten later:
        cpu_backend.c:279-292).  Fixed-size state cannot be rewound this way: it needs the copy
        that ``snapshot`` takes."""
        if self.state and length != seq.length:
            raise ValueError("cache: a sequence with fixed-size state cannot be rewound by truncation "
                             "(take a snapshot and restore it)")
        self._forget_after(seq, length)

    def _forget_after(self, seq: Sequence, length: int) -> None:
        if not seq.open:
            raise ValueError(f"cache: sequence {seq.seq_id} is closed")
        if length > seq.length or length < 0:
            raise ValueError("cache: truncate needs 0 <= length <= current length")
        keep = pages_for(length)
        for gi, g in enumerate(self.groups):
            w = g.need.window
            if w is not None and any(p is None for p in seq.pages[gi][max(0, (length - w)) // PAGE_TOKENS:keep]):
                raise ValueError("cache: pages inside the rewound window were already given back")
        for gi, g in enumerate(self.groups):
            tail = seq.pages[gi][keep:]
            g.pool.free([p for p in tail if p is not None])
            del seq.pages[gi][keep:]
        seq.pages_version += 1
        seq.length = length

    def snapshot(self, seq: Sequence) -> "Snapshot":
        """Remembers where a sequence stands: its length and a copy of its fixed-size state (the
        reference's snapshot copies its other layer kind's state and notes the position,
        cpu_backend.c:265-277).  Keys and values are not copied: a restore forgets the later ones."""
        if not seq.open:
            raise ValueError(f"cache: sequence {seq.seq_id} is closed")
        return Snapshot(seq.seq_id, seq.length, {e: t[seq.state_slot].clone() for e, t in self.state.items()})

    def restore(self, seq: Sequence, snap: "Snapshot") -> None:
        """Takes a sequence back to a snapshot of itself: later keys and values are forgotten,
        the fixed-size state is the snapshot's again."""
        if snap.seq_id != seq.seq_id:
            raise ValueError(f"cache: the snapshot is of sequence {snap.seq_id}, not of {seq.seq_id}")
        self._forget_after(seq, snap.length)
        for e, t in self.state.items():
            t[seq.state_slot].copy_(snap.state[e])

    # ------------------------------------------------------------------ views
    def group_of(self, entry: int) -> int:
        return self._group_of_entry[entry]

    def view(self, entry: int) -> Optional[LayerCache]:
        gi = self._group_of_entry.get(entry)
        if gi is None:
            return None
        g = self.groups[gi]
        i = g.index_of[entry]
        return LayerCache(g.k[i], g.v[i], gi, g.need.window)

    def state_view(self, entry: int) -> Optional[torch.Tensor]:
        return self.state.get(entry)

    # ------------------------------------------------------------------ accounting
    def tokens_capacity(self) -> int:
        return self.num_pages * PAGE_TOKENS

    def pages_free(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(es) for g in self.groups)
