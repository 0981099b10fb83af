"""The cache's bookkeeping (no GPU): no page or slot lost, held twice or freed twice."""
import random

import pytest
import torch

from hilbert_pruned_8b_b200.cache import PAGE_TOKENS, CacheFull, CacheManager, IndexPool, pages_for
from hilbert_pruned_8b_b200.parts.base import CacheNeed, StateNeed

CPU = torch.device("cpu")


def _manager(max_tokens=1024, window=None, state=False, **kw):
    needs = {0: CacheNeed(2, 16), 1: CacheNeed(2, 16), 2: CacheNeed(1, 32, window)}
    states = {1: StateNeed((3, 4))} if state else {}
    return CacheManager(needs, states, max_tokens, CPU, torch.float32, **kw)


def test_pool_rejects_double_free_and_foreign_indices():
    p = IndexPool(4)
    a = p.alloc(3)
    assert sorted(a) == [0, 1, 2] and p.num_free == 1
    p.free([1])
    with pytest.raises(ValueError, match="not held"):
        p.free([1])
    with pytest.raises(ValueError, match="outside"):
        p.free([9])
    with pytest.raises(CacheFull):
        p.alloc(3)
    assert p.alloc(2) == [1, 3]          # lowest first, the freed one again
    assert p.num_free == 0


def test_groups_have_storage_of_their_own():
    m = _manager()
    assert len(m.groups) == 2
    full = m.groups[m.group_of(0)]
    assert full.entries == [0, 1] and full.k.shape == (2, 16, 2, PAGE_TOKENS, 16)
    other = m.groups[m.group_of(2)]
    assert other.entries == [2] and other.k.shape == (1, 16, 1, PAGE_TOKENS, 32)
    assert m.view(1).k.data_ptr() == full.k[1].data_ptr() and m.view(1).group == m.group_of(0)
    assert m.view(7) is None


def test_sequences_grow_in_pages_and_give_everything_back():
    m = _manager(max_tokens=640)
    assert m.num_pages == 10
    a, b = m.open(), m.open()
    m.reserve([(a, 1), (b, 130)])
    m.commit(a, 1), m.commit(b, 130)
    assert [len(a.pages[g]) for g in range(2)] == [1, 1] and [len(b.pages[g]) for g in range(2)] == [3, 3]
    assert m.pages_free() == [6, 6]
    m.reserve([(a, 64)])                      # still inside its page
    assert m.pages_free() == [6, 6]
    m.reserve([(a, 65)])
    m.commit(a, 65)
    assert m.pages_free() == [5, 5]
    held = [p for s in (a, b) for p in s.pages[0]]
    assert len(set(held)) == len(held) == 5   # no page held twice
    with pytest.raises(CacheFull):
        m.reserve([(a, 65 + 6 * 64)])
    assert m.pages_free() == [5, 5]           # a refused step takes nothing
    m.close(a)
    with pytest.raises(ValueError, match="closed twice"):
        m.close(a)
    with pytest.raises(ValueError, match="is closed"):
        m.reserve([(a, 3)])
    m.close(b)
    assert m.pages_free() == [10, 10] and m.slots.num_held == 0 and not m.live_sequences()


def test_slots_are_used_again_lowest_first():
    m = _manager(max_tokens=256, state=True, max_sequences=3)
    s = [m.open() for _ in range(3)]
    assert sorted(x.state_slot for x in s) == [0, 1, 2]
    with pytest.raises(CacheFull):
        m.open()
    m.state_view(1)[s[1].state_slot] += 5.0
    m.close(s[1])
    again = m.open()
    assert again.state_slot == s[1].state_slot
    assert torch.all(m.state_view(1)[again.state_slot] == 0)      # zeroed when the sequence opens
    assert m.state_view(0) is None and m.state_view(1).shape == (3, 3, 4)


def test_window_group_gives_pages_back_early():
    m = _manager(max_tokens=64 * 8, window=70)
    g_win = m.group_of(2)
    g_full = m.group_of(0)
    s = m.open()
    m.reserve([(s, 300)])
    m.commit(s, 300)
    assert m.pages_free()[g_full] == 8 - 5 and m.pages_free()[g_win] == 8 - 5
    m.reserve([(s, 301)])                     # next token at position 300 sees keys 231..300
    m.commit(s, 301)
    assert s.pages[g_win][:3] == [None, None, None] and s.pages[g_win][3] is not None
    assert m.pages_free()[g_win] == 8 - 2 and m.pages_free()[g_full] == 8 - 5
    with pytest.raises(ValueError):
        m.truncate(s, 100)
    m.close(s)
    assert m.pages_free() == [8, 8]


def test_truncate_rewinds_a_sequence():
    m = _manager(max_tokens=512)
    s = m.open()
    m.reserve([(s, 200)])
    m.commit(s, 200)
    m.truncate(s, 65)
    assert s.length == 65 and [len(p) for p in s.pages] == [2, 2] and m.pages_free() == [6, 6]
    with pytest.raises(ValueError):
        m.truncate(s, 66)
    m.close(s)


def test_snapshot_and_restore_rewind_keys_and_fixed_size_state():
    """Truncation alone cannot rewind fixed-size state; a snapshot carries a copy of it, and a
    restore gives the later pages back and puts the copy in place."""
    m = _manager(max_tokens=512, state=True)
    s, other = m.open(), m.open()
    m.reserve([(s, 70)])
    m.commit(s, 70)
    m.state_view(1)[s.state_slot].fill_(3.0)
    snap = m.snapshot(s)
    m.reserve([(s, 200)])
    m.commit(s, 200)
    m.state_view(1)[s.state_slot].fill_(9.0)
    version = s.pages_version
    with pytest.raises(ValueError, match="fixed-size state"):
        m.truncate(s, 70)
    with pytest.raises(ValueError, match="snapshot is of sequence"):
        m.restore(other, snap)
    m.restore(s, snap)
    assert s.length == 70 and [len(p) for p in s.pages] == [2, 2] and s.pages_version > version
    assert torch.all(m.state_view(1)[s.state_slot] == 3.0)
    assert m.pages_free() == [6, 6]
    m.restore(s, snap)                                 # a snapshot can be gone back to again
    m.reserve([(s, 130)])
    m.commit(s, 130)
    m.restore(s, snap)
    assert s.length == 70 and m.pages_free() == [6, 6]
    m.close(s)
    m.close(other)
    with pytest.raises(ValueError, match="closed"):
        m.restore(s, snap)
    assert m.pages_free() == [8, 8] and m.slots.num_held == 0


def test_check_room_reserves_nothing():
    m = _manager(max_tokens=64 * 4)
    s = m.open()
    m.check_room([(s, 256)])
    with pytest.raises(CacheFull, match="needs 5 more pages"):
        m.check_room([(s, 257)])
    assert m.pages_free() == [4, 4] and s.pages == [[], []]
    m.close(s)


def test_random_traffic_never_loses_a_page():
    rng = random.Random(0)
    m = _manager(max_tokens=64 * 40, window=100, state=True)
    live = []
    for _ in range(400):
        if live and rng.random() < 0.3:
            m.close(live.pop(rng.randrange(len(live))))
        elif rng.random() < 0.5 and len(live) < 10:
            live.append(m.open())
        elif live:
            s = rng.choice(live)
            new = s.length + rng.randint(1, 90)
            try:
                m.reserve([(s, new)])
                m.commit(s, new)
            except CacheFull:
                pass
        for gi, g in enumerate(m.groups):
            held = [p for s in live for p in s.pages[gi] if p is not None]
            assert len(held) == len(set(held)) == g.pool.num_held
            assert all(g.pool.is_held(p) for p in held)
        assert m.slots.num_held == len(live) and len({s.state_slot for s in live}) == len(live)
    for s in live:
        m.close(s)
    assert m.pages_free() == [40, 40] and m.slots.num_held == 0
    assert pages_for(1) == 1 and pages_for(64) == 1 and pages_for(65) == 2


def test_decode_metadata_kept_from_step_to_step_equals_a_fresh_build():
    """DecodeMeta writes only what changed since the last step (tokens, positions, lengths,
    page-table rows of sequences whose pages changed); the device array must equal what
    build_step writes from scratch, step after step: pages added, pages a window gave back,
    a sequence replaced by another, more steps than the ring of host buffers is long."""
    from hilbert_pruned_8b_b200.engine.batch import DecodeMeta, StepEntry, build_step
    from hilbert_pruned_8b_b200.engine.workspace import Workspace
    m = _manager(max_tokens=4096, window=70)
    ws_a, ws_b = Workspace(CPU), Workspace(CPU)
    rnd = random.Random(5)
    seqs = [m.open() for _ in range(3)]
    for s, n in zip(seqs, (3, 60, 130)):                 # prompts
        m.reserve([(s, n)])
        m.commit(s, n)
    width = 8
    meta = DecodeMeta(3, width, m, ws_a, CPU, "meta")
    for step in range(150):
        if step == 40:                                   # one sequence ends, another takes its place
            m.close(seqs[1])
            seqs[1] = m.open()
            m.reserve([(seqs[1], 5)])
            m.commit(seqs[1], 5)
        entries = [StepEntry(s, [rnd.randrange(1000)], [0]) for s in seqs]
        m.reserve([(e.seq, e.seq.length + 1) for e in entries])
        kept = meta.fill(entries)
        fresh = build_step(entries, m, ws_b, CPU, table_width=width, meta_name="fresh")
        for name in ("tokens", "positions", "tok_seq", "seq_start", "seq_pos0", "seq_len", "state_slots", "want_rows"):
            assert torch.equal(getattr(kept, name), getattr(fresh, name)), (step, name)
        for a, b in zip(kept.page_tables, fresh.page_tables):
            assert torch.equal(a, b), step
        assert kept.host_len == fresh.host_len and kept.is_decode and fresh.is_decode
        assert kept.shared == {}
        kept.shared["x"] = 1                             # what a part leaves there must not survive the step
        for e in entries:
            m.commit(e.seq, e.seq.length + 1)
    assert any(p is None for p in seqs[2].pages[m.group_of(2)])      # the window did give pages back
