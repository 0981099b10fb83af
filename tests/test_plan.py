"""Launch-shape decisions of the host that need no device (``kernels/plan.py``)."""
import pytest

from hilbert_pruned_8b_b200.kernels.plan import decode_splits

SLOTS = 296        # 148 SMs x 2 resident CTAs of the head-size-128 kernel


def test_decode_splits_at_the_measured_points():
    # batch 8, 16, 32, 48, 64 at 8192 tokens (128 pages), 8 kv heads: what measured fastest
    assert [decode_splits(b, 8, 128, SLOTS) for b in (8, 16, 32, 48, 64)] == [4, 2, 1, 2, 1]
    assert decode_splits(24, 8, 128, SLOTS) == 3          # 192 CTAs would leave a third of the device idle
    assert decode_splits(1, 8, 128, SLOTS) == 16          # one sequence: as many splits as allowed
    assert decode_splits(1, 8, 512, SLOTS) == 16


@pytest.mark.parametrize("slots", [1, 7, 148, 296, 592])
def test_decode_splits_bounds(slots):
    for sequences in (1, 2, 3, 8, 24, 40, 48, 64, 100, 500):
        for kv in (1, 4, 8):
            for pages in (1, 2, 7, 8, 9, 31, 32, 64, 100, 128, 1000):
                s = decode_splits(sequences, kv, pages, slots)
                assert 1 <= s <= 16
                assert s <= -(-pages // 8), (sequences, kv, pages, slots, s)      # a split for every eight pages at most
                if sequences * kv * s > slots and s > 1:        # several waves only with long splits
                    assert -(-pages // s) >= 32, (sequences, kv, pages, slots, s)


def test_decode_splits_fill_the_device_for_few_long_sequences():
    for sequences in (1, 2, 4, 8, 16):
        s = decode_splits(sequences, 8, 1024, SLOTS)
        assert sequences * 8 * s > SLOTS // 2 or s == 16
