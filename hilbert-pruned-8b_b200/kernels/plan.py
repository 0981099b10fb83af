"""Launch-shape decisions of the host that need no device: pure functions, tested on the CPU."""
from __future__ import annotations


def decode_splits(sequences: int, kv_heads: int, max_pages: int, cta_slots: int) -> int:
    """Key splits of split-K decode attention for ``sequences`` x ``kv_heads`` (sequence, kv head)
    pairs whose longest cache holds ``max_pages`` pages, on a device that holds ``cta_slots``
    of the kernel's CTAs at once.

    At most 16 splits and at most one for every eight pages (measured: more splits cost more in
    the combination than they gain).  One wave of the resident CTAs if that fills the device:
    batch 8 at 8192 tokens takes 4 splits on 296 slots.  Where one wave would leave a third of
    the device idle (batch 24: 192 CTAs) or a second wave would (batch 48: 384 CTAs), the
    splits that fill whole waves best, of 32 pages or more each (12 % of a step at batch 48)."""
    slots = max(1, cta_slots)
    pairs = max(1, sequences * kv_heads)
    limit = max(1, min(16, -(-max_pages // 8)))

    def fill(s: int) -> float:            # share of the waves' CTA slots that have work
        ctas = pairs * s
        return ctas / (-(-ctas // slots) * slots)

    best = max(1, min(slots // pairs, limit))
    if fill(best) < 0.8:
        for s in range(1, limit + 1):
            if -(-max_pages // s) >= 32 and fill(s) - 0.01 * s > fill(best) - 0.01 * best + 0.1:
                best = s
    return best
