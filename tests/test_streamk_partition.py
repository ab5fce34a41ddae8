"""The work division of the decode-width FP8 projection (fngine_b200/csrc/linear_fp8.cu: dec_begin, dec_owner,
the partial-tile slots and the grid rule of fb_linear_fp8_decode), restated with integers and checked over many
shapes: every (row tile, K block) position belongs to exactly one CTA, the CTAs that share a tile are a
contiguous range, no two partial segments use the same workspace slot, and the division-free test that picks a
contributor's slot agrees with the definition. The kernel itself is checked on the GPU for a few shapes; this
covers the arithmetic for all of them."""
import itertools

import pytest


def begin(c, G, total):
    return (total * c) // G


def owner(p, G, total):
    c = (p * G) // total
    while c + 1 < G and begin(c + 1, G, total) <= p:
        c += 1
    while c > 0 and begin(c, G, total) > p:
        c -= 1
    return c


def segments(c, G, total, kbt):
    """(tile, kb0, kb1, slot or None) of CTA c in the order the kernel walks them."""
    pos, end, out = begin(c, G, total), begin(c + 1, G, total), []
    first = pos
    while pos < end:
        m, kb0 = divmod(pos, kbt)
        kb1 = min(kbt, kb0 + (end - pos))
        full = kb0 == 0 and kb1 == kbt
        out.append((m, kb0, kb1, None if full else 2 * c + (0 if pos == first else 1)))
        pos += kb1 - kb0
    return out


def grid_for(m_tiles, kbt, sms):
    total = m_tiles * kbt
    want = max(total // 2, 1)
    grid = min(want, sms)
    if m_tiles <= sms and 4 * m_tiles >= 3 * sms:
        grid = m_tiles
    return grid


SHAPES = [(128, 20), (20, 48), (10, 20), (20, 5), (1940, 20), (3, 80), (8, 3), (1, 1), (2, 2), (194, 20), (104, 20),
          (147, 7), (149, 7), (111, 20), (110, 20), (37, 13)]


@pytest.mark.parametrize("m_tiles,kbt", SHAPES)
@pytest.mark.parametrize("sms", [148, 132, 7])
def test_every_position_once_and_slots_unique(m_tiles, kbt, sms):
    total = m_tiles * kbt
    G = grid_for(m_tiles, kbt, sms)
    assert 1 <= G <= min(total, sms)
    covered = [0] * total
    slots = {}
    by_tile = {}
    for c in range(G):
        segs = segments(c, G, total, kbt)
        assert segs, "every CTA has work"
        assert sum(1 for s in segs if s[3] is not None) <= 2
        for m, kb0, kb1, slot in segs:
            for kb in range(kb0, kb1):
                covered[m * kbt + kb] += 1
            if slot is not None:
                assert slot not in slots
                slots[slot] = (c, m)
                by_tile.setdefault(m, []).append((c, slot))
    assert covered == [1] * total
    assert max(slots, default=0) < 2 * 256  # the workspace holds two partial tiles for each of 256 CTAs
    for m, parts in by_tile.items():
        c_first, c_last = owner(m * kbt, G, total), owner((m + 1) * kbt - 1, G, total)
        assert [c for c, _ in parts] == list(range(c_first, c_last + 1)) and c_last > c_first
        for c, slot in parts:
            first_seg = total * c >= m * kbt * G              # the kernel's division-free test
            assert first_seg == (begin(c, G, total) // kbt == m)
            assert slot == 2 * c + (0 if first_seg else 1)
    # a tile held by one CTA is finished from tensor memory: no partial, no ticket
    for m in range(m_tiles):
        if owner(m * kbt, G, total) == owner((m + 1) * kbt - 1, G, total):
            assert m not in by_tile
    if m_tiles <= sms and 4 * m_tiles >= 3 * sms:
        assert not slots  # one CTA per row tile


def test_owner_is_the_cta_whose_range_holds_the_position():
    for G, total in itertools.product([1, 2, 5, 50, 148], [1, 7, 100, 200, 2560, 38800]):
        if G > total:
            continue
        for p in sorted({0, 1, total // 3, total // 2, total - 2, total - 1} & set(range(total))):
            c = owner(p, G, total)
            assert begin(c, G, total) <= p < begin(c + 1, G, total)
