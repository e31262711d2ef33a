"""Host arithmetic of the decode schedule (the kernel computes the same split on the device)."""
import numpy as np
import pytest

from hy3_b200.attn import decode_schedule


@pytest.mark.parametrize("lens,heads,ctas", [([32768], 8, 148), ([1], 8, 148), ([128, 129, 0, 5000], 8, 148),
                                              ([1000] * 64, 4, 148), ([65536, 1024], 1, 7), ([0, 0], 8, 148),
                                              ([300] * 18, 8, 148), ([300] * 19, 8, 148), ([70000, 5], 8, 148)])
def test_schedule_partitions_units(lens, heads, ctas):
    """Every unit belongs to exactly one CTA; ranges are ordered; with few segments no range crosses a
    segment boundary; with many segments the ranges are balanced to one page."""
    pages = [(n + 127) // 128 for n in lens]
    total = sum(pages) * heads
    ranges = []
    for c in range(ctas):
        tot, u0, u1 = decode_schedule(lens, heads, ctas, c)
        assert tot == total and u1 >= u0
        if u1 > u0:
            ranges.append((u0, u1))
    assert sorted(ranges) == ranges
    covered = 0
    for u0, u1 in ranges:
        assert u0 == covered
        covered = u1
    assert covered == total
    if len(lens) * heads < ctas:
        bounds = set()
        acc = 0
        for p in pages:
            for _ in range(heads):
                bounds.add(acc)
                acc += p
        for u0, u1 in ranges:
            assert not any(u0 < b < u1 for b in bounds), "a CTA straddles two segments"
    elif ranges:
        sizes = [b - a for a, b in ranges]
        assert max(sizes) - min(sizes) <= 1


def test_piece_count_formula_matches_ranges():
    """c_first / c_last as computed in the kernel: ceil((u+1)*C/U)-1 is the CTA that owns unit u."""
    rng = np.random.default_rng(0)
    for _ in range(200):
        C = int(rng.integers(1, 300))
        U = int(rng.integers(1, 5000))
        starts = [c * U // C for c in range(C + 1)]
        for u in rng.integers(0, U, 20):
            u = int(u)
            owner = -(-((u + 1) * C) // U) - 1
            assert starts[owner] <= u < starts[owner + 1]
