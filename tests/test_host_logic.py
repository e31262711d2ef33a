"""Host arithmetic of the decode schedule (the kernel computes the same split on the device)."""
import numpy as np
import pytest

from hy3_b200.attn import decode_schedule


@pytest.mark.parametrize("lens,heads,ctas", [([32768], 8, 148), ([1], 8, 148), ([128, 129, 0, 5000], 8, 148),
                                              ([1000] * 64, 4, 148), ([65536, 1024], 1, 7), ([0, 0], 8, 148)])
def test_schedule_partitions_units(lens, heads, ctas):
    total = sum((n + 127) // 128 for n in lens) * heads
    prev = 0
    sizes = []
    for c in range(ctas):
        tot, u0, u1 = decode_schedule(lens, heads, ctas, c)
        assert tot == total and u0 == prev and u1 >= u0
        prev = u1
        sizes.append(u1 - u0)
    assert prev == total
    active = [x for x in sizes[:min(ctas, total)]]
    assert not active or (max(active) - min(active) <= 1 and min(active) >= 1)   # balanced to one page, no idle CTA inside
    assert all(x == 0 for x in sizes[min(ctas, total):])


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
