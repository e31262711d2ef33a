"""Host arithmetic of the decode schedule (the kernel computes the same split on the device)."""
import numpy as np
import pytest

from hy3_b200.attn import decode_schedule


@pytest.mark.parametrize("lens,heads,ctas", [([32768], 8, 148), ([1], 8, 148), ([128, 129, 0, 5000], 8, 148),
                                              ([1000] * 64, 4, 148), ([65536, 1024], 1, 7), ([0, 0], 8, 148),
                                              ([300] * 18, 8, 148), ([300] * 19, 8, 148), ([70000, 5], 8, 148),
                                              ([1024 + (7919 * i) % 64513 for i in range(64)], 1, 148), ([5000] * 16, 8, 148)])
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
    sizes = [b - a for a, b in ranges]
    if len(lens) * heads < ctas and ranges and max(sizes) - min(sizes) > 1:
        # the aligned split (whole CTAs per segment) was kept: nobody has more than 5/4 of the even share (+ 1 page)
        assert max(sizes) * 4 <= -(-total // ctas) * 5 + 4
        bounds = set()
        acc = 0
        for p in pages:
            for _ in range(heads):
                bounds.add(acc)
                acc += p
        for u0, u1 in ranges:
            assert not any(u0 < b < u1 for b in bounds), "a CTA straddles two segments"
    elif ranges and len(lens) * heads >= ctas:
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


def test_plan_eval_follows_the_reference_walk():
    """hy3_gpu.cu:857-889: with a chunk size and more than one token, all tokens but the last go through chunks; the
    position of the first token is cache_len / n_layers."""
    from hy3_b200.session import plan_eval, read_env
    assert plan_eval(0, 3, 80, 0) == [("token", 0), ("token", 1), ("token", 2)]
    assert plan_eval(160, 1300, 80, 512) == [("chunk", 2, 512), ("chunk", 514, 512), ("chunk", 1026, 275), ("token", 1301)]
    assert plan_eval(80, 1, 80, 512) == [("token", 1)]                     # a single token never takes the chunk path
    assert plan_eval(0, 2, 80, 512) == [("chunk", 0, 1), ("token", 1)]
    assert plan_eval(0, 513, 2, 512) == [("chunk", 0, 512), ("token", 512)]
    e = read_env({"HY3_KV_INT4": "1", "HY3_PREFILL_CHUNK": "abc", "HY3_POS_STRIDE": "-3", "HY3_POS_JUMP": "7"})
    assert e == {"kv_dtype": "int4", "chunk": 0, "pos_stride": 1, "pos_jump": 7, "pos_jump_at": 0}
    assert read_env({})["kv_dtype"] == "int8" and read_env({"HY3_KV_FP16": "1"})["kv_dtype"] == "fp16"
