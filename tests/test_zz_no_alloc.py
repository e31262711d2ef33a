"""hy3a_decode_noalloc: the decode entry point whose merge scratch is a fixed array inside the library.

It is meant for callers that cannot allocate device memory on the decode path (the allocator is locked
or drained by someone else, or an allocation's implicit synchronisation is not acceptable).  The test
calls it through the C ABI twice in a row and compares each result with hy3a_decode on the same
context and inputs; the two share every kernel instruction, so the outputs must agree to the tolerance
the other decode tests use (in practice bit for bit).  It also checks the documented limit from both sides: a
batch of 8 rows x 8 KV heads (the 64 segments the built-in scratch covers) is served, 9 rows are refused, and a
context that owns 2 of the 8 KV heads works the same way.
"""
import numpy as np
import pytest

from helpers import ATTN_TOL, SEED, check_attention, make_slots, slots_to_float

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", ["int8", "fp16"])
def test_noalloc_matches_decode_twice(cuda, oracle, dt):
    import torch
    from hy3_b200 import Hy3Attn
    lens = [5000, 129, 1]                      # long enough that segments span many CTAs (the scratch is used)
    B = len(lens)
    ctx = Hy3Attn(kv_dtype=dt, n_layers=1, max_seqs=B, max_batch=16, max_tokens=8192, max_tokens_per_seq=5120)
    K = [oracle.fill_normal((n, 8, 128), SEED, 700 + i) for i, n in enumerate(lens)]
    V = [oracle.fill_normal((n, 8, 128), SEED, 800 + i) for i, n in enumerate(lens)]
    for s in range(B):
        ctx.import_kv(0, s, 0, make_slots(oracle, K[s], dt), make_slots(oracle, V[s], dt))
    ctx.batch_set(list(range(B)), [n - 1 for n in lens])
    for call in range(2):
        q = oracle.fill_normal((B, 64, 128), SEED, 900 + call)
        tq = torch.from_numpy(q).to(cuda)
        want = ctx.decode(0, tq)
        got = torch.full((B, 64, 128), float("nan"), dtype=torch.float32, device=cuda)
        rc = ctx.lib.hy3a_decode_noalloc(ctx.h, 0, tq.data_ptr(), tq.stride(0), got.data_ptr(), got.stride(0))
        assert rc == 0, ctx.lib.hy3a_last_error(ctx.h)
        ctx.sync()
        got, want = got.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= ATTN_TOL, "call %d: %.3g" % (call, np.abs(got - want).max())
        for s in range(B):
            Kf = slots_to_float(oracle, make_slots(oracle, K[s], dt), dt)
            Vf = slots_to_float(oracle, make_slots(oracle, V[s], dt), dt)
            check_attention(got[s], oracle.attention(q[s], Kf, Vf), "noalloc %s call %d seq %d" % (dt, call, s))
    # more (row, KV head) pairs than the built-in scratch covers -> a clear refusal, not a launch
    ctx.batch_set([0] * 9, [10] * 9)
    q9 = torch.zeros((9, 64, 128), dtype=torch.float32, device=cuda)
    rc = ctx.lib.hy3a_decode_noalloc(ctx.h, 0, q9.data_ptr(), q9.stride(0), q9.data_ptr(), q9.stride(0))
    assert rc == -1 and b"exceed the built-in scratch" in ctx.lib.hy3a_last_error(ctx.h)
    ctx.close()


def _compare_with_decode(ctx, cuda, B, seed):
    import torch
    from hy3_b200.attn import H
    q = torch.randn((B, H, 128), dtype=torch.float32, device=cuda, generator=torch.Generator(device=cuda).manual_seed(seed))
    want = ctx.decode(0, q)
    got = torch.full((B, H, 128), float("nan"), dtype=torch.float32, device=cuda)
    rc = ctx.lib.hy3a_decode_noalloc(ctx.h, 0, q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0))
    assert rc == 0, ctx.lib.hy3a_last_error(ctx.h)
    ctx.sync()
    return got.cpu().numpy(), want.cpu().numpy()


def test_noalloc_at_the_documented_limit(cuda):
    """8 rows x 8 KV heads = 64 segments, the most the built-in scratch holds; one row is long, so its segments are
    split over several CTAs and the highest record indices are used.  Two calls in a row."""
    from hy3_b200 import Hy3Attn
    lens = [6000, 300, 129, 128, 127, 17, 2, 1]
    B = len(lens)
    ctx = Hy3Attn(kv_dtype="int8", n_layers=1, max_seqs=B, max_batch=B, max_tokens=sum(lens) + 128 * B, max_tokens_per_seq=6144)
    for s, n in enumerate(lens):
        ctx.fill_random(0, s, 0, n, 40 + s)
    ctx.batch_set(list(range(B)), [n - 1 for n in lens])
    for call in range(2):
        got, want = _compare_with_decode(ctx, cuda, B, 100 + call)
        assert np.isfinite(got).all() and np.abs(got - want).max() <= ATTN_TOL
    ctx.close()


def test_noalloc_on_a_kv_head_shard(cuda):
    """A context that owns KV heads 4 and 5 only: the owned 16 query heads agree with hy3a_decode, the others stay untouched."""
    from hy3_b200 import Hy3Attn
    ctx = Hy3Attn(kv_dtype="int8", n_layers=1, kv_head_begin=4, kv_head_count=2, max_seqs=2, max_batch=2, max_tokens=8192, max_tokens_per_seq=5120)
    lens = [5000, 200]
    for s, n in enumerate(lens):
        ctx.fill_random(0, s, 0, n, 60 + s)
    ctx.batch_set([0, 1], [n - 1 for n in lens])
    for call in range(2):
        got, want = _compare_with_decode(ctx, cuda, 2, 200 + call)
        own = slice(32, 48)
        assert np.isfinite(got[:, own]).all() and np.abs(got[:, own] - want[:, own]).max() <= ATTN_TOL
        assert np.isnan(got[:, :32]).all() and np.isnan(got[:, 48:]).all()
    ctx.close()
