"""hy3a_decode_noalloc: the decode entry point whose merge scratch is a fixed array inside the library.

It is meant for callers that cannot allocate device memory on the decode path (the allocator is locked
or drained by someone else, or an allocation's implicit synchronisation is not acceptable).  The test
calls it through the C ABI twice in a row and compares each result with hy3a_decode on the same
context and inputs; the two share every kernel instruction, so the outputs must agree to the tolerance
the other decode tests use (in practice bit for bit).  It also checks that oversize batches are refused.
Collected last on purpose, so that a failure here cannot hide the other GPU tests behind `-x`.
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
