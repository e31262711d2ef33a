"""GPU parity of the tcgen05 chunk-prefill attention (through the C ABI) against the oracle's causal
prefill -- one decode attention per query over the keys [0, base+i] (restatement of hy3_gpu.cu:379-412 /
hy3.c:617-652) -- evaluated on the SAME stored K/V and the same fp16 queries."""
import numpy as np
import pytest

from helpers import SEED, check_attention, slots_to_float

pytestmark = pytest.mark.gpu


def run_case(cuda, oracle, dt, base, nq, rows=None, eps=1e-6):
    import torch
    from hy3_b200 import Hy3Attn
    ntok = base + nq
    ctx = Hy3Attn(kv_dtype=dt, n_layers=2, max_batch=max(nq, base, 1), max_tokens=ntok + 256, rms_eps=eps)
    w = (1.0 + 0.02 * oracle.fill_normal((2, 128), SEED, 3)).astype(np.float32)
    ctx.set_norm_weights(1, w[0], w[1])
    q = oracle.fill_normal((ntok, 64, 128), SEED, 501)
    k = oracle.fill_normal((ntok, 8, 128), SEED, 502)
    v = oracle.fill_normal((ntok, 8, 128), SEED, 503)
    tq, tk, tv = (torch.from_numpy(a).to(cuda) for a in (q, k, v))
    if base:                                                  # an earlier turn / earlier chunks
        ctx.batch_set([0] * base, list(range(base)))
        ctx.append(1, tq[:base], tk[:base], tv[:base])
    ctx.batch_set([0] * nq, list(range(base, ntok)))
    q16 = torch.empty((nq, 64, 128), dtype=torch.float16, device=cuda)
    ctx.append(1, tq[base:], tk[base:], tv[base:], q_out16=q16)
    out = ctx.prefill(1, 0, base, q16)
    ctx.sync()
    ks, vs = ctx.export_kv(1, 0, 0, ntok)
    Kf, Vf = slots_to_float(oracle, ks, dt), slots_to_float(oracle, vs, dt)
    qf = q16.float().cpu().numpy()
    out = out.cpu().numpy()
    rows = list(range(nq)) if rows is None else rows
    want = oracle.prefill_causal(qf, Kf, Vf, base, rows=rows)
    worst = 0.0
    for i in rows:
        err, _ = check_attention(out[i], want[i], "%s base=%d nq=%d row %d" % (dt, base, nq, i))
        worst = max(worst, err)
    ctx.close()
    return worst


@pytest.mark.parametrize("dt", ["fp16", "int8", "int4"])
@pytest.mark.parametrize("base,nq", [(0, 1), (0, 16), (0, 40), (0, 129), (100, 28), (127, 130), (256, 256)])
def test_prefill_small(cuda, oracle, dt, base, nq):
    worst = run_case(cuda, oracle, dt, base, nq)
    print("prefill %s base=%d nq=%d worst max-abs %.3g" % (dt, base, nq, worst))


@pytest.mark.parametrize("dt", ["fp16", "int8"])
def test_prefill_chunk_over_prefix(cuda, oracle, dt):
    """A 512-token chunk on top of a 1536-token prefix; sampled rows at the chunk and tile boundaries."""
    run_case(cuda, oracle, dt, 1536, 512, rows=[0, 1, 15, 16, 127, 128, 255, 256, 500, 511])


def _chunked(cuda, oracle, dt, chunks, mirror_mb, monkeypatch, redo=None):
    """Feeds `chunks` (token counts) one after the other through append + prefill on ONE context; `redo` =
    (keep_ntok, n): after the last chunk the sequence is cut back to keep_ntok tokens and n DIFFERENT tokens follow.
    Returns the outputs of all prefill calls and the exported cache."""
    import torch
    from hy3_b200 import Hy3Attn
    if mirror_mb is None:
        monkeypatch.delenv("HY3A_PF_MIRROR_MB", raising=False)
    else:
        monkeypatch.setenv("HY3A_PF_MIRROR_MB", str(mirror_mb))
    total = sum(chunks)
    ctx = Hy3Attn(kv_dtype=dt, n_layers=2, max_batch=max(max(chunks), (redo or (0, 1))[1]), max_tokens=total + 512)
    q = oracle.fill_normal((total + 512, 64, 128), SEED, 511)
    k = oracle.fill_normal((total + 512, 8, 128), SEED, 512)
    v = oracle.fill_normal((total + 512, 8, 128), SEED, 513)
    tq, tk, tv = (torch.from_numpy(a).to(cuda) for a in (q, k, v))
    outs, base = [], 0
    steps = [(c, 0) for c in chunks]
    for n, shift in steps + ([(redo[1], 256)] if redo else []):
        if shift:                                            # cut back, then other tokens at the same slots
            base = redo[0]
            ctx.seq_release(0, base)
        ctx.batch_set([0] * n, list(range(base, base + n)))
        q16 = torch.empty((n, 64, 128), dtype=torch.float16, device=cuda)
        src = slice(base + shift, base + shift + n)
        ctx.append(1, tq[src], tk[src], tv[src], q_out=False, q_out16=q16)
        out = ctx.prefill(1, 0, base, q16)
        ctx.sync()
        outs.append((base, n, q16.float().cpu().numpy(), out.cpu().numpy()))
        base += n
    ks, vs = ctx.export_kv(1, 0, 0, base)
    ctx.close()
    return outs, ks, vs


@pytest.mark.parametrize("dt", ["fp16", "int8"])
def test_prefill_chunks_reuse_converted_pages(cuda, oracle, dt, monkeypatch):
    """Successive chunks convert only the pages they appended (the per-layer fp16 operand mirror).  The outputs must
    equal, bit for bit, those of a context that rebuilds the operands on every call, and must match the oracle also
    after the sequence was cut back and continued with different tokens (a stale mirror would show there)."""
    chunks, redo = [100, 156, 300, 84, 200], (300, 170)
    a, ks, vs = _chunked(cuda, oracle, dt, chunks, None, monkeypatch, redo)
    b, ks0, vs0 = _chunked(cuda, oracle, dt, chunks, 0, monkeypatch, redo)
    assert np.array_equal(ks, ks0) and np.array_equal(vs, vs0)
    for (base, n, _, oa), (_, _, _, ob) in zip(a, b):
        assert np.array_equal(oa, ob), "chunk at %d differs between mirrored and rebuilt operands" % base
    # oracle: the last call (after the cut) sees exactly the exported cache
    base, n, qf, out = a[-1]
    Kf, Vf = slots_to_float(oracle, ks, dt), slots_to_float(oracle, vs, dt)
    rows = [0, 1, 27, 28, 100, n - 1]
    want = oracle.prefill_causal(qf, Kf, Vf, base, rows=rows)
    for i in rows:
        check_attention(out[i], want[i], "%s after cut: base=%d row %d" % (dt, base, i))
    # and one call before the cut, against the cache as it was then = the same slots below its end (those below the
    # cut were not rewritten; only check a chunk that ends at or below the cut)
    base, n, qf, out = a[1]
    assert base + n <= redo[0]
    want = oracle.prefill_causal(qf, Kf, Vf, base, rows=[0, n - 1])
    for i in (0, n - 1):
        check_attention(out[i], want[i], "%s before cut: base=%d row %d" % (dt, base, i))


@pytest.mark.parametrize("dt", ["fp16", "int8"])
def test_append_twice_refreshes_operands(cuda, oracle, dt):
    """The same batch appended a second time with other K/V (no new hy3a_batch_set in between): the chunk attention
    must see the second version, i.e. the kept fp16 operands of the layer may not go stale."""
    import torch
    from hy3_b200 import Hy3Attn
    n = 200
    ctx = Hy3Attn(kv_dtype=dt, n_layers=1, max_batch=n, max_tokens=512)
    q = oracle.fill_normal((n, 64, 128), SEED, 901)
    kv = [(oracle.fill_normal((n, 8, 128), SEED, 902 + 2 * i), oracle.fill_normal((n, 8, 128), SEED, 903 + 2 * i)) for i in range(2)]
    tq = torch.from_numpy(q).to(cuda)
    q16 = torch.empty((n, 64, 128), dtype=torch.float16, device=cuda)
    ctx.batch_set([0] * n, list(range(n)))
    for k, v in kv:
        ctx.append(0, tq, torch.from_numpy(k).to(cuda), torch.from_numpy(v).to(cuda), q_out=False, q_out16=q16)
        out = ctx.prefill(0, 0, 0, q16)
    ctx.sync()
    ks, vs = ctx.export_kv(0, 0, 0, n)
    rows = [0, 1, 100, n - 1]
    want = oracle.prefill_causal(q16.float().cpu().numpy(), slots_to_float(oracle, ks, dt), slots_to_float(oracle, vs, dt), 0, rows=rows)
    out = out.cpu().numpy()
    for i in rows:
        check_attention(out[i], want[i], "%s second append, row %d" % (dt, i))
    ctx.close()
