"""GPU parity of the split-KV GQA decode kernel (and its LSE-merge epilogue) through the C ABI,
against the oracle attention (restatement of hy3.c:617-652) evaluated on the same stored K/V."""
import numpy as np
import pytest

from helpers import SEED, check_attention, make_slots, slots_to_float

pytestmark = pytest.mark.gpu

LENS = [1, 2, 7, 8, 9, 15, 16, 17, 31, 32, 33, 127, 128, 129, 255, 256, 257, 1000, 4097]


def load_cache(ctx, oracle, dt, layer, seq, K, V):
    ks, vs = make_slots(oracle, K, dt), make_slots(oracle, V, dt)
    ctx.import_kv(layer, seq, 0, ks, vs)
    return slots_to_float(oracle, ks, dt), slots_to_float(oracle, vs, dt)


@pytest.fixture(params=["staged", "direct"])
def variant(request, monkeypatch):
    """The two load paths of the decode kernel: bulk-copy ring in shared memory, or direct 128-bit loads."""
    monkeypatch.delenv("HY3A_DECODE_STAGES", raising=False)
    if request.param == "direct":
        monkeypatch.setenv("HY3A_DECODE_STAGES", "0")
    return request.param


@pytest.mark.parametrize("dt", ["int8", "int4", "fp16"])
def test_decode_lengths(cuda, oracle, dt, variant):
    import torch
    from hy3_b200 import Hy3Attn
    nmax = max(LENS)
    ctx = Hy3Attn(kv_dtype=dt, n_layers=3, max_batch=4, max_tokens=nmax + 256)
    K = oracle.fill_normal((nmax, 8, 128), SEED, 51)
    V = oracle.fill_normal((nmax, 8, 128), SEED, 52)
    Kf, Vf = load_cache(ctx, oracle, dt, 2, 0, K, V)
    ks, vs = ctx.export_kv(2, 0, 0, nmax)          # import/export round trip is the identity
    assert np.array_equal(ks, make_slots(oracle, K, dt)) and np.array_equal(vs, make_slots(oracle, V, dt))
    q = oracle.fill_normal((64, 128), SEED, 53)
    tq = torch.from_numpy(q[None]).to(cuda)
    worst = 0.0
    for n in LENS:
        ctx.batch_set([0], [n - 1])
        out = ctx.decode(2, tq)
        ctx.sync()
        err, _ = check_attention(out[0].cpu().numpy(), oracle.attention(q, Kf[:n], Vf[:n]), "%s ntok=%d" % (dt, n))
        worst = max(worst, err)
    print("decode %s worst max-abs vs oracle-on-stored-KV: %.3g" % (dt, worst))
    ctx.close()


@pytest.mark.parametrize("dt", ["int8", "int4", "fp16"])
def test_decode_long_context_many_ctas(cuda, oracle, dt, variant):
    """Long enough that every CTA gets work and (row, head) segments span many CTAs (merge epilogue)."""
    import torch
    from hy3_b200 import Hy3Attn
    n = 40000
    ctx = Hy3Attn(kv_dtype=dt, n_layers=1, max_batch=2, max_tokens=n + 128)
    K = oracle.fill_normal((n, 8, 128), SEED, 61)
    V = oracle.fill_normal((n, 8, 128), SEED, 62)
    Kf, Vf = load_cache(ctx, oracle, dt, 0, 0, K, V)
    q = 1.5 * oracle.fill_normal((64, 128), SEED, 63)
    tq = torch.from_numpy(q[None]).to(cuda)
    ctx.batch_set([0], [n - 1])
    for _ in range(3):                              # repeated launches reuse the self-resetting counters
        out = ctx.decode(0, tq)
    ctx.sync()
    want = oracle.attention_f64(q, Kf, Vf).astype(np.float32)
    check_attention(out[0].cpu().numpy(), want, "%s ntok=%d" % (dt, n))
    ctx.close()


@pytest.mark.parametrize("dt", ["fp16", "int4", "int8"])
def test_decode_is_bitwise_repeatable(cuda, dt):
    """The same launch repeated back to back gives the same bits: fold orders are fixed, and no warp may read a ring stage
    that is still being filled (FP16 pages leave room for a two-stage ring only; a consumer warp that holds no granule of
    a page used to be able to pass its next wait on a stale barrier phase there)."""
    import torch
    from hy3_b200 import Hy3Attn
    n = 40000
    ctx = Hy3Attn(kv_dtype=dt, n_layers=2, max_batch=2, max_tokens=n + 128)
    for l in range(2):
        ctx.fill_random(l, 0, 0, n, 3 + l)
    q = torch.randn((1, 64, 128), device=cuda, generator=torch.Generator(device=cuda).manual_seed(5))
    ctx.batch_set([0], [n - 1])
    ref = [ctx.decode(l, q).clone() for l in range(2)]
    torch.cuda.synchronize()
    differing = 0
    for _ in range(60):
        outs = [(l, ctx.decode(l, q)) for _ in range(3) for l in range(2)]
        torch.cuda.synchronize()
        differing += sum(0 if torch.equal(o, ref[l]) else 1 for l, o in outs)
    ctx.sync()
    ctx.close()
    assert differing == 0, "%d of 360 launches differ from the first" % differing


def test_decode_ragged_batch_and_poison(cuda, oracle):
    """Several sequences of different lengths in one launch; cache bytes past each length are poison."""
    import torch
    from hy3_b200 import Hy3Attn
    lens = [1, 130, 257, 1000, 77, 128, 3000]
    B = len(lens)
    ctx = Hy3Attn(kv_dtype="int8", n_layers=2, max_seqs=B, max_batch=B, max_tokens=sum(lens) + 128 * B, max_tokens_per_seq=4096)
    Kf, Vf = [], []
    for s, n in enumerate(lens):
        cap = (n + 127) // 128 * 128
        K = oracle.fill_normal((cap, 8, 128), SEED, 100 + s)
        V = oracle.fill_normal((cap, 8, 128), SEED, 200 + s)
        K[n:] = 1e4                                  # poison past the valid length (finite, huge)
        V[n:] = -1e4
        a, b = load_cache(ctx, oracle, "int8", 1, s, K, V)
        Kf.append(a[:n]); Vf.append(b[:n])
    q = oracle.fill_normal((B, 64, 128), SEED, 300)
    ctx.batch_set(list(range(B)), [n - 1 for n in lens])
    out = ctx.decode(1, torch.from_numpy(q).to(cuda))
    ctx.sync()
    out = out.cpu().numpy()
    for s in range(B):
        check_attention(out[s], oracle.attention(q[s], Kf[s], Vf[s]), "seq %d len %d" % (s, lens[s]))
    ctx.close()


def test_decode_many_segments_share_ctas(cuda, oracle):
    """More (row, KV head) segments than CTAs: every CTA walks through several segments and segments straddle CTAs
    (the equal-unit-range schedule); a fused step, so that the appends land in many different CTAs."""
    import torch
    from hy3_b200 import Hy3Attn
    rng = np.random.default_rng(7)
    lens0 = [int(x) for x in rng.integers(1, 900, size=40)]      # 320 segments for 148 CTAs
    lens0[3], lens0[17] = 0, 2600
    B = len(lens0)
    ctx = Hy3Attn(kv_dtype="int8", n_layers=1, max_seqs=B, max_batch=B, max_tokens=sum(lens0) + 256 * B, max_tokens_per_seq=4096)
    for s_, n0 in enumerate(lens0):
        if n0:
            ctx.fill_random(0, s_, 0, n0, 500 + s_)
    q = oracle.fill_normal((2, B, 64, 128), SEED, 331)
    k = oracle.fill_normal((2, B, 8, 128), SEED, 332)
    v = oracle.fill_normal((2, B, 8, 128), SEED, 333)
    tq, tk, tv = (torch.from_numpy(x).to(cuda) for x in (q, k, v))
    qo = torch.zeros((B, 64, 128), dtype=torch.float32, device=cuda)
    for t in range(2):
        ctx.batch_set(list(range(B)), [n0 + t for n0 in lens0])
        out = ctx.decode_step(0, tq[t], tk[t], tv[t], q_out=qo)
    ctx.sync()
    out, qo = out.cpu().numpy(), qo.cpu().numpy()
    for s_ in range(B):
        ks, vs = ctx.export_kv(0, s_, 0, lens0[s_] + 2)
        check_attention(out[s_], oracle.attention(qo[s_], slots_to_float(oracle, ks, "int8"), slots_to_float(oracle, vs, "int8")), "seq %d len %d" % (s_, lens0[s_] + 2))
    ctx.close()


def test_append_then_decode_end_to_end(cuda, oracle):
    """The real step: fused append of token t, then attention over [0, t], for a few steps."""
    import torch
    from hy3_b200 import Hy3Attn
    steps, eps = 140, 1e-6
    ctx = Hy3Attn(kv_dtype="int8", n_layers=1, max_batch=1, max_tokens=512, rms_eps=eps)
    w = (1.0 + 0.02 * oracle.fill_normal((2, 128), SEED, 3)).astype(np.float32)
    ctx.set_norm_weights(0, w[0], w[1])
    inv, af = oracle.rope_table()
    q = oracle.fill_normal((steps, 64, 128), SEED, 71)
    k = oracle.fill_normal((steps, 8, 128), SEED, 72)
    v = oracle.fill_normal((steps, 8, 128), SEED, 73)
    tq, tk, tv = (torch.from_numpy(a).to(cuda) for a in (q, k, v))
    outs = []
    for t in range(steps):
        ctx.batch_set([0], [t])
        qo = ctx.append(0, tq[t:t + 1], tk[t:t + 1], tv[t:t + 1])
        outs.append((qo, ctx.decode(0, qo)))
    ctx.sync()
    ks, vs = ctx.export_kv(0, 0, 0, steps)
    Kf, Vf = slots_to_float(oracle, ks, "int8"), slots_to_float(oracle, vs, "int8")
    for t in (0, 1, 15, 16, 127, 128, 139):
        qo, out = outs[t]
        oq, ok = oracle.qk_norm_rope(q[t], k[t], w[0], w[1], eps, t, inv, af)
        # the cache holds exactly what the oracle pipeline would have stored (K within +-1 code of ulp effects)
        want_k = oracle.stored_kv(ok, "int8")
        assert np.abs(Kf[t] - want_k).max() <= 1.01 * np.abs(ok).max() / 127
        check_attention(out[0].cpu().numpy(), oracle.attention(qo[0].cpu().numpy(), Kf[:t + 1], Vf[:t + 1]), "step %d" % t)
        # against the un-quantised fp32 pipeline: report the INT8 bound separately
    t = steps - 1
    oq_all = [oracle.qk_norm_rope(q[i], k[i], w[0], w[1], eps, i, inv, af) for i in range(steps)]
    K32 = np.stack([x[1] for x in oq_all])
    full = oracle.attention(oq_all[t][0], K32, v)
    err = np.abs(outs[t][1][0].cpu().numpy() - full).max()
    print("INT8 KV end-to-end vs un-quantised fp32 pipeline at ntok=%d: max-abs %.3g" % (steps, err))
    assert err < 3e-2
    ctx.close()


@pytest.mark.parametrize("dt", ["int8", "int4", "fp16"])
def test_fused_step_equals_append_plus_decode(cuda, oracle, dt):
    """hy3a_decode_step (one kernel) against hy3a_append + hy3a_decode: identical cache bytes, identical
    queries, identical outputs; a ragged batch so that page and granule boundaries are crossed."""
    import torch
    from hy3_b200 import Hy3Attn
    lens0 = [0, 15, 16, 127, 128, 300, 2000]          # tokens already cached per sequence
    B, steps = len(lens0), 18
    w = (1.0 + 0.02 * oracle.fill_normal((2, 128), SEED, 3)).astype(np.float32)
    q = oracle.fill_normal((steps, B, 64, 128), SEED, 401)
    k = oracle.fill_normal((steps, B, 8, 128), SEED, 402)
    v = oracle.fill_normal((steps, B, 8, 128), SEED, 403)
    res = {}
    for mode in ("two_kernels", "fused"):
        ctx = Hy3Attn(kv_dtype=dt, n_layers=2, max_seqs=B, max_batch=B, max_tokens=4096 + 128 * B, max_tokens_per_seq=2560, rms_eps=1e-6)
        ctx.set_norm_weights(1, w[0], w[1])
        for s_, n0 in enumerate(lens0):
            if n0:
                ctx.fill_random(1, s_, 0, n0, 77)
        outs, qos = [], []
        tq, tk, tv = (torch.from_numpy(a).to(cuda) for a in (q, k, v))
        for t in range(steps):
            ctx.batch_set(list(range(B)), [n0 + t for n0 in lens0], [n0 + t + 5 for n0 in lens0])
            if mode == "fused":
                qo = torch.zeros((B, 64, 128), dtype=torch.float32, device=cuda)
                out = ctx.decode_step(1, tq[t], tk[t], tv[t], q_out=qo)
            else:
                qo = ctx.append(1, tq[t], tk[t], tv[t])
                out = ctx.decode(1, qo)
            outs.append(out); qos.append(qo)
        ctx.sync()
        caches = [ctx.export_kv(1, s_, 0, n0 + steps) for s_, n0 in enumerate(lens0)]
        res[mode] = (torch.stack(outs).cpu().numpy(), torch.stack(qos).cpu().numpy(), caches)
        if mode == "fused":        # and against the oracle on the stored cache, last step
            for s_ in (0, 3, 6):
                Kf = slots_to_float(oracle, caches[s_][0], dt); Vf = slots_to_float(oracle, caches[s_][1], dt)
                check_attention(res[mode][0][-1, s_], oracle.attention(res[mode][1][-1, s_], Kf, Vf), "fused %s seq %d" % (dt, s_))
        ctx.close()
    a, b = res["two_kernels"], res["fused"]
    assert np.array_equal(a[1], b[1]), "queries differ"
    for (ka, va), (kb, vb) in zip(a[2], b[2]):
        assert np.array_equal(ka, kb) and np.array_equal(va, vb), "cache bytes differ"
    assert np.array_equal(a[0], b[0]), "outputs differ: max %.3g" % np.abs(a[0] - b[0]).max()


def test_partials_and_merge_sequence_shards(cuda, oracle):
    """Two contexts hold the two halves of one sequence; per-shard {m,l,acc} + merge == full attention."""
    import torch
    from hy3_b200 import Hy3Attn
    n, cut = 3000, 1700
    K = oracle.fill_normal((n, 8, 128), SEED, 81)
    V = oracle.fill_normal((n, 8, 128), SEED, 82)
    q = oracle.fill_normal((2, 64, 128), SEED, 83)
    tq = torch.from_numpy(q).to(cuda)
    parts, Kf, Vf = [], [], []
    ctxs = []
    for lo, hi in ((0, cut), (cut, n)):
        ctx = Hy3Attn(kv_dtype="int8", n_layers=1, max_seqs=2, max_batch=2, max_tokens=2 * n, max_tokens_per_seq=n + 128)
        a, b = load_cache(ctx, oracle, "int8", 0, 0, K[lo:hi], V[lo:hi])
        Kf.append(a); Vf.append(b)
        ctx.batch_set([0, 1], [hi - lo - 1, -1])     # row 1: a sequence with no keys on this shard
        p = torch.empty((2, 64, 130), dtype=torch.float32, device=cuda)
        ctx.decode(0, tq, partials=p)
        ctx.sync()
        parts.append(p)
        ctxs.append(ctx)
    Kf, Vf = np.concatenate(Kf), np.concatenate(Vf)
    for r, (lo, hi) in enumerate(((0, cut), (cut, n))):
        got = parts[r][0].cpu().numpy()
        want = oracle.attention_partial(q[0], Kf, Vf, lo, hi)
        # same record up to the (m, l, acc) gauge: compare after normalising by the oracle's m
        f = np.exp(got[:, 0] - want[:, 0])
        assert np.allclose(got[:, 1] * f, want[:, 1], rtol=2e-3)
        assert np.abs(got[:, 2:] * f[:, None] - want[:, 2:]).max() <= 2e-3 * max(1.0, np.abs(want[:, 2:]).max())
        empty = parts[r][1].cpu().numpy()
        assert np.isneginf(empty[:, 0]).all() and not empty[:, 1:].any()
    allp = torch.stack(parts)                         # [2 shards][2 rows][64][130] == all-gather layout
    out = torch.zeros((2, 64, 128), dtype=torch.float32, device=cuda)
    ctxs[0].merge_partials(allp, 2, 2, 64, out)
    ctxs[0].sync()
    check_attention(out[0].cpu().numpy(), oracle.attention(q[0], Kf, Vf), "merged shards")
    assert not out[1].cpu().numpy().any()             # no keys anywhere -> zeros (hy3_gpu.cu:245)
    for c in ctxs:
        c.close()


def test_kv_head_shard_writes_only_its_heads(cuda, oracle):
    import torch
    from hy3_b200 import Hy3Attn
    n = 700
    K = oracle.fill_normal((n, 8, 128), SEED, 91)
    V = oracle.fill_normal((n, 8, 128), SEED, 92)
    q = oracle.fill_normal((1, 64, 128), SEED, 93)
    ctx = Hy3Attn(kv_dtype="int4", n_layers=1, kv_head_begin=2, kv_head_count=2, max_batch=1, max_tokens=1024)
    Kf, Vf = load_cache(ctx, oracle, "int4", 0, 0, K, V)
    ks, _ = ctx.export_kv(0, 0, 0, n)
    full = make_slots(oracle, K, "int4")
    assert np.array_equal(ks[:, 16 + 2 * 64:16 + 4 * 64], full[:, 16 + 2 * 64:16 + 4 * 64]) and not ks[:, 16:16 + 128].any()
    ctx.batch_set([0], [n - 1])
    out = torch.full((1, 64, 128), 7.0, dtype=torch.float32, device=cuda)
    ctx.decode(0, torch.from_numpy(q).to(cuda), out=out)
    ctx.sync()
    out = out.cpu().numpy()[0]
    want = oracle.attention(q[0], Kf, Vf)
    check_attention(out[16:32], want[16:32], "owned heads")
    assert (out[:16] == 7.0).all() and (out[32:] == 7.0).all()
    ctx.close()


@pytest.mark.parametrize("dt", ["int8", "int4"])
def test_one_kv_head_of_a_ragged_batch(cuda, oracle, dt):
    """A context that owns ONE KV head of 60 sequences (the KV-head shard of a ragged batch on 8 GPUs): fewer segments than
    CTAs, but so many that giving every segment whole CTAs would leave some CTAs with far more pages than others -- the
    kernel then takes the equal split over all units (CTAs straddle segments).  A fused step, checked per sequence."""
    import torch
    from hy3_b200 import Hy3Attn
    from hy3_b200.attn import decode_schedule
    rng = np.random.default_rng(11)
    lens0 = [int(x) for x in rng.integers(100, 6000, size=60)]
    B = len(lens0)
    # the host mirror of the schedule says: not the aligned split (ranges are equal to a page)
    sizes = [u1 - u0 for u0, u1 in (decode_schedule([n + 1 for n in lens0], 1, 148, c)[1:] for c in range(148))]
    assert max(sizes) - min(sizes) <= 1
    hb = 5
    ctx = Hy3Attn(kv_dtype=dt, n_layers=1, kv_head_begin=hb, kv_head_count=1, max_seqs=B, max_batch=B,
                  max_tokens=sum(lens0) + 256 * B, max_tokens_per_seq=8192)
    for s_, n0 in enumerate(lens0):
        ctx.fill_random(0, s_, 0, n0, 900 + s_)
    q = oracle.fill_normal((B, 64, 128), SEED, 431)
    k = oracle.fill_normal((B, 8, 128), SEED, 432)
    v = oracle.fill_normal((B, 8, 128), SEED, 433)
    tq, tk, tv = (torch.from_numpy(x).to(cuda) for x in (q, k, v))
    qo = torch.zeros((B, 64, 128), dtype=torch.float32, device=cuda)
    out = torch.full((B, 64, 128), 7.0, dtype=torch.float32, device=cuda)
    ctx.batch_set(list(range(B)), lens0)
    ctx.decode_step(0, tq, tk, tv, out=out, q_out=qo)
    ctx.sync()
    out, qo = out.cpu().numpy(), qo.cpu().numpy()
    assert (out[:, :8 * hb] == 7.0).all() and (out[:, 8 * hb + 8:] == 7.0).all()          # only the owned heads are written
    for s_ in range(0, B, 7):
        ks, vs = ctx.export_kv(0, s_, 0, lens0[s_] + 1)
        Kf, Vf = slots_to_float(oracle, ks, dt), slots_to_float(oracle, vs, dt)
        want = oracle.attention(qo[s_], Kf, Vf)
        check_attention(out[s_][8 * hb:8 * hb + 8], want[8 * hb:8 * hb + 8], "seq %d len %d" % (s_, lens0[s_] + 1))
    ctx.close()


def test_errors_are_codes_not_exits(cuda, oracle):
    import torch
    from hy3_b200 import Hy3Attn, Hy3AttnError
    ctx = Hy3Attn(kv_dtype="int8", n_layers=1, max_batch=2, max_tokens=256)
    q = torch.zeros((1, 64, 128), dtype=torch.float32, device=cuda)
    assert ctx.lib.hy3a_decode(ctx.h, 0, q.data_ptr(), 8192, q.data_ptr(), 8192, None) == -5   # no batch set
    with pytest.raises(Hy3AttnError) as e:
        ctx.batch_set([0], [100000])                    # beyond the pool
    assert e.value.code == -2
    with pytest.raises(Hy3AttnError):
        ctx.batch_set([3], [0])                         # sequence out of range
    ctx.batch_set([0], [5])
    with pytest.raises(Hy3AttnError):
        ctx._chk(ctx.lib.hy3a_decode(ctx.h, 9, q.data_ptr(), 8192, q.data_ptr(), 8192, None))  # bad layer
    ctx.close()
