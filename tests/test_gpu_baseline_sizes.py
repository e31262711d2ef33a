"""GPU parity at the sizes of the benchmark configurations themselves (the other test files use reduced sizes):

 - chunked prefill of an 8192-token prompt in 512-token chunks on an FP16 cache, 128 key tiles per CTA in the last
   chunk, plus the multi-turn case (4096 cached tokens, 2 x 512 new ones) on FP16 and INT8 caches;
 - decode with an INT4 cache, YaRN factor 4, 262 144 positions, the new token appended by the fused step;
 - the seeded ragged batch of 64 sequences (lengths 1024 .. 65 536) on an INT8 cache.

The oracle is evaluated on the cache as stored (exported in the reference's slot format), on sampled rows /
sequences so that it finishes in seconds.  Causal definition: hy3_gpu.cu:379-412; attention: hy3.c:617-652.
"""
import numpy as np
import pytest

from helpers import SEED, check_attention, slots_to_float

pytestmark = pytest.mark.gpu

ROWS = [0, 1, 15, 16, 511]


def _feed(ctx, torch, cuda, oracle, layer, t0, n, seed_off, want_out):
    """Append tokens [t0, t0+n) (seeded) and, if want_out, run the chunk attention; returns (q16, out) as numpy."""
    q = oracle.fill_normal((n, 64, 128), SEED, 7000 + seed_off)
    k = oracle.fill_normal((n, 8, 128), SEED, 8000 + seed_off)
    v = oracle.fill_normal((n, 8, 128), SEED, 9000 + seed_off)
    ctx.batch_set([0] * n, list(range(t0, t0 + n)))
    q16 = torch.empty((n, 64, 128), dtype=torch.float16, device=cuda)
    ctx.append(layer, *(torch.from_numpy(a).to(cuda) for a in (q, k, v)), q_out=False, q_out16=q16)
    if not want_out:
        return None
    out = ctx.prefill(layer, 0, t0, q16)
    ctx.sync()
    return q16.float().cpu().numpy(), out.cpu().numpy()


def test_prefill_8192_in_512_chunks_fp16(cuda, oracle):
    import torch
    from hy3_b200 import Hy3Attn
    prompt, chunk = 8192, 512
    ctx = Hy3Attn(kv_dtype="fp16", n_layers=1, max_batch=chunk, max_tokens=prompt + 256)
    keep = {}
    for c in range(prompt // chunk):
        r = _feed(ctx, torch, cuda, oracle, 0, c * chunk, chunk, c, True)
        if c in (0, 1, 8, 15):
            keep[c] = r
    ks, vs = ctx.export_kv(0, 0, 0, prompt)
    ctx.close()
    Kf, Vf = slots_to_float(oracle, ks, "fp16"), slots_to_float(oracle, vs, "fp16")
    worst = 0.0
    for c, (qf, out) in keep.items():
        rows = list(range(chunk)) if c == 0 else ROWS
        want = oracle.prefill_causal(qf, Kf, Vf, c * chunk, rows=rows)
        for i in rows:
            worst = max(worst, check_attention(out[i], want[i], "chunk %d row %d (global %d)" % (c, i, c * chunk + i))[0])
    print("prefill 8192/512 fp16: worst max-abs %.3g" % worst)


@pytest.mark.parametrize("dt", ["fp16", "int8"])
def test_prefill_multiturn_4096_plus_1024(cuda, oracle, dt):
    """A cached prefix of 4096 tokens (appended, never attended: an earlier turn), then 1024 new tokens in two chunks."""
    import torch
    from hy3_b200 import Hy3Attn
    prefix, chunk = 4096, 512
    ctx = Hy3Attn(kv_dtype=dt, n_layers=1, max_batch=chunk, max_tokens=prefix + 2 * chunk + 256)
    for c in range(prefix // chunk):
        _feed(ctx, torch, cuda, oracle, 0, c * chunk, chunk, c, False)
    res = [_feed(ctx, torch, cuda, oracle, 0, prefix + j * chunk, chunk, 100 + j, True) for j in range(2)]
    ks, vs = ctx.export_kv(0, 0, 0, prefix + 2 * chunk)
    ctx.close()
    Kf, Vf = slots_to_float(oracle, ks, dt), slots_to_float(oracle, vs, dt)
    for j, (qf, out) in enumerate(res):
        want = oracle.prefill_causal(qf, Kf, Vf, prefix + j * chunk, rows=ROWS)
        for i in ROWS:
            check_attention(out[i], want[i], "%s multi-turn chunk %d row %d" % (dt, j, i))


def test_decode_int4_yarn4_262144(cuda, oracle):
    import torch
    from hy3_b200 import Hy3Attn
    n = 262144
    ctx = Hy3Attn(kv_dtype="int4", n_layers=1, max_batch=1, max_tokens=n + 256)
    inv, af = oracle.rope_table(yarn=1, factor=4.0)
    ctx.set_rope(inv, af)
    ctx.fill_random(0, 0, 0, n - 1, 4242)
    q = oracle.fill_normal((1, 64, 128), SEED, 71)
    k = oracle.fill_normal((1, 8, 128), SEED, 72)
    v = oracle.fill_normal((1, 8, 128), SEED, 73)
    ctx.batch_set([0], [n - 1])
    qo = torch.empty((1, 64, 128), dtype=torch.float32, device=cuda)
    out = ctx.decode_step(0, *(torch.from_numpy(a).to(cuda) for a in (q, k, v)), q_out=qo)
    ctx.sync()
    ks, vs = ctx.export_kv(0, 0, 0, n)
    ctx.close()
    qr = qo[0].cpu().numpy()
    oq, _ = oracle.qk_norm_rope(q[0], k[0], np.ones(128, np.float32), np.ones(128, np.float32), 1e-5, n - 1, inv, af)
    assert (np.abs(qr - oq) <= 2e-5 * np.maximum(1.0, np.abs(oq))).all(), "rotated query at position %d" % (n - 1)
    Kf, Vf = slots_to_float(oracle, ks, "int4"), slots_to_float(oracle, vs, "int4")
    want = oracle.attention_f64(qr, Kf, Vf).astype(np.float32)
    err, rel = check_attention(out[0].cpu().numpy(), want, "int4 yarn4 ntok=%d" % n)
    print("decode int4 + YaRN x4 at %d positions: max-abs %.3g rel-rms %.3g" % (n, err, rel))


def test_decode_ragged_batch_of_64(cuda, oracle):
    """The seeded batch bench.py measures: 64 sequences, lengths 1024 + (rng % 64513); three of them are checked."""
    import torch
    from hy3_b200 import Hy3Attn
    rng = np.random.default_rng(SEED)
    lens = [int(1024 + rng.integers(0, 64513)) for _ in range(64)]
    B = len(lens)
    ctx = Hy3Attn(kv_dtype="int8", n_layers=1, max_seqs=B, max_batch=B, max_tokens=sum(lens) + 256 * B,
                  max_tokens_per_seq=max(lens) + 256)
    for i, n in enumerate(lens):
        ctx.fill_random(0, i, 0, n, SEED + i)
    q = oracle.fill_normal((B, 64, 128), SEED, 81)
    k = oracle.fill_normal((B, 8, 128), SEED, 82)
    v = oracle.fill_normal((B, 8, 128), SEED, 83)
    ctx.batch_set(list(range(B)), lens)                      # the new token of sequence i goes to slot lens[i]
    qo = torch.empty((B, 64, 128), dtype=torch.float32, device=cuda)
    out = ctx.decode_step(0, *(torch.from_numpy(a).to(cuda) for a in (q, k, v)), q_out=qo)
    ctx.sync()
    out, qo = out.cpu().numpy(), qo.cpu().numpy()
    assert np.isfinite(out).all()
    order = np.argsort(lens)
    for i in (int(order[0]), int(order[B // 2]), int(order[-1])):
        ks, vs = ctx.export_kv(0, i, 0, lens[i] + 1)
        want = oracle.attention_f64(qo[i], slots_to_float(oracle, ks, "int8"), slots_to_float(oracle, vs, "int8")).astype(np.float32)
        check_attention(out[i], want, "ragged batch seq %d len %d" % (i, lens[i] + 1))
    ctx.close()
