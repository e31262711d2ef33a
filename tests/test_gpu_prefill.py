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
