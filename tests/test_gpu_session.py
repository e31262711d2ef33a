"""GPU test of EvalSession, the host mirror of the attention side of hy3_eval_gpu (hy3_gpu.cu:844-961): positions from
cache_len, chunked prompt ingest with the last token through the decode path, and a caller that sets cache_len back
to a reused prefix and continues with other tokens (hy3.c:1514).  Checked against the oracle on the exported cache."""
import io

import numpy as np
import pytest

from helpers import SEED, check_attention, slots_to_float

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv", ["int8", "fp16"])
def test_session_prompt_rollback_continue(cuda, oracle, kv):
    import torch
    from hy3_b200.session import EvalSession
    L, T = 2, 520
    inv, af = oracle.rope_table()
    w = (1.0 + 0.02 * oracle.fill_normal((L, 2, 128), SEED, 5)).astype(np.float32)
    data = {"q": oracle.fill_normal((L, T, 64, 128), SEED, 601), "k": oracle.fill_normal((L, T, 8, 128), SEED, 602),
            "v": oracle.fill_normal((L, T, 8, 128), SEED, 603)}
    dev = {n: torch.from_numpy(a).to(cuda) for n, a in data.items()}
    env = {"HY3_PREFILL_CHUNK": "128", "HY3_POS_STRIDE": "2"}
    if kv == "fp16":
        env["HY3_KV_FP16"] = "1"
    log = io.StringIO()
    s = EvalSession(n_layers=L, max_tokens=1024, inv_freq=inv, attn_factor=af, norm_weights=[(w[l, 0], w[l, 1]) for l in range(L)],
                    rms_eps=1e-5, env=env, log=log)
    assert "initialized (2 layers, %s KV, online attn)" % kv.upper() in log.getvalue() and "chunk=128" in log.getvalue()
    shift = [0]                                  # which stretch of the synthetic rows the "model" is fed from
    got = {}

    def qkv_fn(layer, t0, n):
        sl = slice(t0 + shift[0], t0 + shift[0] + n)
        return dev["q"][layer, sl], dev["k"][layer, sl], dev["v"][layer, sl]

    def out_fn(layer, t0, n, attn):
        got[(layer, t0, n)] = attn.clone()

    def check(layer, t, row_out, src_t, K, V):
        oq, _ = oracle.qk_norm_rope(data["q"][layer, src_t], data["k"][layer, src_t], w[layer, 0], w[layer, 1], 1e-5, t, inv, af, 2)
        oq = oq if kv != "fp16" else oq                       # decode attends with fp32 queries
        check_attention(row_out, oracle.attention(oq, K[:t + 1], V[:t + 1]), "%s layer %d token %d" % (kv, layer, t))

    # a 300-token prompt: chunks of 128, 128, 43 and the last token through the decode path
    assert s.eval(300, qkv_fn, out_fn) == 300 * L and s.cache_len == 300 * L
    s.ctx.sync()
    assert sorted(k for k in got if k[0] == 0) == [(0, 0, 128), (0, 128, 128), (0, 256, 43), (0, 299, 1)]
    for layer in range(L):
        ks, vs = s.ctx.export_kv(layer, 0, 0, 300)
        K, V = slots_to_float(oracle, ks, kv), slots_to_float(oracle, vs, kv)
        check(layer, 299, got[(layer, 299, 1)][0].cpu().numpy(), 299, K, V)
        # a row inside a chunk: same definition (query i attends keys 0..i); the chunk's queries are fp16-rounded
        oq, _ = oracle.qk_norm_rope(data["q"][layer, 200], data["k"][layer, 200], w[layer, 0], w[layer, 1], 1e-5, 200, inv, af, 2)
        q16 = oq.astype(np.float16).astype(np.float32)
        check_attention(got[(layer, 128, 128)][72].cpu().numpy(), oracle.attention(q16, K[:201], V[:201]), "chunk row 200")
    # the caller reuses the first 100 tokens and continues with 60 other tokens (rows 350.. of the synthetic data)
    got.clear()
    s.cache_len = 100 * L
    shift[0] = 250
    assert s.eval(60, qkv_fn, out_fn) == 160 * L
    s.ctx.sync()
    for layer in range(L):
        ks, vs = s.ctx.export_kv(layer, 0, 0, 160)
        K, V = slots_to_float(oracle, ks, kv), slots_to_float(oracle, vs, kv)
        check(layer, 159, got[(layer, 159, 1)][0].cpu().numpy(), 159 + 250, K, V)
        oq, _ = oracle.qk_norm_rope(data["q"][layer, 130 + 250], data["k"][layer, 130 + 250], w[layer, 0], w[layer, 1], 1e-5, 130, inv, af, 2)
        q16 = oq.astype(np.float16).astype(np.float32)
        check_attention(got[(layer, 100, 59)][30].cpu().numpy(), oracle.attention(q16, K[:131], V[:131]), "chunk row 130 after the cut")
    # single tokens (decode only), then reset
    got.clear()
    assert s.eval(1, qkv_fn, out_fn) == 161 * L and (0, 160, 1) in got
    s.reset()
    assert s.cache_len == 0
    s.close()
