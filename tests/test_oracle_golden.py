"""The C restatement (oracle/hy3_oracle.c) against the committed fixtures that the COMPILED
REFERENCE produced (tests/golden/make_golden.py).  Runs anywhere, no reference checkout."""
import os
import sys
import zlib

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as mg  # noqa: E402  (case tables only; nothing is generated here)

SEED = mg.SEED


def crc(a):
    return np.uint32(zlib.crc32(np.ascontiguousarray(a).tobytes()))


def env_to_table(oracle, env):
    yarn, factor, orig, bf, bs, afo = 0, 1.0, 262144.0, 32.0, 1.0, -1.0
    if "HY3_ROPE_ORIG_CTX" in env:
        orig = float(env["HY3_ROPE_ORIG_CTX"])
    if "HY3_ROPE_FACTOR" in env and float(env["HY3_ROPE_FACTOR"]) > 1.0:
        factor, yarn = float(env["HY3_ROPE_FACTOR"]), 1
    if "HY3_CTX" in env and float(env["HY3_CTX"]) > orig:
        factor, yarn = max(factor, float(env["HY3_CTX"]) / orig), 1
    if "HY3_ROPE_BETA_FAST" in env:
        bf = float(env["HY3_ROPE_BETA_FAST"])
    if "HY3_ROPE_BETA_SLOW" in env:
        bs = float(env["HY3_ROPE_BETA_SLOW"])
    if "HY3_ROPE_ATTN_FACTOR" in env:
        afo = float(env["HY3_ROPE_ATTN_FACTOR"])
    return oracle.rope_table(yarn=yarn, factor=factor, orig_ctx=orig, beta_fast=bf, beta_slow=bs, attn_factor_override=afo)


@pytest.fixture(scope="module")
def qkw(oracle, golden_cpu):
    q = oracle.fill_normal((64, 128), SEED, 1)
    k = oracle.fill_normal((8, 128), SEED, 2)
    w = (1.0 + 0.02 * oracle.fill_normal((2, 128), SEED, 3)).astype(np.float32)
    assert list(golden_cpu["in_crc_qkw"]) == [crc(q), crc(k), crc(w)], "seeded inputs drifted (libm?)"
    return q, k, w


@pytest.mark.parametrize("name", list(mg.ROPE_ENVS))
def test_rope_table_matches_reference(oracle, golden_cpu, name):
    inv, af = env_to_table(oracle, mg.ROPE_ENVS[name])
    assert np.array_equal(inv, golden_cpu["table_%s_inv" % name])
    assert np.float32(af) == golden_cpu["table_%s_af" % name]


def test_known_table_values(oracle):
    inv, af = oracle.rope_table()
    assert af == 1.0 and inv[0] == 1.0
    assert abs(inv[1] - 0.776034355) < 1e-8 and abs(inv[63] - 1.15478201e-07) < 1e-14
    inv4, af4 = oracle.rope_table(yarn=1, factor=4.0)
    assert abs(af4 - 1.13862944) < 1e-7 and abs(inv4[63] - 2.88695503e-08) < 1e-15


@pytest.mark.parametrize("eps_name,eps", [("1e-5", 1e-5), ("1e-6", 1e-6)])
def test_rms_norm_bit_exact(oracle, golden_cpu, qkw, eps_name, eps):
    q, k, w = qkw
    got_q = np.stack([oracle.rms_norm(q[h], w[0], eps) for h in range(64)])
    got_k = np.stack([oracle.rms_norm(k[h], w[1], eps) for h in range(8)])
    assert np.array_equal(got_q, golden_cpu["norm_q_eps%s" % eps_name])
    assert np.array_equal(got_k, golden_cpu["norm_k_eps%s" % eps_name])


@pytest.mark.parametrize("name,env,pos", mg.ROPE_CASES)
def test_rope_bit_exact(oracle, golden_cpu, qkw, name, env, pos):
    q, k, _ = qkw
    inv, af = env_to_table(oracle, env)
    st = int(env.get("HY3_POS_STRIDE", 1))
    j, ja = int(env.get("HY3_POS_JUMP", 0)), int(env.get("HY3_POS_JUMP_AT", 0))
    assert np.array_equal(oracle.rope(q, pos, inv, af, st, j, ja), golden_cpu["rope_%s_q" % name])
    assert np.array_equal(oracle.rope(k, pos, inv, af, st, j, ja), golden_cpu["rope_%s_k" % name])


@pytest.mark.parametrize("ntok", mg.ATTN_NTOK)
def test_attention_bit_exact(oracle, golden_cpu, qkw, ntok):
    q = qkw[0]
    K = oracle.fill_normal((ntok, 8, 128), SEED, 10 + ntok)
    V = oracle.fill_normal((ntok, 8, 128), SEED, 5000 + ntok)
    assert list(golden_cpu["attn_%d_crc" % ntok]) == [crc(K), crc(V)]
    out = oracle.attention(q, K, V)
    assert np.array_equal(out, golden_cpu["attn_%d_l0" % ntok])      # strict build of the reference, layer 0
    assert np.array_equal(out, golden_cpu["attn_%d_l79" % ntok])     # the layer index only moves the slots
    # the reference as shipped (-ffast-math) differs only at rounding level
    assert np.abs(out - golden_cpu["attn_%d_fastmath" % ntok]).max() < 2e-6
    assert np.abs(oracle.attention_f64(q, K, V) - out).max() < 5e-6


def test_partials_merge_equals_attention(oracle, qkw):
    q = qkw[0]
    K = oracle.fill_normal((300, 8, 128), SEED, 77)
    V = oracle.fill_normal((300, 8, 128), SEED, 78)
    cuts = [0, 1, 128, 128, 257, 300]  # includes an empty range
    parts = np.stack([oracle.attention_partial(q, K, V, a, b) for a, b in zip(cuts[:-1], cuts[1:])])
    assert np.isneginf(parts[2, :, 0]).all() and (parts[2, :, 1] == 0).all()
    assert np.abs(oracle.merge_partials(parts) - oracle.attention(q, K, V)).max() < 2e-6


def test_prefill_is_per_token_decode(oracle, qkw):
    rng = np.random.default_rng(5)
    K = oracle.fill_normal((40, 8, 128), SEED, 91)
    V = oracle.fill_normal((40, 8, 128), SEED, 92)
    q = rng.standard_normal((8, 64, 128)).astype(np.float32)
    out = oracle.prefill_causal(q, K, V, base_tok=32)
    for i in (0, 3, 7):
        assert np.array_equal(out[i], oracle.attention(q[i], K[:33 + i], V[:33 + i]))
    sub = oracle.prefill_causal(q, K, V, base_tok=32, rows=[7, 0])
    assert np.array_equal(sub[7], out[7]) and np.array_equal(sub[0], out[0]) and not sub[3].any()
