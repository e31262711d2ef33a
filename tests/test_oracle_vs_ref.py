"""Live pin: the C restatement against the reference's own hy3.c compiled into oracle/_ref/.
Skipped when oracle/_ref/ was not built (no reference checkout); the committed fixtures in
tests/golden/ then carry the pin (test_oracle_golden.py)."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def refs(oracle):
    if oracle.ref_cpu is None or oracle.ref_cpu_strict is None:
        pytest.skip("oracle/_ref not built")
    return oracle.ref_cpu, oracle.ref_cpu_strict


def test_tables_equal(oracle, refs):
    fast, strict = refs
    for env, kw in [({}, {}), ({"HY3_ROPE_FACTOR": "4"}, dict(yarn=1, factor=4.0)),
                    ({"HY3_CTX": "524288"}, dict(yarn=1, factor=2.0)),
                    ({"HY3_ROPE_FACTOR": "4", "HY3_ROPE_YARN": "0"}, {})]:
        inv, af = oracle.rope_table(**kw)
        for r in (fast, strict):
            rinv, raf = r.rope_init(env)
            assert np.array_equal(inv, rinv) and af == raf


@pytest.mark.parametrize("ntok", [1, 5, 64, 1023, 4096])
def test_attention_bit_equal_to_strict_reference(oracle, refs, ntok):
    fast, strict = refs
    rng = np.random.default_rng(ntok)
    q = rng.standard_normal((64, 128)).astype(np.float32)
    K = rng.standard_normal((ntok, 8, 128)).astype(np.float32)
    V = rng.standard_normal((ntok, 8, 128)).astype(np.float32)
    strict.load_layer(K, V, 17)
    fast.load_layer(K, V, 17)
    mine = oracle.attention(q, K, V)
    assert np.array_equal(mine, strict.attention(q, ntok, 17))
    shipped = fast.attention(q, ntok, 17)
    assert np.abs(mine - shipped).max() < 2e-6
    assert np.array_equal(shipped, fast.attention(q, ntok, 17, threads=8))   # per-group threading changes nothing


def test_reference_drops_keys_past_4096(oracle, refs):
    """hy3.c:628-629: scores[4096] caps the CPU attention; the restatement does not."""
    _, strict = refs
    rng = np.random.default_rng(9)
    n = 4097
    q = rng.standard_normal((64, 128)).astype(np.float32)
    K = rng.standard_normal((n, 8, 128)).astype(np.float32)
    V = rng.standard_normal((n, 8, 128)).astype(np.float32)
    strict.load_layer(K, V, 0)
    capped = strict.attention(q, n, 0)
    assert np.array_equal(capped, oracle.attention(q, K[:4096], V[:4096]))
    assert not np.array_equal(capped, oracle.attention(q, K, V))


def test_norm_rope_bit_equal(oracle, refs):
    _, strict = refs
    rng = np.random.default_rng(4)
    q = rng.standard_normal((64, 128)).astype(np.float32)
    k = rng.standard_normal((8, 128)).astype(np.float32)
    w = (1 + 0.02 * rng.standard_normal(128)).astype(np.float32)
    assert np.array_equal(strict.rms_norm(q[3], w, 1e-6), oracle.rms_norm(q[3], w, 1e-6))
    inv, af = strict.rope_init({"HY3_ROPE_FACTOR": "4", "HY3_POS_STRIDE": "3"})
    rq, rk = strict.rope(q, k, 99999)
    assert np.array_equal(rq, oracle.rope(q, 99999, inv, af, 3))
    assert np.array_equal(rk, oracle.rope(k, 99999, inv, af, 3))
