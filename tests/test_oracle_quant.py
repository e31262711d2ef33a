"""Properties of the restated quantisers (hy3_gpu.cu:250-270, :329-352) and fp16 helpers.
Bit-level pins against the reference's CUDA quantiser itself live in the GPU tests (they need
a GPU to run the reference kernel) and in tests/golden/ref_gpu.npz."""
import numpy as np


def test_half_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 300, 7e4)])
    x = np.concatenate([x, np.array([0, -0.0, 65504, 65519.99, 65520, 1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001, 6.1e-5,
                                     np.inf, -np.inf], np.float32)])
    got = np.array([oracle.lib.hy3o_float_to_half(float(v)) for v in x], np.uint16)
    want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)
    back = np.array([oracle.lib.hy3o_half_to_float(int(h)) for h in range(0, 0x7C01, 7)], np.float32)
    assert np.array_equal(back, np.arange(0, 0x7C01, 7, dtype=np.uint16).view(np.float16).astype(np.float32))


def test_int8_quantiser_rules(oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((50, 128)).astype(np.float32) * rng.uniform(1e-3, 50, (50, 1)).astype(np.float32)
    codes, scales = oracle.quant_int8(x)
    m = np.abs(x).max(-1)
    s = (m / np.float32(127.0) + np.float32(1e-8)).astype(np.float32)
    assert np.array_equal(scales, s.astype(np.float16).view(np.uint16))
    inv = (np.float32(1.0) / s).astype(np.float32)
    f = np.clip(x * inv[:, None], -127, 127).astype(np.float32)
    want = np.where(f >= 0, np.floor(f + np.float32(0.5)), np.ceil(f - np.float32(0.5)))  # roundf: half away from zero
    assert np.array_equal(codes.astype(np.float32), want)
    assert np.abs(codes).max() == 127
    # reconstruction error bounded by half a step (+ fp16 scale rounding)
    rec = oracle.dequant_int8(codes, scales)
    assert (np.abs(rec - x) <= (0.5 + 127 * 2.0 ** -11) * s[:, None] * 1.0001).all()


def test_int4_quantiser_rules_and_nibble_order(oracle):
    x = np.zeros(128, np.float32)
    x[0], x[1], x[2], x[3] = 7.0, -7.0, 3.4, -3.6
    packed, scale = oracle.quant_int4(x)
    assert packed[0] == (7 | ((-7 & 0xF) << 4))          # even dim in the low nibble
    assert packed[1] == (3 | ((-4 & 0xF) << 4))
    rec = oracle.dequant_int4(packed, scale)
    s = np.float32(np.float16(np.float32(7.0) / np.float32(7.0) + np.float32(1e-8)))
    assert np.allclose(rec[:4], np.array([7, -7, 3, -4], np.float32) * s)
    rng = np.random.default_rng(2)
    y = rng.standard_normal((20, 128)).astype(np.float32)
    p, sc = oracle.quant_int4(y)
    lo, hi = (p & 0xF).astype(int), (p >> 4).astype(int)
    lo, hi = np.where(lo > 7, lo - 16, lo), np.where(hi > 7, hi - 16, hi)
    assert lo.min() >= -7 and hi.max() <= 7 and max(np.abs(lo).max(), np.abs(hi).max()) == 7


def test_zero_row_and_ties(oracle):
    codes, scale = oracle.quant_int8(np.zeros(128, np.float32))
    assert not codes.any() and scale == np.float32(1e-8).astype(np.float16).view(np.uint16) == 0
    x = np.zeros(128, np.float32)
    x[0] = 127.0
    x[1:5] = [0.5, 1.5, -0.5, -2.5]
    c, s = oracle.quant_int8(x)   # scale = 1 + 1e-8 -> 1.0f, inv = 1
    assert list(c[:5]) == [127, 1, 2, -1, -3]


def test_stored_kv_views(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 8, 128)).astype(np.float32)
    assert np.array_equal(oracle.stored_kv(x, "fp16"), x.astype(np.float16).astype(np.float32))
    assert np.abs(oracle.stored_kv(x, "int8") - x).max() < 0.03
    assert np.abs(oracle.stored_kv(x, "int4") - x).max() < 0.45
