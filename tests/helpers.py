"""Shared helpers of the GPU parity tests: build reference-format slots on the host with the
oracle quantiser, and compare device results with the oracle attention."""
import numpy as np

SEED = 0x4859335F53454544
# max-abs tolerance of the attention output against the fp32 oracle evaluated on the SAME stored
# (rounded / dequantised) K and V; fp16 tensor-core compute against fp32 reference.
ATTN_TOL = 2e-3
REL_RMS_TOL = 1e-3


def make_slots(oracle, x, kv_dtype):
    """x [n, 8, 128] fp32 -> reference-format slots uint8 [n, slot_bytes] (hy3_gpu.cu:26-35)."""
    n = x.shape[0]
    if kv_dtype == "fp16":
        return np.ascontiguousarray(x.astype(np.float16)).view(np.uint8).reshape(n, 2048)
    if kv_dtype == "int8":
        codes, scales = oracle.quant_int8(x)
        out = np.zeros((n, 1040), np.uint8)
        out[:, :16] = scales.astype(np.uint16).view(np.uint8).reshape(n, 16)
        out[:, 16:] = codes.view(np.uint8).reshape(n, 1024)
        return out
    packed, scales = oracle.quant_int4(x)
    out = np.zeros((n, 528), np.uint8)
    out[:, :16] = scales.astype(np.uint16).view(np.uint8).reshape(n, 16)
    out[:, 16:] = packed.reshape(n, 512)
    return out


def slots_to_float(oracle, slots, kv_dtype):
    """Reference-format slots -> the fp32 values attention sees, [n, 8, 128]."""
    n = slots.shape[0]
    if kv_dtype == "fp16":
        return slots.reshape(n, 8, 256).copy().view(np.float16).astype(np.float32).reshape(n, 8, 128)
    scales, codes = oracle.split_slots(slots, int4=(kv_dtype == "int4"))
    return oracle.dequant_int4(codes, scales) if kv_dtype == "int4" else oracle.dequant_int8(codes, scales)


def check_attention(got, want, what=""):
    err = np.abs(got - want).max()
    rel = np.sqrt(((got - want) ** 2).mean() / max((want ** 2).mean(), 1e-30))
    assert np.isfinite(got).all(), "%s: non-finite output" % what
    assert err <= ATTN_TOL, "%s: max-abs %.3g > %.3g" % (what, err, ATTN_TOL)
    assert rel <= REL_RMS_TOL, "%s: relative RMS %.3g > %.3g" % (what, rel, REL_RMS_TOL)
    return err, rel
