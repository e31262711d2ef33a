"""ctypes front-end of the test oracle (TEST INFRASTRUCTURE ONLY).

``oracle.lib``      -- the C restatement in oracle/hy3_oracle.c (always available; built on demand)
``oracle.ref_cpu``  -- the reference's own hy3.c compiled into oracle/_ref/ (None when absent)
``oracle.ref_gpu``  -- the reference's own hy3_gpu.cu kernels in oracle/_ref/ (None when absent)

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this package;
the product package must never do so.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
H, G, D = 64, 8, 128


def build(verbose=False):
    """(Re)build liboracle.so and, when the reference checkout is present, oracle/_ref/."""
    r = subprocess.run(["make", "-C", _HERE, "all"], capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("oracle build failed")


def _load(path, mode=C.DEFAULT_MODE):
    return C.CDLL(path, mode=mode) if os.path.exists(path) else None


if not os.path.exists(os.path.join(_HERE, "liboracle.so")):
    build()
lib = _load(os.path.join(_HERE, "liboracle.so"))

_f = C.POINTER(C.c_float)
_u8 = C.POINTER(C.c_uint8)


def _p(a, t=C.c_float):
    return a.ctypes.data_as(C.POINTER(t))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


lib.hy3o_half_to_float.restype = C.c_float
lib.hy3o_half_to_float.argtypes = [C.c_uint16]
lib.hy3o_float_to_half.restype = C.c_uint16
lib.hy3o_float_to_half.argtypes = [C.c_float]


# ------------------------------------------------------------------ restatement wrappers
def rope_table(base=11158840.0, yarn=0, factor=1.0, orig_ctx=262144.0, beta_fast=32.0, beta_slow=1.0,
               attn_factor_override=-1.0):
    inv = np.zeros(64, np.float32)
    af = C.c_float(0)
    lib.hy3o_rope_table(C.c_double(base), C.c_int(yarn), C.c_double(factor), C.c_double(orig_ctx),
                        C.c_double(beta_fast), C.c_double(beta_slow), C.c_double(attn_factor_override),
                        _p(inv), C.byref(af))
    return inv, float(af.value)


def rms_norm(x, w, eps):
    x = _f32(x)
    out = np.empty_like(x)
    lib.hy3o_rms_norm(_p(out), _p(x), _p(_f32(w)), C.c_int(x.size), C.c_float(eps))
    return out


def rope(x, pos, inv_freq, af=1.0, stride=1, jump=0, jump_at=0):
    """x: [n_heads, 128]; returns a rotated copy."""
    x = _f32(x).copy()
    lib.hy3o_rope(_p(x), C.c_int(x.shape[0]), C.c_int(pos), _p(_f32(inv_freq)), C.c_float(af),
                  C.c_int(stride), C.c_int(jump), C.c_int(jump_at))
    return x


def qk_norm_rope(q, k, qw, kw, eps, pos, inv_freq, af=1.0, stride=1, jump=0, jump_at=0):
    q = _f32(q).copy()
    k = _f32(k).copy()
    lib.hy3o_qk_norm_rope(_p(q), _p(k), _p(_f32(qw)), _p(_f32(kw)), C.c_float(eps),
                          C.c_int(q.size // D), C.c_int(k.size // D), C.c_int(pos), _p(_f32(inv_freq)),
                          C.c_float(af), C.c_int(stride), C.c_int(jump), C.c_int(jump_at))
    return q, k


def quant_int8(x):
    """x: [..., 128] -> (codes int8 [..., 128], scales uint16 [...])."""
    x = _f32(x)
    rows = x.reshape(-1, D)
    codes = np.empty(rows.shape, np.int8)
    scales = np.empty(rows.shape[0], np.uint16)
    for i in range(rows.shape[0]):
        lib.hy3o_quant_int8(_p(rows[i]), _p(scales[i:i + 1], C.c_uint16), _p(codes[i], C.c_int8))
    return codes.reshape(x.shape), scales.reshape(x.shape[:-1])


def quant_int4(x):
    """x: [..., 128] -> (packed uint8 [..., 64], scales uint16 [...])."""
    x = _f32(x)
    rows = x.reshape(-1, D)
    packed = np.empty((rows.shape[0], D // 2), np.uint8)
    scales = np.empty(rows.shape[0], np.uint16)
    for i in range(rows.shape[0]):
        lib.hy3o_quant_int4(_p(rows[i]), _p(scales[i:i + 1], C.c_uint16), _p(packed[i], C.c_uint8))
    return packed.reshape(x.shape[:-1] + (D // 2,)), scales.reshape(x.shape[:-1])


def half_to_float(h):
    return np.asarray(h, np.uint16).view(np.float16).astype(np.float32)


def dequant_int8(codes, scales):
    return codes.astype(np.float32) * half_to_float(scales)[..., None]


def dequant_int4(packed, scales):
    lo = (packed & 0xF).astype(np.int32)
    hi = (packed >> 4).astype(np.int32)
    lo = np.where(lo > 7, lo - 16, lo)
    hi = np.where(hi > 7, hi - 16, hi)
    codes = np.stack([lo, hi], axis=-1).reshape(packed.shape[:-1] + (D,))
    return codes.astype(np.float32) * half_to_float(scales)[..., None]


def round_fp16(x):
    return _f32(x).astype(np.float16).astype(np.float32)


def stored_kv(x, kv_dtype):
    """What attention sees after x (fp32 [..., 128]) went through the cache of the given dtype."""
    if kv_dtype == "fp16":
        return round_fp16(x)
    if kv_dtype == "int8":
        return dequant_int8(*quant_int8(x))
    if kv_dtype == "int4":
        return dequant_int4(*quant_int4(x))
    raise ValueError(kv_dtype)


def attention(q, k, v):
    """q [n_heads,128], k/v [ntok, n_kv, 128] -> out [n_heads,128] (fp32 two-pass, uncapped)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty_like(q)
    lib.hy3o_attention(_p(out), _p(q), _p(k), _p(v), C.c_int(q.shape[0]), C.c_int(k.shape[1]), C.c_int(k.shape[0]))
    return out


def attention_f64(q, k, v):
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty(q.shape, np.float64)
    lib.hy3o_attention_f64(_p(out, C.c_double), _p(q), _p(k), _p(v), C.c_int(q.shape[0]), C.c_int(k.shape[1]),
                           C.c_int(k.shape[0]))
    return out


def attention_partial(q, k, v, t0, t1):
    q, k, v = _f32(q), _f32(k), _f32(v)
    part = np.empty((q.shape[0], 130), np.float32)
    lib.hy3o_attention_partial(_p(part), _p(q), _p(k), _p(v), C.c_int(q.shape[0]), C.c_int(k.shape[1]),
                               C.c_int(t0), C.c_int(t1))
    return part


def merge_partials(partials):
    """partials [n_parts, n_heads, 130] -> out [n_heads, 128]."""
    partials = _f32(partials)
    out = np.empty((partials.shape[1], D), np.float32)
    lib.hy3o_merge_partials(_p(out), _p(partials), C.c_int(partials.shape[0]), C.c_int(partials.shape[1]))
    return out


def prefill_causal(q, k, v, base_tok, rows=None):
    """q [nq, n_heads, 128]; k, v [>= base_tok+nq, n_kv, 128]; rows: chunk-local indices or None."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    nq, nh = q.shape[0], q.shape[1]
    out = np.zeros_like(q)
    if rows is None:
        rp, nr = None, 0
    else:
        rows = np.ascontiguousarray(rows, np.int32)
        rp, nr = _p(rows, C.c_int), rows.size
    lib.hy3o_prefill_causal(_p(out), _p(q), _p(k), _p(v), C.c_int(nh), C.c_int(k.shape[1]), C.c_int(base_tok),
                            C.c_int(nq), C.c_size_t(nh * D), C.c_size_t(nh * D), rp, C.c_int(nr))
    return out


def fill_normal(shape, seed, tensor_id):
    out = np.empty(shape, np.float32)
    lib.hy3o_fill_normal(_p(out), C.c_size_t(out.size), C.c_uint64(seed), C.c_uint64(tensor_id))
    return out


# ------------------------------------------------------------------ compiled reference (optional)
class _RefCpu:
    """The reference's own CPU functions (hy3.c) from oracle/_ref/."""

    def __init__(self, path):
        self.lib = C.CDLL(path)
        self.lib.hy3ref_max_threads.restype = C.c_int

    def rope_init(self, env=None):
        """Run hy3_rope_init under the given HY3_* environment; returns (inv_freq[64], attn_factor)."""
        keys = ["HY3_ROPE_YARN", "HY3_ROPE_FACTOR", "HY3_ROPE_ORIG_CTX", "HY3_ROPE_BETA_FAST", "HY3_ROPE_BETA_SLOW",
                "HY3_ROPE_ATTN_FACTOR", "HY3_CTX", "HY3_POS_STRIDE", "HY3_POS_JUMP", "HY3_POS_JUMP_AT"]
        libc = C.CDLL(None)
        for k in keys:
            libc.unsetenv(k.encode())
        for k, v in (env or {}).items():
            libc.setenv(k.encode(), str(v).encode(), 1)
        inv = np.zeros(64, np.float32)
        af = C.c_float(0)
        self.lib.hy3ref_rope_init(_p(inv), C.byref(af))
        for k in (env or {}):
            libc.unsetenv(k.encode())
        return inv, float(af.value)

    def rope(self, q, k, pos):
        q, k = _f32(q).copy(), _f32(k).copy()
        self.lib.hy3ref_rope(_p(q), _p(k), C.c_int(pos))
        return q, k

    def rms_norm(self, x, w, eps):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.hy3ref_rms_norm(_p(out), _p(x), _p(_f32(w)), C.c_int(x.size), C.c_float(eps))
        return out

    def load_layer(self, k, v, layer=0):
        k, v = _f32(k), _f32(v)
        if self.lib.hy3ref_load_layer(_p(k), _p(v), C.c_int(k.shape[0]), C.c_int(layer)):
            raise MemoryError("reference slot mapping failed")

    def attention(self, q, ntok, layer=0, threads=1):
        q = _f32(q)
        out = np.zeros_like(q)
        fn = self.lib.hy3ref_attention_mt if threads > 1 else self.lib.hy3ref_attention
        fn(_p(out), _p(q), C.c_int(ntok), C.c_int(layer))
        return out

    def attention_layers(self, q, ntok):
        """q [n_layers, 64, 128]; all layers previously loaded with load_layer; all host threads."""
        q = _f32(q)
        out = np.zeros_like(q)
        self.lib.hy3ref_attention_layers_mt(_p(out), _p(q), C.c_int(ntok), C.c_int(q.shape[0]))
        return out

    def max_threads(self):
        return int(self.lib.hy3ref_max_threads())

    def set_threads(self, n):
        """OpenMP team size of the *_mt entry points; returns the size in effect."""
        self.lib.hy3ref_set_threads.restype = C.c_int
        return int(self.lib.hy3ref_set_threads(C.c_int(int(n))))


class _RefGpu:
    """The reference's own CUDA kernels (hy3_gpu.cu) from oracle/_ref/; needs a GPU to call."""

    def __init__(self, path):
        self.lib = C.CDLL(path)

    @staticmethod
    def _chk(rc, what):
        if rc:
            raise RuntimeError("reference CUDA harness: %s failed (%d)" % (what, rc))

    def qk_norm_rope(self, q, k, qw, kw, pos, inv_freq, af=1.0, stride=1, jump=0, jump_at=0):
        q, k = _f32(q).copy(), _f32(k).copy()
        self._chk(self.lib.hy3refgpu_qk_norm_rope(_p(q), _p(k), _p(_f32(qw)), _p(_f32(kw)), C.c_int(pos),
                                                  _p(_f32(inv_freq)), C.c_float(af), C.c_int(stride),
                                                  C.c_int(jump), C.c_int(jump_at)), "qk_norm_rope")
        return q, k

    def kv_quantize(self, k, v, int4=False):
        """k, v [n, 8, 128] fp32 -> raw reference slots (uint8 [n, 1040|528]) for K and V."""
        k, v = _f32(k), _f32(v)
        n = k.shape[0]
        stride = 528 if int4 else 1040
        ks = np.zeros((n, stride), np.uint8)
        vs = np.zeros((n, stride), np.uint8)
        self._chk(self.lib.hy3refgpu_kv_quantize(C.c_int(int(int4)), _p(k), _p(v), C.c_int(n), _p(ks, C.c_uint8),
                                                 _p(vs, C.c_uint8)), "kv_quantize")
        return ks, vs

    def decode(self, q, kslots, vslots, nsplits=16, int4=False):
        q = _f32(q)
        out = np.zeros_like(q)
        self._chk(self.lib.hy3refgpu_decode(C.c_int(int(int4)), _p(q), _p(kslots, C.c_uint8), _p(vslots, C.c_uint8),
                                            C.c_int(kslots.shape[0]), C.c_int(nsplits), _p(out)), "decode")
        return out

    def prefill(self, q, kslots, vslots, base_tok, int4=False):
        q = _f32(q)
        out = np.zeros_like(q)
        self._chk(self.lib.hy3refgpu_prefill(C.c_int(int(int4)), _p(q), _p(kslots, C.c_uint8), _p(vslots, C.c_uint8),
                                             C.c_int(base_tok), C.c_int(q.shape[0]), _p(out)), "prefill")
        return out

    def decode_bench(self, ntok, nl, iters, int4=False):
        ms = C.c_float(0)
        self._chk(self.lib.hy3refgpu_decode_bench(C.c_int(int(int4)), C.c_int(ntok), C.c_int(nl), C.c_int(iters),
                                                  C.byref(ms)), "decode_bench")
        return float(ms.value)


def split_slots(slots, int4=False):
    """Reference slot bytes [n, 1040|528] -> (scales uint16 [n, 8], codes [n, 8, 128|64])."""
    n = slots.shape[0]
    scales = slots[:, :16].copy().view(np.uint16).reshape(n, 8)
    body = slots[:, 16:].reshape(n, 8, -1)
    return scales, (body.copy() if int4 else body.copy().view(np.int8))


def _try(cls, name):
    path = os.path.join(_HERE, "_ref", name)
    if not os.path.exists(path):
        return None
    try:
        return cls(path)
    except OSError:
        return None


ref_cpu = _try(_RefCpu, "libhy3ref_cpu.so")
ref_cpu_strict = _try(_RefCpu, "libhy3ref_cpu_strict.so")


def ref_gpu():
    """Loaded lazily: needs libcudart/libcublas and is only meaningful on a GPU box."""
    return _try(_RefGpu, "libhy3ref_gpu.so")
