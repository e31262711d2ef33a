"""The reference engine's backend API on the B200 attention library: hy3_gpu_init / hy3_eval_gpu / hy3_gpu_free
(hy3_b200/libhy3_gpu.so, include/hy3_gpu_dropin.h) against the engine's own CPU path.

The host program is the reference engine itself, compiled from its sources into oracle/_ref/libhy3ref_model.so
(test infrastructure), with a seeded in-memory 80-layer model (no checkpoint): layer 0 dense, layers 1..79 sharing one
set of MoE tensors.  The same token sequence goes through hy3_eval on the CPU (hy3.c:1367-1416) and through
hy3_eval_gpu, with the call pattern of hy3_generate (hy3.c:1487-1573): a prompt in one call (chunked prefill for all
but its last token, HY3_PREFILL_CHUNK), cache_len set back to a shorter prefix (hy3.c:1514), then single-token calls.

Bound: the CPU path keeps fp32 K/V; the backend stores FP16 / INT8 / INT4 K/V and computes attention in fp16, through 80
layers.  The logits must agree within the relative RMS stated per cache type below (measured on B200 with this model:
fp16 5e-5 .. 8e-5, int8 2.3e-2 .. 3.0e-2, int4 7e-2 .. 9.2e-2; the printed line shows the values of the run).

The test tensors hold no zero or subnormal half: the engine's CPU half decoder (hy3.c:354-369) reads those as
(1 + mantissa / 1024) * 2^-15 while the device decodes IEEE halves, so such values would compare the two decoders, not
the backends.
"""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
VOCAB = 1024
OUT_SCALE = 0.05      # every layer perturbs the residual stream a little: rounding differences are not amplified chaotically


class Tokens(C.Structure):
    _fields_ = [("v", C.POINTER(C.c_int)), ("len", C.c_int), ("cap", C.c_int)]


@pytest.fixture(scope="module")
def engine():
    path = os.path.join(ROOT, "oracle", "_ref", "libhy3ref_model.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libhy3ref_model.so not built (needs the reference checkout at build time)")
    host = C.CDLL(path, mode=C.RTLD_GLOBAL)          # provides hy3_rope_get_params / forward_layer_* to the backend
    host.hy3h_model_new.restype = C.c_void_p
    host.hy3h_model_new.argtypes = [C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
    host.hy3h_model_free.argtypes = [C.c_void_p]
    host.hy3h_eval_cpu.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_int)]
    for f in ("hy3h_get_cache_len", "hy3h_gpu_layers", "hy3h_has_gpu_ctx"):
        getattr(host, f).argtypes = [C.c_void_p]
    host.hy3h_set_cache_len.argtypes = [C.c_void_p, C.c_int]
    host.hy3h_set_expert_used.argtypes = [C.c_void_p, C.c_int]
    gpu = C.CDLL(os.path.join(ROOT, "hy3_b200", "libhy3_gpu.so"))
    gpu.hy3_gpu_init.argtypes = [C.c_void_p, C.c_int]
    gpu.hy3_gpu_free.argtypes = [C.c_void_p]
    gpu.hy3_eval_gpu.argtypes = [C.c_void_p, C.POINTER(Tokens), C.POINTER(C.c_float), C.POINTER(C.c_int)]
    gpu.hy3_gpu_last_error.restype = C.c_char_p
    gpu.hy3_gpu_last_error.argtypes = [C.c_void_p]
    return host, gpu


def eval_cpu(host, m, toks):
    arr = (C.c_int * len(toks))(*toks)
    logits = np.zeros(VOCAB, np.float32)
    pos = C.c_int(-1)
    assert host.hy3h_eval_cpu(m, arr, len(toks), logits.ctypes.data_as(C.POINTER(C.c_float)), C.byref(pos)) == 0
    return logits, pos.value


def eval_gpu(gpu, m, toks):
    arr = (C.c_int * len(toks))(*toks)
    t = Tokens(arr, len(toks), len(toks))
    logits = np.zeros(VOCAB, np.float32)
    pos = C.c_int(-1)
    rc = gpu.hy3_eval_gpu(m, C.byref(t), logits.ctypes.data_as(C.POINTER(C.c_float)), C.byref(pos))
    assert rc == 0, gpu.hy3_gpu_last_error(m)
    return logits, pos.value


def rel_rms(a, b):
    return float(np.sqrt(((a - b) ** 2).mean() / (b ** 2).mean()))


PROMPT = [3, 141, 59, 26, 535, 897, 93, 238, 462]       # 9 tokens: chunks of 4 + 4, the last one through the decode path
NEXT = [643, 383, 279]                                  # after the cut back to 3 tokens: eager, graph capture, graph replay


def reference_run(host, m):
    host.hy3h_set_cache_len(m, 0)
    out = [eval_cpu(host, m, PROMPT)]
    host.hy3h_set_cache_len(m, 3 * 80)                   # prefix reuse: keep 3 tokens (hy3.c:1514)
    for t in NEXT:
        out.append(eval_cpu(host, m, [t]))
    return out


@pytest.fixture(scope="module")
def model_and_reference(engine):
    host, _ = engine
    m = host.hy3h_model_new(20261125, VOCAB, 4, 0, 0, OUT_SCALE)
    assert m
    host.hy3h_set_expert_used(m, 2)                      # the run-time top-k (hy3.h: n_expert_used), to keep the CPU side short
    ref = reference_run(host, m)
    yield m, ref
    host.hy3h_model_free(m)


@pytest.mark.parametrize("kv,bound", [("fp16", 1e-3), ("int8", 6e-2), ("int4", 2e-1)])
def test_eval_gpu_matches_cpu_eval(engine, model_and_reference, monkeypatch, capfd, kv, bound):
    host, gpu = engine
    m, ref = model_and_reference
    for k in ("HY3_KV_INT4", "HY3_KV_FP16"):
        monkeypatch.delenv(k, raising=False)
    if kv != "int8":
        monkeypatch.setenv("HY3_KV_" + kv.upper(), "1")
    monkeypatch.setenv("HY3_PREFILL_CHUNK", "4")
    monkeypatch.setenv("HY3_KV_TOKENS", "1024")
    assert gpu.hy3_gpu_init(m, 0) == 0
    try:
        assert host.hy3h_has_gpu_ctx(m) and host.hy3h_gpu_layers(m) == 81          # clamp of hy3_gpu.cu:555
        err = capfd.readouterr().err
        assert "hy3_gpu: initialized (81 layers, %s KV, online attn)" % kv.upper() in err   # the line eval/hy3_needle.py:103 reads
        assert "chunked prefill enabled (chunk=4 tokens)" in err
        host.hy3h_set_cache_len(m, 0)
        got = [eval_gpu(gpu, m, PROMPT)]
        assert got[0][1] == len(PROMPT) * 80 == host.hy3h_get_cache_len(m)
        host.hy3h_set_cache_len(m, 3 * 80)
        for t in NEXT:
            got.append(eval_gpu(gpu, m, [t]))
        errs = []
        for (lg, pg), (lc, pc) in zip(got, ref):
            assert pg == pc and np.isfinite(lg).all()
            errs.append(rel_rms(lg, lc))
        print("hy3_eval_gpu vs hy3_eval (CPU), %s KV: relative RMS of the logits per call %s; arg-max equal: %s"
              % (kv, ["%.2e" % e for e in errs], [int(np.argmax(a[0]) == np.argmax(b[0])) for a, b in zip(got, ref)]))
        assert max(errs) <= bound
        # cutting back and feeding the same tokens again reproduces the same logits bit for bit (K/V below cache_len persist)
        host.hy3h_set_cache_len(m, 4 * 80)
        again, _ = eval_gpu(gpu, m, [NEXT[1]])
        assert np.array_equal(again, got[2][0])
    finally:
        gpu.hy3_gpu_free(m)
    assert not host.hy3h_has_gpu_ctx(m)


def test_partial_offload_runs_the_tail_on_the_host(engine, model_and_reference, monkeypatch):
    """n_gpu_layers = 78: layers 78 and 79 run through the engine's forward_layer_moe on the host (hy3_gpu.cu:945-950)."""
    host, gpu = engine
    m, ref = model_and_reference
    for k in ("HY3_KV_INT4", "HY3_PREFILL_CHUNK"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("HY3_KV_FP16", "1")
    monkeypatch.setenv("HY3_KV_TOKENS", "256")
    assert gpu.hy3_gpu_init(m, 78) == 0
    try:
        host.hy3h_set_cache_len(m, 0)
        lg, pos = eval_gpu(gpu, m, PROMPT[:2])
        assert pos == 160
        host.hy3h_set_cache_len(m, 0)
        lc, _ = eval_cpu(host, m, PROMPT[:2])
        assert rel_rms(lg, lc) <= 2e-2
    finally:
        gpu.hy3_gpu_free(m)


def test_q4k_and_f16_tensors(engine, monkeypatch):
    """Routed experts kept as Q4_K blocks on the device and an F16 query projection: against the engine's own
    dequantising CPU matmul (hy3.c:1007-1041, :1080-1155)."""
    host, gpu = engine
    m = host.hy3h_model_new(7, VOCAB, 2, 12, 1, 0.4)     # Q4_K scales must be normal halves: the expert down projection cannot be made smaller
    assert m
    host.hy3h_set_expert_used(m, 2)
    for k in ("HY3_KV_INT4", "HY3_PREFILL_CHUNK"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("HY3_KV_FP16", "1")
    monkeypatch.setenv("HY3_KV_TOKENS", "256")
    try:
        lc, _ = eval_cpu(host, m, PROMPT[:2])
        assert gpu.hy3_gpu_init(m, 0) == 0
        host.hy3h_set_cache_len(m, 0)
        lg, _ = eval_gpu(gpu, m, PROMPT[:2])
        e = rel_rms(lg, lc)
        print("Q4_K experts + F16 projection: relative RMS of the logits %.2e" % e)
        assert e <= 5e-2
    finally:
        gpu.hy3_gpu_free(m)
        host.hy3h_model_free(m)


def test_cache_capacity_is_an_error_code(engine, model_and_reference, monkeypatch):
    """A call that would run past the KV pool (HY3_KV_TOKENS) returns -1 with a message (the reference grows by realloc + copy,
    hy3_gpu.cu:692-698, and exits when that fails); the context stays usable for a sequence that fits."""
    host, gpu = engine
    m, ref = model_and_reference
    for k in ("HY3_KV_INT4", "HY3_KV_FP16"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("HY3_PREFILL_CHUNK", "64")
    monkeypatch.setenv("HY3_KV_TOKENS", "128")
    assert gpu.hy3_gpu_init(m, 0) == 0
    try:
        host.hy3h_set_cache_len(m, 0)
        toks = [(7 * i + 3) % VOCAB for i in range(200)]
        arr = (C.c_int * len(toks))(*toks)
        t = Tokens(arr, len(toks), len(toks))
        logits = np.zeros(VOCAB, np.float32)
        pos = C.c_int(-1)
        assert gpu.hy3_eval_gpu(m, C.byref(t), logits.ctypes.data_as(C.POINTER(C.c_float)), C.byref(pos)) == -1
        assert b"HY3_KV_TOKENS" in gpu.hy3_gpu_last_error(m)
        host.hy3h_set_cache_len(m, 0)
        got, _ = eval_gpu(gpu, m, PROMPT)                    # chunk 64 > 8 tokens: one chunk + the last token
        assert rel_rms(got, ref[0][0]) <= 6e-2               # INT8 cache: the bound of the parity test above
    finally:
        gpu.hy3_gpu_free(m)
