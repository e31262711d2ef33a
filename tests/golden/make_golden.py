"""Generate the committed golden fixtures from the COMPILED REFERENCE (oracle/_ref).

Run in the development container, where the reference checkout is mounted and
`make -C oracle` has produced oracle/_ref/:

    python tests/golden/make_golden.py            # CPU fixtures (reference hy3.c)
    python tests/golden/make_golden.py --gpu OUT  # GPU fixtures (reference hy3_gpu.cu kernels; needs a GPU)

Inputs are regenerated from seeds by oracle.fill_normal (a checksum of every input is
stored so drift is detected); outputs are what the reference's own code returned.
The fixtures pin the C restatement in oracle/hy3_oracle.c (tests/test_oracle_golden.py).
"""
import os
import sys
import zlib

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SEED = 0x4859335F53454544

ROPE_ENVS = {
    "default": {},
    "yarn4": {"HY3_ROPE_FACTOR": "4"},
    "ctx1m": {"HY3_CTX": "1048576"},
    "yarn2_beta": {"HY3_ROPE_FACTOR": "2", "HY3_ROPE_BETA_FAST": "16", "HY3_ROPE_BETA_SLOW": "2"},
    "yarn8_af": {"HY3_ROPE_FACTOR": "8", "HY3_ROPE_ATTN_FACTOR": "1.25", "HY3_ROPE_ORIG_CTX": "131072"},
}
# (name, env for the reference, pos)
ROPE_CASES = [
    ("p0", {}, 0), ("p1", {}, 1), ("p4096", {}, 4096), ("p262143", {}, 262143),
    ("yarn4_p1048575", {"HY3_ROPE_FACTOR": "4"}, 1048575),
    ("stride7_p300", {"HY3_POS_STRIDE": "7"}, 300),
    ("jump_p50", {"HY3_POS_JUMP": "300000", "HY3_POS_JUMP_AT": "40"}, 50),
    ("jump_p39", {"HY3_POS_JUMP": "300000", "HY3_POS_JUMP_AT": "40"}, 39),
]
ATTN_NTOK = [1, 2, 7, 129, 640]


def crc(a):
    return np.uint32(zlib.crc32(np.ascontiguousarray(a).tobytes()))


def cpu_fixtures():
    ref = oracle.ref_cpu_strict
    fast = oracle.ref_cpu
    assert ref is not None and fast is not None, "build oracle/_ref first (make -C oracle)"
    out = {}
    for name, env in ROPE_ENVS.items():
        inv, af = ref.rope_init(env)
        out["table_%s_inv" % name] = inv
        out["table_%s_af" % name] = np.float32(af)
    q = oracle.fill_normal((64, 128), SEED, 1)
    k = oracle.fill_normal((8, 128), SEED, 2)
    w = (1.0 + 0.02 * oracle.fill_normal((2, 128), SEED, 3)).astype(np.float32)
    out["in_crc_qkw"] = np.array([crc(q), crc(k), crc(w)], np.uint32)
    for eps_name, eps in (("1e-5", 1e-5), ("1e-6", 1e-6)):
        out["norm_q_eps%s" % eps_name] = np.stack([ref.rms_norm(q[h], w[0], eps) for h in range(64)])
        out["norm_k_eps%s" % eps_name] = np.stack([ref.rms_norm(k[h], w[1], eps) for h in range(8)])
    for name, env, pos in ROPE_CASES:
        ref.rope_init(env)
        rq, rk = ref.rope(q, k, pos)
        out["rope_%s_q" % name] = rq
        out["rope_%s_k" % name] = rk
    for ntok in ATTN_NTOK:
        K = oracle.fill_normal((ntok, 8, 128), SEED, 10 + ntok)
        V = oracle.fill_normal((ntok, 8, 128), SEED, 5000 + ntok)
        out["attn_%d_crc" % ntok] = np.array([crc(K), crc(V)], np.uint32)
        for layer in (0, 79):
            ref.load_layer(K, V, layer)
            out["attn_%d_l%d" % (ntok, layer)] = ref.attention(q, ntok, layer)
        fast.load_layer(K, V, 0)
        out["attn_%d_fastmath" % ntok] = fast.attention(q, ntok, 0)
    np.savez_compressed(os.path.join(HERE, "ref_cpu.npz"), **out)
    print("wrote ref_cpu.npz with", len(out), "arrays")


def gpu_fixtures(outdir):
    rg = oracle.ref_gpu()
    assert rg is not None, "oracle/_ref/libhy3ref_gpu.so missing"
    out = {}
    n = 24
    k = oracle.fill_normal((n, 8, 128), SEED, 21)
    v = oracle.fill_normal((n, 8, 128), SEED, 22)
    # edge rows: zeros, a single spike, exact .5 ties after scaling, huge and tiny magnitudes
    k[0] = 0.0
    v[0, :, 5] = 3.0
    v[0, :, 6:] = 0.0
    k[1, 0, :] = np.arange(128, dtype=np.float32) - 63.5
    v[1, 0, :] = (np.arange(128, dtype=np.float32) - 64.0) * 0.5
    k[2] *= 1e4
    v[2] *= 1e-6
    k[3, :, :] = 127.0
    v[3, :, :] = -7.0
    out["in_crc"] = np.array([crc(k), crc(v)], np.uint32)
    out["in_k"], out["in_v"] = k, v
    for int4 in (False, True):
        ks, vs = rg.kv_quantize(k, v, int4=int4)
        tag = "int4" if int4 else "int8"
        out["kslots_" + tag], out["vslots_" + tag] = ks, vs
    q = oracle.fill_normal((64, 128), SEED, 1)
    kk = oracle.fill_normal((8, 128), SEED, 2)
    w = (1.0 + 0.02 * oracle.fill_normal((2, 128), SEED, 3)).astype(np.float32)
    inv, af = oracle.rope_table()
    inv4, af4 = oracle.rope_table(yarn=1, factor=4.0)
    for name, (tab, a, pos, st, j, ja) in {
        "p0": (inv, af, 0, 1, 0, 0), "p4096": (inv, af, 4096, 1, 0, 0),
        "yarn4_p1048575": (inv4, af4, 1048575, 1, 0, 0), "stride7_p300": (inv, af, 300, 7, 0, 0),
        "jump_p50": (inv, af, 50, 1, 300000, 40),
    }.items():
        gq, gk = rg.qk_norm_rope(q, kk, w[0], w[1], pos, tab, a, st, j, ja)
        out["gpu_normrope_%s_q" % name], out["gpu_normrope_%s_k" % name] = gq, gk
    os.makedirs(outdir, exist_ok=True)
    np.savez_compressed(os.path.join(outdir, "ref_gpu.npz"), **out)
    print("wrote", os.path.join(outdir, "ref_gpu.npz"))


if __name__ == "__main__":
    if len(sys.argv) >= 3 and sys.argv[1] == "--gpu":
        gpu_fixtures(sys.argv[2])
    else:
        cpu_fixtures()
