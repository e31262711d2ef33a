"""Sequence-sharded decode whose exchange is fused into the kernels: the decode epilogue stores each
rank's {m, l, acc} records into every rank's gather buffer through peer mappings, waits (bounded)
for the other ranks' records of the same (row, KV head) and folds them (rule of hy3_gpu.cu:233-247).

* world = 1 on one GPU exercises the push, the arrival counters over several rounds and the fold,
  and must equal hy3a_decode_step bit for bit;
* a wait that nothing satisfies must end with HY3A_ETIMEOUT and leave the context usable;
* world = 2 runs as two child processes on two GPUs (skipped where the box has one) and is compared
  with the oracle attention over the whole sequence."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from helpers import SEED, check_attention, slots_to_float

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dt", ["int8", "fp16"])
def test_world1_push_and_merge_equals_decode_step(cuda, oracle, dt):
    import torch
    from hy3_b200 import Hy3Attn
    lens0 = [0, 200, 3000]
    B, steps, L = len(lens0), 5, 2
    q = oracle.fill_normal((steps, L, B, 64, 128), SEED, 501)
    k = oracle.fill_normal((steps, L, B, 8, 128), SEED, 502)
    v = oracle.fill_normal((steps, L, B, 8, 128), SEED, 503)
    res = {}
    for mode in ("plain", "pushed"):
        ctx = Hy3Attn(kv_dtype=dt, n_layers=L, max_seqs=B, max_batch=B, max_tokens=4096 + 128 * B, max_tokens_per_seq=3200)
        for l in range(L):
            for s_, n0 in enumerate(lens0):
                if n0:
                    ctx.fill_random(l, s_, 0, n0, 90 + l)
        if mode == "pushed":
            ctx.shard_connect([ctx.shard_init(0, 1, L, B)])
        tq, tk, tv = (torch.from_numpy(a).to(cuda) for a in (q, k, v))
        outs = []
        for t in range(steps):
            ctx.batch_set(list(range(B)), [n0 + t for n0 in lens0])
            for l in range(L):
                if mode == "pushed":
                    o = torch.full((B, 64, 128), 7.0, dtype=torch.float32, device=cuda)
                    ctx.decode_step_sharded(l, l, tq[t, l], tk[t, l], tv[t, l], out=o)
                else:
                    o = ctx.decode_step(l, tq[t, l], tk[t, l], tv[t, l])
                outs.append(o)
        ctx.sync()
        res[mode] = torch.stack(outs).cpu().numpy()
        ctx.close()
    assert np.array_equal(res["plain"], res["pushed"]), "max diff %.3g" % np.abs(res["plain"] - res["pushed"]).max()


def test_wait_for_a_silent_peer_runs_out_with_a_status(cuda, oracle):
    """world = 2 with a stand-in for rank 1 that never pushes: the kernel's wait must give up after about a
    second, hy3a_sync must report HY3A_ETIMEOUT, and the context must still decode correctly afterwards."""
    import time
    import torch
    from hy3_b200 import Hy3Attn, Hy3AttnError
    ctx = Hy3Attn(kv_dtype="int8", n_layers=2, max_batch=1, max_tokens=1024)
    ctx.shard_init(0, 2, 2, 1)
    ctx.shard_connect_local()
    ctx.fill_random(0, 0, 0, 300, 5)
    ctx.fill_random(1, 0, 0, 300, 6)
    ctx.batch_set([0], [300])
    q = torch.from_numpy(oracle.fill_normal((1, 64, 128), SEED, 9)).to(cuda)
    kv = torch.from_numpy(oracle.fill_normal((2, 1, 8, 128), SEED, 10)).to(cuda)
    t0 = time.time()
    ctx.decode_step_sharded(0, 0, q, kv[0], kv[1])
    ctx.decode_step_sharded(1, 1, q, kv[0], kv[1])      # later waits return at once while the error word is set
    with pytest.raises(Hy3AttnError) as ei:
        ctx.sync()
    assert ei.value.code == -6
    assert time.time() - t0 < 20.0
    got = ctx.decode(0, q)
    ctx.sync()
    ks, vs = ctx.export_kv(0, 0, 0, 301)
    check_attention(got[0].cpu().numpy(), oracle.attention(q[0].cpu().numpy(), slots_to_float(oracle, ks, "int8"), slots_to_float(oracle, vs, "int8")), "after timeout")
    ctx.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_world2_two_gpus(cuda):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", env["MASTER_PORT"], os.path.join(ROOT, "tests", "shard_peer_worker.py")]
    r = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "SHARD_PEER_OK" in r.stdout
