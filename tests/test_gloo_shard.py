"""The multi-GPU exchange logic on CPU ranks (gloo, world size 2): sequence-sharded decode =
per-rank partials {m, l, acc} -> one all-gather -> fold in rank order; KV-head sharding = no
collective.  The compute callables are the oracle's (the CUDA ones are injected the same way in
hy3_b200/sharding.py: make_cuda_sharded_decode)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ntok, q, K, V, ret):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import oracle
    from hy3_b200.sharding import SequenceShardedDecode, sequence_range, merge_partials_numpy
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    t0, t1 = sequence_range(rank, world, ntok)
    n_rows = q.shape[0]

    def partial_fn(layer, qq, buf):
        for r in range(n_rows):
            # row 1 is a short sequence that lives entirely on rank 0: other ranks emit the empty record
            hi = min(t1, 200) if r == 1 else t1
            lo = min(t0, hi)
            buf[r] = torch.from_numpy(oracle.attention_partial(qq[r], K, V, lo, hi))

    def all_gather_fn(gathered, local):
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local)
        for i, p in enumerate(parts):
            gathered[i] = p

    def merge_fn(gathered, n_parts, out):
        g = gathered.numpy() if n_parts > 1 else gathered.numpy()[None]
        out[:] = torch.from_numpy(merge_partials_numpy(g))

    sd = SequenceShardedDecode(partial_fn, merge_fn, all_gather_fn, world, n_rows, 64,
                               lambda shape: torch.zeros(shape, dtype=torch.float32))
    out = torch.zeros((n_rows, 64, 128))
    sd.step(0, q, out)
    # every rank ends with identical bits (fixed fold order)
    mine = out.numpy().copy()
    allo = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(allo, out)
    same = all(np.array_equal(mine, o.numpy()) for o in allo)
    if rank == 0:
        ret.put((mine, same, (t0, t1)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_sequence_sharded_decode_gloo(oracle, world):
    import torch.multiprocessing as mp
    ntok = 1000
    q = oracle.fill_normal((2, 64, 128), 7, 1)
    K = oracle.fill_normal((ntok, 8, 128), 7, 2)
    V = oracle.fill_normal((ntok, 8, 128), 7, 3)
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ntok, q, K, V, ret)) for r in range(world)]
    for p in procs:
        p.start()
    out, same, rng = ret.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same, "ranks disagree after the merge"
    assert np.abs(out[0] - oracle.attention(q[0], K, V)).max() < 2e-6
    assert np.abs(out[1] - oracle.attention(q[1], K[:200], V[:200])).max() < 2e-6


def test_ranges():
    from hy3_b200.sharding import kv_head_range, sequence_range
    assert [kv_head_range(r, 4) for r in range(4)] == [(0, 2), (2, 2), (4, 2), (6, 2)]
    assert kv_head_range(0, 1) == (0, 8) and kv_head_range(7, 8) == (7, 1)
    with pytest.raises(ValueError):
        kv_head_range(0, 3)
    for ntok in (1, 127, 128, 129, 1000, 262144, 1048576):
        for world in (1, 2, 4, 8):
            rs = [sequence_range(r, world, ntok) for r in range(world)]
            assert rs[0][0] == 0 and rs[-1][1] == ntok
            assert all(a[1] == b[0] for a, b in zip(rs[:-1], rs[1:]))
            assert all(a[0] % 128 == 0 for a in rs if a[1] > a[0])      # non-empty shards start on page boundaries
            sizes = [(b - a + 127) // 128 for a, b in rs]
            assert max(sizes) - min(sizes) <= 1


# ------------------------------------------------------------------ failure path: a rank that never enters the exchange
EXCHANGE_TIMEOUT_S = 3.0


def _failing_worker(rank, world, port, ntok, q, K, V, ret):
    """Rank 1 computes nothing and never enters the all-gather (it sleeps past the time-out and leaves); rank 0 must get
    an error status from exchange_merge within the stated time-out, not hang, and decode correctly afterwards alone."""
    sys.path.insert(0, ROOT)
    import time
    import torch
    import torch.distributed as dist
    import oracle
    from hy3_b200.sharding import SequenceShardedDecode, ExchangeError, ETIMEOUT, sequence_range, merge_partials_numpy
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if rank != 0:
        time.sleep(EXCHANGE_TIMEOUT_S + 4.0)          # between steps: nothing of this rank is in flight
        os._exit(0)
    t0, t1 = sequence_range(rank, world, ntok)
    n_rows = q.shape[0]

    def partial_fn(layer, qq, buf):
        for r in range(n_rows):
            buf[r] = torch.from_numpy(oracle.attention_partial(qq[r], K, V, t0, t1))

    def all_gather_fn(gathered, local):
        parts = [torch.empty_like(local) for _ in range(world)]
        work = dist.all_gather(parts, local, async_op=True)

        class Handle:
            def wait(self, timeout=None):
                ok = work.wait(timeout) if timeout is not None else work.wait()
                for i, p in enumerate(parts):
                    gathered[i] = p
                return ok
        return Handle()

    def merge_fn(gathered, n_parts, out):
        g = gathered.numpy() if n_parts > 1 else gathered.numpy()[None]
        out[:] = torch.from_numpy(merge_partials_numpy(g))

    sd = SequenceShardedDecode(partial_fn, merge_fn, all_gather_fn, world, n_rows, 64,
                               lambda shape: torch.zeros(shape, dtype=torch.float32), timeout_s=EXCHANGE_TIMEOUT_S)
    out = torch.full((n_rows, 64, 128), 7.0)
    sd.partial(0, q, 0)
    t_start = time.monotonic()
    status, msg = 0, ""
    try:
        sd.exchange_merge(0, out)
    except ExchangeError as e:
        status, msg = e.status, str(e)
    waited = time.monotonic() - t_start
    untouched = bool((out == 7.0).all())
    # afterwards: this rank continues on its own tokens
    sd.detach()
    sd.step(0, q, out)
    ret.put((status, status == ETIMEOUT, msg, waited, untouched, out.numpy().copy(), (t0, t1)))
    ret.close()
    ret.join_thread()                                 # the queue's feeder thread must have sent the item before the hard exit
    os._exit(0)                                       # the process group is broken: leave without the collective teardown


def test_exchange_times_out_when_a_rank_never_joins(oracle):
    import torch.multiprocessing as mp
    ntok, world = 600, 2
    q = oracle.fill_normal((1, 64, 128), 9, 1)
    K = oracle.fill_normal((ntok, 8, 128), 9, 2)
    V = oracle.fill_normal((ntok, 8, 128), 9, 3)
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, ntok, q, K, V, ret)) for r in range(world)]
    for p in procs:
        p.start()
    status, is_timeout, msg, waited, untouched, out, (t0, t1) = ret.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert status != 0 and is_timeout, "exchange_merge returned no error status: %r" % msg
    assert waited < EXCHANGE_TIMEOUT_S + 10.0, "exchange_merge took %.1f s" % waited
    assert untouched, "a failed exchange must not write the output"
    # rank 0 alone afterwards: attention over its own token range
    assert np.abs(out[0] - oracle.attention(q[0], K[t0:t1], V[t0:t1])).max() < 2e-6
