"""Child process of test_gpu_shard_peer.py::test_world2_two_gpus (one per GPU, started by
torch.distributed.run).  Every rank holds a contiguous token range of each sequence; the tail rank
appends the new token; records travel through peer memory inside the decode kernel.  Checks:
all ranks end with identical bits; they agree with a single-GPU context holding the whole sequence
(rank 0 runs it) and, through it, with the oracle attention on the stored cache."""
import os
import sys


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import torch
    import torch.distributed as dist
    import oracle
    from helpers import SEED, check_attention, make_slots, slots_to_float
    from hy3_b200 import Hy3Attn
    from hy3_b200.sharding import sequence_range

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    dt, L, steps = "int8", 3, 6
    lens0 = [5000, 100, 0]                     # tokens cached before the first step, per sequence
    B = len(lens0)
    K = [oracle.fill_normal((n, 8, 128), SEED, 601 + i) for i, n in enumerate(lens0)]
    V = [oracle.fill_normal((n, 8, 128), SEED, 611 + i) for i, n in enumerate(lens0)]
    q = oracle.fill_normal((steps, L, B, 64, 128), SEED, 621)
    k = oracle.fill_normal((steps, L, B, 8, 128), SEED, 622)
    v = oracle.fill_normal((steps, L, B, 8, 128), SEED, 623)
    tq, tk, tv = (torch.from_numpy(a).to(dev) for a in (q, k, v))

    ctx = Hy3Attn(kv_dtype=dt, n_layers=L, max_seqs=B, max_batch=B, max_tokens=8192, max_tokens_per_seq=5632, device=dev.index)
    ranges = [sequence_range(rank, world, n) for n in lens0]
    for s_, (t0, t1) in enumerate(ranges):
        if t1 > t0:
            for l in range(L):
                ctx.import_kv(l, s_, 0, make_slots(oracle, K[s_][t0:t1], dt), make_slots(oracle, V[s_][t0:t1], dt))
    handles = [None] * world
    dist.all_gather_object(handles, ctx.shard_init(rank, world, L, B))
    ctx.shard_connect(handles)
    dist.barrier()

    owner = rank == world - 1
    outs = torch.zeros((steps, L, B, 64, 128), dtype=torch.float32, device=dev)
    for t in range(steps):
        local = [(t1 - t0) + t if owner else (t1 - t0) - 1 for (t0, t1) in ranges]
        ctx.batch_set(list(range(B)), local, [n + t for n in lens0])
        for l in range(L):
            ctx.decode_step_sharded(l, l, tq[t, l], tk[t, l] if owner else None, tv[t, l] if owner else None, out=outs[t, l])
    ctx.sync()
    mine = outs.cpu()
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    assert all(torch.equal(mine, o) for o in everyone), "ranks disagree"

    if rank == 0:
        full = Hy3Attn(kv_dtype=dt, n_layers=L, max_seqs=B, max_batch=B, max_tokens=8192, max_tokens_per_seq=5632, device=dev.index)
        for s_, n in enumerate(lens0):
            if n:
                for l in range(L):
                    full.import_kv(l, s_, 0, make_slots(oracle, K[s_], dt), make_slots(oracle, V[s_], dt))
        qo = torch.zeros((B, 64, 128), dtype=torch.float32, device=dev)
        worst = 0.0
        for t in range(steps):
            full.batch_set(list(range(B)), [n + t for n in lens0])
            for l in range(L):
                want = full.decode_step(l, tq[t, l], tk[t, l], tv[t, l], q_out=qo)
                full.sync()
                worst = max(worst, float((want - outs[t, l]).abs().max()))
        # not bit-equal: the ranks cut the sequence elsewhere than the CTAs of one GPU do; fp16 P (mma.sync kernel) differs by
        # ~1e-5, the two-digit fixed-point P of the tcgen05 kernel by ~1e-4 -- both far inside the 2e-3 bound checked below
        assert worst <= 5e-4, "sharded vs single-GPU: %g" % worst
        for s_ in range(B):                   # last step, last layer, against the oracle on the stored cache
            ks, vs = full.export_kv(L - 1, s_, 0, lens0[s_] + steps)
            check_attention(outs[-1, -1, s_].cpu().numpy(),
                            oracle.attention(qo[s_].cpu().numpy(), slots_to_float(oracle, ks, dt), slots_to_float(oracle, vs, dt)),
                            "2-GPU sharded seq %d" % s_)
        full.close()
        print("SHARD_PEER_OK worst diff vs single GPU %.3g" % worst, flush=True)
    ctx.shard_disconnect()
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
