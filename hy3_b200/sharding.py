"""Multi-GPU decode, one process per GPU (torch.distributed over NCCL for the exchange).

Two partitions of the attention path, neither present in the single-GPU reference:

* by KV head  -- rank r owns KV heads [r*8/W, (r+1)*8/W) of every cache and the matching query
  heads; attention needs NO collective, outputs stay head-sharded (kv_head_range()).
* by sequence -- rank r holds a contiguous token range of every sequence; each rank runs the same
  split-KV kernel over its range and emits one unnormalised {m, l, acc[128]} record per head (the
  record of hy3_gpu.cu:183-230); ONE all-gather of those records per layer-step and a local fold in
  rank order with the rule of attention_reduce_kernel (hy3_gpu.cu:233-247) gives every rank the same
  bits.  The newest token is appended on the rank that owns the tail of the sequence only.

The compute callables are injected so that the exchange logic can run on CPU ranks (gloo) in tests.
"""
import datetime

import numpy as np

PARTIAL_FLOATS = 130
ETIMEOUT = -6       # HY3A_ETIMEOUT of include/hy3_attn.h: the status a bounded wait returns when it runs out


class ExchangeError(RuntimeError):
    """The all-gather of a layer's records did not complete (a rank never joined, left, or the collective failed).
    `status` is the library's time-out status; the local records of the step are intact."""

    def __init__(self, status, message):
        RuntimeError.__init__(self, message)
        self.status = status


def kv_head_range(rank, world, n_kv_heads=8):
    """(first KV head, count) owned by `rank`; world must divide 8."""
    if n_kv_heads % world:
        raise ValueError("world size %d does not divide %d KV heads" % (world, n_kv_heads))
    per = n_kv_heads // world
    return rank * per, per


def sequence_range(rank, world, ntok, align=128):
    """Contiguous, page-aligned token range [t0, t1) of a sequence of ntok tokens owned by `rank`.
    Ranges are cut at multiples of `align`; the last rank takes the remainder (and new tokens)."""
    pages = (ntok + align - 1) // align
    per = pages // world
    extra = pages % world
    p0 = rank * per + min(rank, extra)
    p1 = p0 + per + (1 if rank < extra else 0)
    return min(p0 * align, ntok), min(p1 * align, ntok)


class SequenceShardedDecode:
    """Per-layer decode step of a sequence-sharded cache: local partials -> all-gather -> merge.

    The two halves are separate methods so that a caller whose layers are independent (or that has
    other work between attention and its consumer) can run the exchange of layer l on a side
    stream while layer l+1 streams its KV: `partial(layer, q, slot)` then, later,
    `exchange_merge(slot, out)`; `n_slots` buffer sets let that many exchanges be in flight."""

    def __init__(self, partial_fn, merge_fn, all_gather_fn, world, n_rows, n_heads, empty_like, n_slots=1, timeout_s=None):
        """partial_fn(layer, q, partial_buf): fill [n_rows, n_heads, 130] for the local token range;
        merge_fn(gathered, n_parts, out): fold [world, n_rows, n_heads, 130] in rank order;
        all_gather_fn(gathered, local): the collective -- it may return a work handle (wait(timeout) -> bool);
        empty_like(shape): buffer factory.
        timeout_s: how long exchange_merge waits for the other ranks before it raises ExchangeError (None: the
        collective's own time-out applies; the reference has no multi-rank path and exits on any CUDA error,
        hy3_gpu.cu:17-20)."""
        self.partial_fn, self.merge_fn, self.all_gather_fn = partial_fn, merge_fn, all_gather_fn
        self.world, self.n_rows, self.n_heads = world, n_rows, n_heads
        self.timeout_s = timeout_s
        self.local = [empty_like((n_rows, n_heads, PARTIAL_FLOATS)) for _ in range(n_slots)]
        self.gathered = [empty_like((world, n_rows, n_heads, PARTIAL_FLOATS)) for _ in range(n_slots)]

    def partial(self, layer, q, slot=0):
        self.partial_fn(layer, q, self.local[slot])

    def exchange_merge(self, slot, out):
        """All-gather of the slot's records and the fold.  Raises ExchangeError (status ETIMEOUT) when the other ranks do
        not deliver within timeout_s; `out` is then untouched and the object stays usable: detach() continues on this
        rank's tokens alone."""
        if self.world == 1:
            self.merge_fn(self.local[slot], 1, out)
            return out
        try:
            work = self.all_gather_fn(self.gathered[slot], self.local[slot])
            if work is not None and hasattr(work, "wait"):
                done = work.wait(datetime.timedelta(seconds=self.timeout_s)) if self.timeout_s is not None else work.wait()
                if done is False:
                    raise ExchangeError(ETIMEOUT, "exchange_merge: the all-gather did not complete within %.1f s" % self.timeout_s)
        except ExchangeError:
            raise
        except RuntimeError as e:       # torch.distributed reports a timed-out or broken collective as RuntimeError
            raise ExchangeError(ETIMEOUT, "exchange_merge: the all-gather failed or timed out (%s)" % str(e).splitlines()[0]) from e
        self.merge_fn(self.gathered[slot], self.world, out)
        return out

    def detach(self):
        """Continue without the other ranks (after an ExchangeError): the fold then covers this rank's records only."""
        self.world = 1

    def step(self, layer, q, out):
        self.partial(layer, q, 0)
        return self.exchange_merge(0, out)


def make_cuda_sharded_decode(ctx, n_rows, group=None, n_slots=1, timeout_s=None):
    """Wire SequenceShardedDecode to a Hy3Attn context and torch.distributed (NCCL).  With timeout_s the all-gather is
    issued as an asynchronous work item and waited for on the host for at most that long."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    dev = torch.device("cuda", torch.cuda.current_device())
    n_heads = 8 * ctx.kv_head_count

    def partial_fn(layer, q, buf):
        if isinstance(q, tuple):            # (q_in, k_in, v_in): fused step on pre-norm rows
            ctx.decode_step(layer, q[0], q[1], q[2], partials=buf)
        else:
            ctx.decode(layer, q, partials=buf)

    def merge_fn(gathered, n_parts, out):
        ctx.merge_partials(gathered, n_parts, n_rows, n_heads, out)

    def all_gather_fn(gathered, local):
        if timeout_s is None:
            dist.all_gather_into_tensor(gathered, local, group=group)      # stream-ordered, no host wait (graph capture safe)
            return None
        return dist.all_gather_into_tensor(gathered, local, group=group, async_op=True)

    def empty(shape):
        return torch.empty(shape, dtype=torch.float32, device=dev)

    return SequenceShardedDecode(partial_fn, merge_fn, all_gather_fn, world, n_rows, n_heads, empty, n_slots, timeout_s)


def merge_partials_numpy(gathered):
    """Reference fold used by CPU tests of the exchange logic: [W, rows, heads, 130] -> [rows, heads, 128]."""
    W, R, Hn, _ = gathered.shape
    out = np.zeros((R, Hn, 128), np.float32)
    for r in range(R):
        for h in range(Hn):
            ms, ss, ov = -np.inf, np.float32(0), np.zeros(128, np.float32)
            for s in range(W):
                pm, pl = gathered[s, r, h, 0], gathered[s, r, h, 1]
                if not pl > 0:
                    continue
                nm = max(ms, pm)
                os_, rs = np.float32(np.exp(ms - nm)), np.float32(np.exp(pm - nm))
                ss = ss * os_ + pl * rs
                ov = ov * os_ + gathered[s, r, h, 2:] * rs
                ms = nm
            out[r, h] = ov / ss if ss > 0 else 0
    return out
