"""Host-side mirror of the ATTENTION side of the reference's evaluation entry point.

`hy3_eval_gpu` (hy3_gpu.cu:844-961) takes a run of tokens, derives their positions from the model's
`cache_len` (counted in slots = tokens x layers and owned -- and mutated -- by the callers: hy3.c:1514 sets it back
to a reused prefix, hy3.c:960 zeroes it), feeds all but the last token through `prefill_chunk_gpu`
(hy3_gpu.cu:811-841) in chunks of HY3_PREFILL_CHUNK when that is set, runs the remaining tokens one by one through
the decode path, and advances `cache_len`.  `EvalSession` keeps exactly that contract for the part of a layer this
library replaces: per layer it asks the caller for the pre-norm q/k/v rows of the tokens (what the QKV projection
produced) and hands back the attention output (what the output projection consumes).  The projections, the MoE and
the logits stay with the caller.

Environment switches read once at construction, as the reference does (hy3_gpu.cu:598-606):
  HY3_KV_INT4=1      INT4 cache, else INT8;  HY3_KV_FP16=1 (new) selects the FP16 cache
  HY3_PREFILL_CHUNK  N > 0: chunk path for calls with more than one token (last token via the decode path)
  HY3_POS_STRIDE, HY3_POS_JUMP, HY3_POS_JUMP_AT   RoPE angle only (hy3_gpu.cu:148-152)
"""
import os
import sys

from .attn import Hy3Attn


def plan_eval(cache_len, n_tokens, n_layers, chunk):
    """The order in which `hy3_eval_gpu` walks n_tokens new tokens (pure host arithmetic).

    Returns a list of ("chunk", t0, nq) and ("token", t) items; positions come from cache_len // n_layers
    (hy3_gpu.cu:814, :870).  With chunk > 0 and more than one token, all tokens but the last go through chunks of at
    most `chunk` (hy3_gpu.cu:857-866); everything else goes token by token."""
    if n_tokens < 0 or cache_len < 0 or n_layers < 1:
        raise ValueError("plan_eval: negative argument")
    t = cache_len // n_layers
    ops = []
    start = 0
    if chunk > 0 and n_tokens > 1:
        npre = n_tokens - 1
        off = 0
        while off < npre:
            c = min(chunk, npre - off)
            ops.append(("chunk", t + off, c))
            off += c
        start = npre
    for i in range(start, n_tokens):
        ops.append(("token", t + i))
    return ops


def read_env(env=None):
    """The reference's switches as a dict (missing or malformed values fall back like atoi does: to 0)."""
    env = os.environ if env is None else env

    def num(name, default=0):
        try:
            return int(env.get(name, default))
        except (TypeError, ValueError):
            return 0
    kv = "int4" if num("HY3_KV_INT4") != 0 else ("fp16" if num("HY3_KV_FP16") != 0 else "int8")
    stride = num("HY3_POS_STRIDE", 1)
    return {"kv_dtype": kv, "chunk": max(num("HY3_PREFILL_CHUNK"), 0), "pos_stride": stride if stride > 0 else 1,
            "pos_jump": num("HY3_POS_JUMP"), "pos_jump_at": num("HY3_POS_JUMP_AT")}


class EvalSession:
    """The attention state of one model instance: a KV cache for one conversation plus `cache_len`.

    qkv_fn(layer, t0, n) -> (q [n,64,128], k [n,8,128], v [n,8,128]) fp32 CUDA tensors: the pre-norm rows of the tokens at
    positions t0 .. t0+n-1 (the reference's QKV projection output, hy3_gpu.cu:749 / :822).
    out_fn(layer, t0, n, attn) receives the attention output [n,64,128] fp32 (the reference's d_attn_out / d_pf_ao);
    the tensor is reused by the next call.

    `cache_len` is a plain attribute in slots (tokens x n_layers), as in hy3_model: set it back to reuse a prefix
    (hy3.c:1514) or to 0 to start over (hy3.c:960); KV beyond it is dead and is overwritten by the next tokens."""

    def __init__(self, n_layers=80, max_tokens=8192, device=None, inv_freq=None, attn_factor=1.0, norm_weights=None,
                 rms_eps=1e-5, env=None, log=sys.stderr):
        cfg = read_env(env)
        self.n_layers, self.chunk, self.kv_dtype = n_layers, cfg["chunk"], cfg["kv_dtype"]
        self.ctx = Hy3Attn(kv_dtype=self.kv_dtype, n_layers=n_layers, max_seqs=1, max_batch=max(self.chunk, 1),
                           max_tokens=max_tokens, device=device, rms_eps=rms_eps)
        if inv_freq is not None:
            self.ctx.set_rope(inv_freq, attn_factor, cfg["pos_stride"], cfg["pos_jump"], cfg["pos_jump_at"])
        elif (cfg["pos_stride"], cfg["pos_jump"], cfg["pos_jump_at"]) != (1, 0, 0):
            raise ValueError("HY3_POS_* are set: pass the RoPE table (inv_freq, attn_factor) they apply to")
        if norm_weights is not None:
            for layer, (qw, kw) in enumerate(norm_weights):
                self.ctx.set_norm_weights(layer, qw, kw)
        self.cache_len = 0
        self._q16 = None
        self._out = None
        if log is not None:
            if self.chunk > 0:
                print("hy3_gpu: chunked prefill enabled (chunk=%d tokens)" % self.chunk, file=log)
            # the needle harness looks for "INT4 KV" / "INT8 KV" in this line (eval/hy3_needle.py:103)
            print("hy3_gpu: initialized (%d layers, %s KV, online attn)" % (n_layers, self.kv_dtype.upper()), file=log)

    def close(self):
        self.ctx.close()

    def reset(self):
        """hy3_reset_context (hy3.c:960)."""
        self.cache_len = 0

    def eval(self, n_tokens, qkv_fn, out_fn):
        """Feed n_tokens new tokens.  Returns the value hy3_eval_gpu stores in *pos: cache_len after the call."""
        import torch
        if n_tokens < 1:
            return self.cache_len
        ctx, L = self.ctx, self.n_layers
        if self.cache_len % L:
            raise ValueError("cache_len %d is not a multiple of the layer count %d" % (self.cache_len, L))
        for op in plan_eval(self.cache_len, n_tokens, L, self.chunk):
            if op[0] == "chunk":
                _, t0, nq = op
                ctx.batch_set([0] * nq, list(range(t0, t0 + nq)))
                for layer in range(L):
                    q, k, v = qkv_fn(layer, t0, nq)
                    if self._q16 is None or self._q16.device != q.device:
                        self._q16 = torch.empty((max(self.chunk, 1), 64, 128), dtype=torch.float16, device=q.device)
                        self._out = torch.empty((max(self.chunk, 1), 64, 128), dtype=torch.float32, device=q.device)
                    q16 = self._q16[:nq]
                    ctx.append(layer, q, k, v, q_out=False, q_out16=q16)
                    out_fn(layer, t0, nq, ctx.prefill(layer, 0, t0, q16, out=self._out[:nq]))
                self.cache_len = (t0 + nq) * L
            else:
                t = op[1]
                ctx.batch_set([0], [t])
                for layer in range(L):
                    q, k, v = qkv_fn(layer, t, 1)
                    if self._out is None or self._out.device != q.device:
                        self._out = torch.empty((max(self.chunk, 1), 64, 128), dtype=torch.float32, device=q.device)
                    out_fn(layer, t, 1, ctx.decode_step(layer, q, k, v, out=self._out[:1]))
                self.cache_len = (t + 1) * L
        return self.cache_len
