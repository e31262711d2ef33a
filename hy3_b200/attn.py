"""Host-side driver of the attention context (mirrors the call order of the reference's
encode_layer_gpu / prefill_chunk_gpu, hy3_gpu.cu:744-763 and :811-841, one method per step)."""
import ctypes as C

import numpy as np

from ._lib import Config, Hy3AttnError, load_library

H, G, D = 64, 8, 128
PAGE_TOKENS = 128
PARTIAL_FLOATS = 130
KV_DTYPES = {"fp16": 0, "int8": 1, "int4": 2}


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


class Hy3Attn:
    """One KV-cache context on one GPU.  Tensors are torch CUDA tensors on that GPU."""

    def __init__(self, kv_dtype="int8", n_layers=80, kv_head_begin=0, kv_head_count=G, max_seqs=1, max_batch=512,
                 max_tokens=8192, max_tokens_per_seq=None, device=None, rms_eps=1e-5, stream=None):
        self.lib = load_library()
        self.kv_dtype = kv_dtype
        cfg = Config()
        self.lib.hy3a_default_config(C.byref(cfg))
        cfg.kv_dtype = KV_DTYPES[kv_dtype]
        cfg.n_layers = n_layers
        cfg.kv_head_begin, cfg.kv_head_count = kv_head_begin, kv_head_count
        cfg.max_seqs, cfg.max_batch = max_seqs, max_batch
        cfg.max_blocks = (max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS + (max_seqs - 1)
        per_seq = max_tokens if max_tokens_per_seq is None else max_tokens_per_seq
        cfg.max_blocks_per_seq = (per_seq + PAGE_TOKENS - 1) // PAGE_TOKENS
        cfg.device = -1 if device is None else int(device)
        cfg.rms_eps = rms_eps
        self.cfg = cfg
        self.n_layers, self.kv_head_begin, self.kv_head_count = n_layers, kv_head_begin, kv_head_count
        h = C.c_void_p()
        rc = self.lib.hy3a_create(C.byref(cfg), C.byref(h))
        if rc:
            raise Hy3AttnError(rc, self.lib.hy3a_last_error(None).decode())
        self.h = h
        self.batch_n = 0
        if stream is None:
            # work is enqueued on torch's current stream, so that it is ordered with the allocations,
            # fills and copies torch does for the tensors handed to this object
            import torch
            stream = torch.cuda.current_stream(cfg.device if cfg.device >= 0 else None)
        self.set_stream(stream)

    # ---- plumbing
    def _chk(self, rc):
        if rc:
            raise Hy3AttnError(rc, self.lib.hy3a_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None):
            self.lib.hy3a_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_stream(self, stream):
        """stream: a torch.cuda.Stream or a raw cudaStream_t integer."""
        raw = getattr(stream, "cuda_stream", stream)
        self._chk(self.lib.hy3a_set_stream(self.h, C.c_void_p(raw)))

    def use_torch_stream(self):
        import torch
        self.set_stream(torch.cuda.current_stream())

    def sync(self):
        self._chk(self.lib.hy3a_sync(self.h))

    @property
    def launches(self):
        return int(self.lib.hy3a_launch_count(self.h))

    def block_bytes(self):
        return int(self.lib.hy3a_block_bytes(C.byref(self.cfg)))

    # ---- parameters
    def set_rope(self, inv_freq, attn_factor=1.0, pos_stride=1, pos_jump=0, pos_jump_at=0):
        inv = np.ascontiguousarray(inv_freq, np.float32)
        assert inv.size == 64
        self._chk(self.lib.hy3a_set_rope(self.h, inv.ctypes.data_as(C.POINTER(C.c_float)), attn_factor, pos_stride,
                                         pos_jump, pos_jump_at))

    def set_norm_weights(self, layer, qw, kw):
        qw = np.ascontiguousarray(qw, np.float32)
        kw = np.ascontiguousarray(kw, np.float32)
        assert qw.size == D and kw.size == D
        fp = C.POINTER(C.c_float)
        self._chk(self.lib.hy3a_set_norm_weights(self.h, layer, qw.ctypes.data_as(fp), kw.ctypes.data_as(fp)))

    # ---- sequences
    def seq_reserve(self, seq, ntok):
        self._chk(self.lib.hy3a_seq_reserve(self.h, seq, ntok))

    def seq_release(self, seq, keep_ntok=0):
        self._chk(self.lib.hy3a_seq_release(self.h, seq, keep_ntok))

    def seq_capacity(self, seq):
        return int(self.lib.hy3a_seq_capacity(self.h, seq))

    def free_blocks(self):
        return int(self.lib.hy3a_free_blocks(self.h))

    def batch_set(self, seq_ids, slots, rope_pos=None):
        s = np.ascontiguousarray(seq_ids, np.int32)
        t = np.ascontiguousarray(slots, np.int32)
        p = t if rope_pos is None else np.ascontiguousarray(rope_pos, np.int32)
        assert s.size == t.size == p.size
        ip = C.POINTER(C.c_int)
        self._chk(self.lib.hy3a_batch_set(self.h, s.size, s.ctypes.data_as(ip), t.ctypes.data_as(ip), p.ctypes.data_as(ip)))
        self.batch_n = int(s.size)

    # ---- hot path
    def append(self, layer, q, k, v, q_out=None, q_out16=None):
        """q [n,64,128] / k,v [n,8,128] fp32 (row stride free, rows dense).  Returns q_out (fp32); q_out=False with a
        q_out16 buffer writes the 16-bit queries only (the chunked prefill reads nothing else)."""
        import torch
        n = self.batch_n
        assert (k is None) == (v is None)
        for t in (q, k, v):
            assert t is None or (t.shape[0] == n and t.dtype == torch.float32 and t.stride(-1) == 1 and t.stride(-2) == D)
        if q_out is False:
            assert q_out16 is not None
            q_out = None
        elif q_out is None:
            q_out = torch.empty((n, H, D), dtype=torch.float32, device=q.device)
        if q_out16 is not None:
            assert q_out16.dtype == torch.float16 and q_out16.is_contiguous() and q_out16.numel() == n * H * D
        self._chk(self.lib.hy3a_append(self.h, layer, _ptr(q), q.stride(0), _ptr(k), 0 if k is None else k.stride(0),
                                       _ptr(v), 0 if v is None else v.stride(0),
                                       _ptr(q_out), 0 if q_out is None else q_out.stride(0), _ptr(q_out16)))
        return q_out

    def decode(self, layer, q, out=None, partials=None):
        """q [n,64,128] fp32 -> out [n,64,128] fp32 (owned heads written) or partials [n, 8*kv_heads, 130]."""
        import torch
        n = self.batch_n
        assert q.shape[0] == n and q.dtype == torch.float32 and q.stride(-1) == 1 and q.stride(-2) == D
        if partials is None and out is None:
            out = torch.zeros((n, H, D), dtype=torch.float32, device=q.device)
        if partials is not None:
            assert partials.is_contiguous() and partials.numel() == n * 8 * self.kv_head_count * PARTIAL_FLOATS
        self._chk(self.lib.hy3a_decode(self.h, layer, _ptr(q), q.stride(0), _ptr(out), 0 if out is None else out.stride(0),
                                       _ptr(partials)))
        return out if partials is None else partials

    def decode_step(self, layer, q, k, v, out=None, q_out=None, partials=None):
        """Fused append + decode of one new token per batch row (pre-norm q [n,64,128], k/v [n,8,128])."""
        import torch
        n = self.batch_n
        assert (k is None) == (v is None)
        for t in (q, k, v):
            assert t is None or (t.shape[0] == n and t.dtype == torch.float32 and t.stride(-1) == 1 and t.stride(-2) == D)
        if partials is None and out is None:
            out = torch.zeros((n, H, D), dtype=torch.float32, device=q.device)
        self._chk(self.lib.hy3a_decode_step(self.h, layer, _ptr(q), q.stride(0), _ptr(k), 0 if k is None else k.stride(0),
                                            _ptr(v), 0 if v is None else v.stride(0), _ptr(q_out),
                                            0 if q_out is None else q_out.stride(0), _ptr(out),
                                            0 if out is None else out.stride(0), _ptr(partials)))
        return out if partials is None else partials

    # ---- sequence sharding over peer memory
    def shard_init(self, rank, world, n_slots, n_rows):
        """Allocate this rank's gather buffer; returns its 64-byte IPC handle (bytes)."""
        buf = C.create_string_buffer(64)
        self._chk(self.lib.hy3a_shard_init(self.h, rank, world, n_slots, n_rows, buf))
        return bytes(buf.raw)

    def shard_connect(self, handles):
        """handles: the IPC handles of all ranks, in rank order."""
        blob = b"".join(handles)
        self._chk(self.lib.hy3a_shard_connect(self.h, C.c_char_p(blob)))

    def shard_disconnect(self):
        self._chk(self.lib.hy3a_shard_disconnect(self.h))

    def shard_connect_local(self):
        """Silent stand-ins for the other ranks (single-process bring-up and tests)."""
        self._chk(self.lib.hy3a_shard_connect_local(self.h))

    def decode_step_sharded(self, layer, slot, q, k, v, out=None):
        """hy3a_decode_step over this rank's tokens + in-kernel exchange and fold: `out` is the attention over ALL ranks' tokens."""
        if out is None:
            import torch
            out = torch.empty((self.batch_n, 64, 128), dtype=torch.float32, device=q.device)
        self._chk(self.lib.hy3a_decode_step_sharded(self.h, layer, slot, _ptr(q), q.stride(0), _ptr(k), 0 if k is None else k.stride(0),
                                                    _ptr(v), 0 if v is None else v.stride(0), _ptr(out), out.stride(0)))
        return out

    def merge_partials(self, partials, n_parts, n_rows, n_heads, out):
        assert partials.is_contiguous() and partials.numel() == n_parts * n_rows * n_heads * PARTIAL_FLOATS
        self._chk(self.lib.hy3a_merge_partials(self.h, _ptr(partials), n_parts, n_rows, n_heads, _ptr(out), out.stride(0)))
        return out

    def prefill(self, layer, seq, base_slot, q16, out=None):
        import torch
        nq = q16.shape[0]
        assert q16.dtype == torch.float16 and q16.is_contiguous()
        if out is None:
            out = torch.zeros((nq, H, D), dtype=torch.float32, device=q16.device)
        self._chk(self.lib.hy3a_prefill(self.h, layer, seq, base_slot, nq, _ptr(q16), _ptr(out), out.stride(0)))
        return out

    # ---- import / export (host numpy)
    def slot_bytes(self):
        return int(self.lib.hy3a_slot_bytes(KV_DTYPES[self.kv_dtype]))

    def export_kv(self, layer, seq, t0, n):
        ks = np.zeros((n, self.slot_bytes()), np.uint8)
        vs = np.zeros((n, self.slot_bytes()), np.uint8)
        self._chk(self.lib.hy3a_export_kv(self.h, layer, seq, t0, n, C.c_void_p(ks.ctypes.data), C.c_void_p(vs.ctypes.data)))
        return ks, vs

    def import_kv(self, layer, seq, t0, kslots, vslots):
        ks = np.ascontiguousarray(kslots, np.uint8)
        vs = np.ascontiguousarray(vslots, np.uint8)
        n = ks.shape[0]
        assert ks.shape == vs.shape == (n, self.slot_bytes())
        self._chk(self.lib.hy3a_import_kv(self.h, layer, seq, t0, n, C.c_void_p(ks.ctypes.data), C.c_void_p(vs.ctypes.data)))

    def fill_random(self, layer, seq, t0, n, seed):
        self._chk(self.lib.hy3a_fill_random(self.h, layer, seq, t0, n, C.c_uint64(seed)))


def decode_schedule(kv_lens, kv_heads, n_ctas, cta):
    """Pure host arithmetic of the decode kernel's unit split (no GPU needed)."""
    lib = load_library()
    lens = np.ascontiguousarray(kv_lens, np.int32)
    tot, u0, u1 = C.c_longlong(), C.c_longlong(), C.c_longlong()
    rc = lib.hy3a_decode_schedule(lens.size, lens.ctypes.data_as(C.POINTER(C.c_int)), kv_heads, n_ctas, cta,
                                  C.byref(tot), C.byref(u0), C.byref(u1))
    if rc:
        raise Hy3AttnError(rc, "bad schedule arguments")
    return tot.value, u0.value, u1.value
