"""ctypes binding of libhy3attn.so: one prototype per symbol of include/hy3_attn.h."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhy3attn.so")


class Hy3AttnError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("hy3attn error %d: %s" % (code, msg))
        self.code = code


class Config(C.Structure):
    """Mirror of hy3a_config (include/hy3_attn.h)."""
    _fields_ = [("kv_dtype", C.c_int), ("n_layers", C.c_int), ("kv_head_begin", C.c_int), ("kv_head_count", C.c_int),
                ("max_seqs", C.c_int), ("max_batch", C.c_int), ("max_blocks", C.c_int), ("max_blocks_per_seq", C.c_int),
                ("device", C.c_int), ("rms_eps", C.c_float)]


_vp, _i, _sz, _u64 = C.c_void_p, C.c_int, C.c_size_t, C.c_uint64
_ip = C.POINTER(C.c_int)
_llp = C.POINTER(C.c_longlong)

# name -> (restype, argtypes); the ABI test checks this table against the header.
PROTOTYPES = {
    "hy3a_default_config": (None, [C.POINTER(Config)]),
    "hy3a_create": (_i, [C.POINTER(Config), C.POINTER(_vp)]),
    "hy3a_destroy": (None, [_vp]),
    "hy3a_last_error": (C.c_char_p, [_vp]),
    "hy3a_block_bytes": (_sz, [C.POINTER(Config)]),
    "hy3a_set_stream": (_i, [_vp, _vp]),
    "hy3a_get_stream": (_vp, [_vp]),
    "hy3a_sync": (_i, [_vp]),
    "hy3a_set_rope": (_i, [_vp, C.POINTER(C.c_float), C.c_float, _i, _i, _i]),
    "hy3a_set_norm_weights": (_i, [_vp, _i, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "hy3a_seq_reserve": (_i, [_vp, _i, _i]),
    "hy3a_seq_release": (_i, [_vp, _i, _i]),
    "hy3a_seq_capacity": (_i, [_vp, _i]),
    "hy3a_free_blocks": (_i, [_vp]),
    "hy3a_batch_set": (_i, [_vp, _i, _ip, _ip, _ip]),
    "hy3a_append": (_i, [_vp, _i, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp]),
    "hy3a_decode": (_i, [_vp, _i, _vp, _sz, _vp, _sz, _vp]),
    "hy3a_decode_step": (_i, [_vp, _i, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _vp]),
    "hy3a_decode_noalloc": (_i, [_vp, _i, _vp, _sz, _vp, _sz]),
    "hy3a_shard_init": (_i, [_vp, _i, _i, _i, _i, _vp]),
    "hy3a_shard_connect": (_i, [_vp, _vp]),
    "hy3a_shard_disconnect": (_i, [_vp]),
    "hy3a_shard_connect_local": (_i, [_vp]),
    "hy3a_decode_step_sharded": (_i, [_vp, _i, _i, _vp, _sz, _vp, _sz, _vp, _sz, _vp, _sz]),
    "hy3a_merge_partials": (_i, [_vp, _vp, _i, _i, _i, _vp, _sz]),
    "hy3a_prefill": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _sz]),
    "hy3a_export_kv": (_i, [_vp, _i, _i, _i, _i, _vp, _vp]),
    "hy3a_import_kv": (_i, [_vp, _i, _i, _i, _i, _vp, _vp]),
    "hy3a_slot_bytes": (_i, [_i]),
    "hy3a_fill_random": (_i, [_vp, _i, _i, _i, _i, _u64]),
    "hy3a_launch_count": (_u64, [_vp]),
    "hy3a_decode_schedule": (_i, [_i, _ip, _i, _i, _i, _llp, _llp, _llp]),
    "hy3a_version": (C.c_char_p, []),
}

_lib = None


def load_library():
    """Load libhy3attn.so (built by ``python -m hy3_b200._build``); raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise Hy3AttnError(-3, "%s not found: build it with `python -m hy3_b200._build` "
                               "(there is no fallback implementation)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError = ABI drift, let it surface
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
