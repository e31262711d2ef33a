"""The drop-in boundary: every symbol include/*.h declares is exported by the built libraries -- the attention-level
ABI (hy3_attn.h, libhy3attn.so, bound by the ctypes table) and the reference engine's own backend API (hy3_gpu_dropin.h,
libhy3_gpu.so: hy3_gpu_init / hy3_gpu_free / hy3_eval_gpu); no compute is called (runs without a GPU)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hy3a?_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    import hy3_b200
    if not os.path.exists(hy3_b200.LIB_PATH):
        from hy3_b200 import _build
        _build.build()
    return hy3_b200.load_library()


def test_attn_header_symbols_exported_and_bound(lib):
    from hy3_b200._lib import PROTOTYPES
    syms = declared_symbols("hy3_attn.h")
    assert len(syms) >= 25
    for s in syms:
        assert hasattr(lib, s), "library does not export %s" % s
    assert sorted(PROTOTYPES) == syms, "ctypes table and header disagree"


def test_engine_api_symbols_exported():
    """The three symbols the reference engine binds (hy3_gpu.h:6-8, hy3.h:79) and what the library expects from the
    engine in return (hy3.h:74, :84-85), read from the dynamic symbol table."""
    import subprocess
    from hy3_b200 import _build
    if not os.path.exists(_build.DROPIN_LIB):
        if _build.reference_dir() is None:
            pytest.skip("libhy3_gpu.so is not built and the reference checkout is not here to build it")
        _build.build()
    out = subprocess.run(["nm", "-D", _build.DROPIN_LIB], capture_output=True, text=True, check=True).stdout
    defined = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    undefined = {ln.split()[-1] for ln in out.splitlines() if ln.strip().startswith("U ")}
    syms = declared_symbols("hy3_gpu_dropin.h")
    assert {"hy3_gpu_init", "hy3_gpu_free", "hy3_eval_gpu"} <= set(syms)
    for s in syms:
        assert s in defined, "libhy3_gpu.so does not export %s" % s
    assert {"hy3_rope_get_params", "forward_layer_dense", "forward_layer_moe"} <= undefined
    assert {s for s in declared_symbols("hy3_attn.h")} <= defined       # the attention ABI is part of the same object set


def test_config_struct_layout(lib):
    from hy3_b200._lib import Config
    cfg = Config()
    lib.hy3a_default_config(C.byref(cfg))
    assert (cfg.kv_dtype, cfg.n_layers, cfg.kv_head_begin, cfg.kv_head_count) == (1, 80, 0, 8)
    assert cfg.max_blocks == 64 and abs(cfg.rms_eps - 1e-5) < 1e-12 and cfg.device == -1
    assert lib.hy3a_block_bytes(C.byref(cfg)) == 80 * 8 * 33280     # = 128 tokens * 80 layers * 2 * 1040 B
    cfg.kv_dtype = 2
    assert lib.hy3a_block_bytes(C.byref(cfg)) == 80 * 8 * 16896     # 128 * 80 * 2 * 528
    cfg.kv_dtype = 0
    assert lib.hy3a_block_bytes(C.byref(cfg)) == 80 * 8 * 65536     # 128 * 80 * 2 * 2048
    assert [lib.hy3a_slot_bytes(d) for d in (0, 1, 2, 3)] == [2048, 1040, 528, -1]


def test_create_fails_loudly_without_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    import hy3_b200
    with pytest.raises(hy3_b200.Hy3AttnError) as e:
        hy3_b200.Hy3Attn()
    assert "no CPU path" in str(e.value)


def test_bad_config_rejected(lib):
    from hy3_b200._lib import Config
    cfg = Config()
    lib.hy3a_default_config(C.byref(cfg))
    cfg.kv_head_begin, cfg.kv_head_count = 6, 4
    h = C.c_void_p()
    assert lib.hy3a_create(C.byref(cfg), C.byref(h)) == -1 and not h.value
    assert b"kv head range" in lib.hy3a_last_error(None)
