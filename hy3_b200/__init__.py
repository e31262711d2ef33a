"""hy3_b200 -- B200 (sm_100a) attention hot path of the Hy3 architecture.

The product is the C-ABI shared library ``libhy3attn.so`` (CUDA kernels + C host layer,
declared in ``include/hy3_attn.h``).  This package is the thin host-side driver used by
the tests and the benchmark: it loads the library with ctypes and passes it device
pointers of torch tensors.  There is no CPU path: importing works anywhere (so the ABI
can be inspected), but creating a context without the library or without a B200 raises.
"""
from ._lib import LIB_PATH, load_library, Hy3AttnError  # noqa: F401
from .attn import Hy3Attn, KV_DTYPES, H, G, D, PAGE_TOKENS, PARTIAL_FLOATS  # noqa: F401
from .session import EvalSession, plan_eval  # noqa: F401
