"""nimllm_b200 -- B200 (sm_100a) grouped-query attention path for nimllm.

The product is the C-ABI library `libnimllm_attn.so` (include/nimllm_attn.h); this package
is its build script, its ctypes binding and a thin host layer named after the reference's
own procedures (KvCache, ropeFwd, attention blocks of forward / forwardCached)."""
from ._lib import BF16, F32, LIB_PATH, NimllmAttnError, lib  # noqa: F401
