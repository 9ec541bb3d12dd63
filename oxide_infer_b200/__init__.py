"""B200-native kernels for oxide-infer's pointer-table KV-cache path.

The compute lives in liboxi_kv.so (hand-written CUDA for sm_100a behind the C
ABI in include/oxi_kv.h); this package is the thin host side used by the tests
and the benchmark.  Importing ``ops`` loads the library and fails loudly when
it is absent — there is no CPU or PyTorch fallback.
"""
from .ops import KvPath, Linear, OxiError, PagedLayout  # noqa: F401
from .rope import rotary_tables  # noqa: F401

__all__ = ["KvPath", "Linear", "OxiError", "PagedLayout", "rotary_tables"]
