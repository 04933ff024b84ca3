"""B200-native paged KV-cache movement behind ElasticMM's engine/v0 call surface.

Python host code (block tables, transfer orchestration, the worker methods the
reference's stage engines call) sits on a C-ABI CUDA library for sm_100a
(`libemm_kv.so`, declared in include/emm_kv.h). Importing the package needs no
GPU; moving KV data does, and there is no CPU fallback.
"""
from . import _lib
from ._lib import EmmError
from .kv_pool import Context, KVPool, compact_plan, get_context

__all__ = ["Context", "KVPool", "EmmError", "compact_plan", "get_context", "_lib"]
__version__ = "0.1.0"
