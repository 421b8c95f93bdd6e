"""B200-native (sm_100a) hot path of the Tair KVCache Manager.

Sub-packages mirror the reference's own layout for the path they replace:
  kernel/   - kv_cache_manager/py_connector/kernel (gather/scatter operators, staging allocator)
  manager/  - kv_cache_manager/manager hash + match operators, batched
All compute goes through the C ABI of libkvcm_b200.so (include/kvcm_b200.h); nothing here
computes on the CPU.
"""
from . import _cabi  # noqa: F401

__all__ = ["_cabi"]
