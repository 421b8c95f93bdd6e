"""GPU-resident block index: the replica of MetaIndexer's table that the matchers probe
(kv_cache_manager/meta/meta_indexer.cc:419-440,650-752)."""
import ctypes
from typing import Iterable, Optional, Sequence, Tuple

import torch

from .. import _cabi

# kv_cache_manager/manager/cache_location.h:44-50
CLS_NOT_FOUND, CLS_NEW, CLS_WRITING, CLS_SERVING, CLS_DELETING = range(5)


def encode_locations(locations: Iterable[Tuple[int, int]]) -> int:
    """Value word of a key from its location map, given as (status, storage class) pairs.

    Bit c: a CLS_SERVING location of class c; bit 16+c: a location of class c whose status is not
    CLS_NOT_FOUND; bit 32: the map is non-empty.  These are exactly the facts SelectForMatch and
    ExistsForWrite (kv_cache_manager/manager/select_location_policy.cc:8-38) read."""
    word = 0
    for status, cls in locations:
        c = min(max(int(cls), 0), 15)
        word |= _cabi.VAL_NONEMPTY
        if status == CLS_SERVING:
            word |= 1 << c
        if status != CLS_NOT_FOUND:
            word |= 1 << (16 + c)
    return word


def avail_mask_from_weights(weights: Sequence[int], default_weight: int = 1) -> int:
    """Bit c set when the policy weight of storage class c is > 0; classes beyond the weight table
    get the default weight (kv_cache_manager/manager/select_location_policy.cc:40-48)."""
    mask = 0
    for c in range(16):
        w = weights[c] if c < len(weights) else default_weight
        if w > 0:
            mask |= 1 << c
    return mask


def _keys(keys: torch.Tensor, device: torch.device) -> torch.Tensor:
    """The C ABI takes dense int64 device arrays; a strided view is compacted first."""
    if keys.dtype != torch.int64 or keys.device != device:
        raise ValueError("keys must be an int64 tensor on %s" % device)
    return keys.contiguous()


class BlockIndex:
    """Handle of one device-resident index (one per instance_id, as MetaIndexerManager keeps them)."""

    def __init__(self, max_keys: int, device: Optional[torch.device] = None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        _cabi.bind_device(self.device.index)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _cabi.call("kvcm_b200_index_create", max_keys, ctypes.byref(handle))
        self._h = handle

    def close(self):
        if getattr(self, "_h", None):
            _cabi.lib().kvcm_b200_index_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except TypeError:  # interpreter shutdown: the module globals are gone, and so is the CUDA context
            pass

    @property
    def handle(self):
        return self._h

    def _s(self):
        _cabi.bind_device(self.device.index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def clear(self):
        _cabi.call("kvcm_b200_index_clear", self._h, self._s())

    def stats(self):
        slots, live = ctypes.c_int64(), ctypes.c_int64()
        _cabi.call("kvcm_b200_index_stats", self._h, ctypes.byref(slots), ctypes.byref(live), self._s())
        return slots.value, live.value

    def upsert(self, keys: torch.Tensor, values: Optional[torch.Tensor] = None, uniform_value: int = 0,
               status: Optional[torch.Tensor] = None):
        """keys int64 CUDA; values uint64-as-int64 CUDA tensor of value words, or one word for all."""
        keys = _keys(keys, self.device)
        if values is not None:
            values = values.contiguous()
        _cabi.call("kvcm_b200_index_upsert", self._h, keys.data_ptr(),
                   values.data_ptr() if values is not None else None, uniform_value, keys.numel(),
                   status.data_ptr() if status is not None else None, self._s())

    def erase(self, keys: torch.Tensor):
        keys = _keys(keys, self.device)
        _cabi.call("kvcm_b200_index_erase", self._h, keys.data_ptr(), keys.numel(), self._s())

    def lookup(self, keys: torch.Tensor) -> torch.Tensor:
        keys = _keys(keys, self.device)
        out = torch.empty(keys.numel(), dtype=torch.int64, device=self.device)
        _cabi.call("kvcm_b200_index_lookup", self._h, keys.data_ptr(), keys.numel(), out.data_ptr(), self._s())
        return out
