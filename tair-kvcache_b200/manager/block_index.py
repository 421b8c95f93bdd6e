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
    ExistsForWrite (kv_cache_manager/manager/select_location_policy.cc:8-38) read.  For classes 0..7 the
    word also carries the status itself (three bits per class, status + 1), which is what
    BlockIndex.update_status compares and rewrites; when a map holds several locations of one class the
    field keeps the first one's status and the key should be maintained with upsert only."""
    word = 0
    for status, cls in locations:
        c = min(max(int(cls), 0), 15)
        word |= _cabi.VAL_NONEMPTY
        if status == CLS_SERVING:
            word |= 1 << c
        if status != CLS_NOT_FOUND:
            word |= 1 << (16 + c)
        shift = _cabi.VAL_STATUS_SHIFT + 3 * c
        if c < 8 and not (word >> shift) & 7:
            word |= (int(status) + 1) << shift
    return word


def status_task(storage_class: int, expected: Optional[int], new_status: Optional[int], keep_key: bool = False) -> int:
    """One task of BlockIndex.update_status: the location of `storage_class` goes from `expected` (None = whatever
    it is) to `new_status` (None = the location is deleted; with `keep_key` the way BatchDeleteLocation deletes,
    which leaves an emptied key in the index and takes an absent key for done)."""
    e = _cabi.STATUS_ANY if expected is None else int(expected)
    n = int(new_status) if new_status is not None else (
        _cabi.STATUS_DELETE_KEEP_KEY if keep_key else _cabi.STATUS_DELETE)
    return int(storage_class) | (e << 8) | (n << 16)


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

    def usage(self):
        """(slots, live keys, slots in use = live keys + tombstones of erased keys)."""
        slots, live, used = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        _cabi.call("kvcm_b200_index_usage", self._h, ctypes.byref(slots), ctypes.byref(live), ctypes.byref(used),
                   self._s())
        return slots.value, live.value, used.value

    def rehash(self, status: Optional[torch.Tensor] = None):
        """Rebuilds the table in place without the tombstones erased keys left behind."""
        need = int(_cabi.lib().kvcm_b200_index_rehash_workspace_bytes(self._h))
        workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        _cabi.call("kvcm_b200_index_rehash", self._h, workspace.data_ptr(), need,
                   status.data_ptr() if status is not None else None, self._s())
        workspace.record_stream(torch.cuda.current_stream(self.device))

    def update_status(self, keys: torch.Tensor, tasks, shard: Optional[Tuple[int, int]] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Location-status transitions on the device (MetaSearcher::BatchUpdateLocationStatus / BatchCASLocationStatus /
        BatchCADLocationStatus / BatchDeleteLocation, kv_cache_manager/manager/meta_searcher.cc:410-820).  `tasks`: one
        status_task() word for all keys, or an int32 CUDA tensor with one word per key.  Returns the int32 result
        code per key (0, KVCM_EC_NOENT, KVCM_EC_MISMATCH, KVCM_EC_BADARGS).  shard=(count, rank) limits the call to
        the keys this shard owns."""
        keys = _keys(keys, self.device)
        if out is None:
            out = torch.zeros(keys.numel(), dtype=torch.int32, device=self.device)
        d_tasks, uniform = None, 0
        if isinstance(tasks, torch.Tensor):
            d_tasks = tasks.to(torch.int32).contiguous()
            if d_tasks.numel() != keys.numel() or d_tasks.device != self.device:
                raise ValueError("one task word per key, on the index's device")
        else:
            uniform = int(tasks)
        if shard is None:
            _cabi.call("kvcm_b200_index_update_status", self._h, keys.data_ptr(),
                       d_tasks.data_ptr() if d_tasks is not None else None, uniform, keys.numel(), out.data_ptr(),
                       self._s())
        else:
            _cabi.call("kvcm_b200_index_update_status_sharded", self._h, keys.data_ptr(),
                       d_tasks.data_ptr() if d_tasks is not None else None, uniform, keys.numel(), shard[0], shard[1],
                       out.data_ptr(), self._s())
        return out

    def add_location(self, keys: torch.Tensor, classes, status: int = CLS_WRITING, shard: Optional[Tuple[int, int]] = None,
                     out: Optional[torch.Tensor] = None, table_full: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One new location per key, merged into the key's location map on the device
        (MetaSearcher::BatchAddLocation, kv_cache_manager/manager/meta_searcher.cc:312-408): `classes` is one storage
        class for all keys or a uint8 CUDA tensor with one per key, `status` the CacheLocationStatus the location
        starts in (CLS_WRITING = 2, as the reference adds it).  An absent key is inserted, a present key keeps its
        other locations.  Returns the int32 result code per key (0, KVCM_EC_EXIST when the key already holds a
        location of that class, KVCM_EC_NOSPC when the table is full, KVCM_EC_BADARGS for a class above 7);
        table_full (uint32 CUDA tensor) counts the refused keys in its first word.  shard=(count, rank) limits the
        call to the keys this shard owns."""
        keys = _keys(keys, self.device)
        if out is None:
            out = torch.zeros(keys.numel(), dtype=torch.int32, device=self.device)
        d_classes, uniform = None, 0
        if isinstance(classes, torch.Tensor):
            d_classes = classes.to(torch.uint8).contiguous()
            if d_classes.numel() != keys.numel() or d_classes.device != self.device:
                raise ValueError("one storage class per key, on the index's device")
        else:
            uniform = int(classes)
        args = [self._h, keys.data_ptr(), d_classes.data_ptr() if d_classes is not None else None, uniform, int(status),
                keys.numel()]
        tail = [out.data_ptr(), table_full.data_ptr() if table_full is not None else None, self._s()]
        if shard is None:
            _cabi.call("kvcm_b200_index_add_location", *args, *tail)
        else:
            _cabi.call("kvcm_b200_index_add_location_sharded", *args, shard[0], shard[1], *tail)
        return out

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
