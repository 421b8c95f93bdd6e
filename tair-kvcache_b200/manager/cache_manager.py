"""The data-path operators of CacheManager over device-resident indexes, one request per call as the reference
serves them: GetCacheLocation, StartWriteCache, FinishWriteCache
(kv_cache_manager/manager/cache_manager.cc:287-501, FilterWriteCache :589-635, GetCacheLocationByQueryType :969-1020).

Same names, same argument meaning, same error codes (the reference's ErrorCode numbers behind KVCM_EC_BASE); what
comes back is what the matchers decide - how many locations, which of them carry a URI, the block mask of a write -
not CacheLocation objects: choosing which of a key's locations to hand out (a weighted random pick) and building its
URIs stay with the caller's CPU-side table, as in the reference-side binding.  Every call runs the library's kernels
on the instance's index: hash (when tokens are given), match / batch-get, filter-write, add-location,
status transitions.  Batches of requests go through BatchMetaSearcher directly.
"""
import secrets
import time
from typing import Dict, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .. import _cabi
from .block_index import CLS_SERVING, CLS_WRITING, BlockIndex, avail_mask_from_weights, status_task
from .hash_util import GenKeyVectorBatch, key_offsets
from .meta_searcher import BatchMetaSearcher, QueryType

BlockMask = Union[int, Sequence[bool]]  # kv_cache_manager/manager/cache_location.h:52-57: an offset or a vector

EC_OK = _cabi.KVCM_OK
EC_ERROR = _cabi.KVCM_EC_ERROR
EC_BADARGS = _cabi.KVCM_EC_BADARGS
EC_INSTANCE_NOT_EXIST = _cabi.KVCM_EC_BASE + 11


def IsIndexInMaskRange(mask: BlockMask, index: int) -> bool:
    """kv_cache_manager/manager/cache_location.cc:9-21"""
    if isinstance(mask, (int, np.integer)):
        return index < int(mask)
    return bool(mask[index]) if index < len(mask) else False


def IsBlockMaskValid(mask: BlockMask, size: int) -> bool:
    """kv_cache_manager/manager/cache_location.cc:22-31"""
    if isinstance(mask, (int, np.integer)):
        return 0 <= int(mask) <= size
    return len(mask) == size


class _Instance:
    def __init__(self, block_size, index, searcher, storage_class):
        self.block_size, self.index, self.searcher, self.storage_class = block_size, index, searcher, storage_class


class GpuCacheManager:
    def __init__(self, device: Optional[torch.device] = None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._instances: Dict[str, _Instance] = {}
        # WriteLocationManager (kv_cache_manager/manager/write_location_manager.h): write_session_id -> the keys
        # that got a location from StartWriteCache, and the storage class it lies in
        self._sessions: Dict[str, Tuple[str, torch.Tensor, float]] = {}

    def RegisterInstance(self, instance_id: str, block_size: int, max_keys: int, storage_class: int = 4,
                         weights: Optional[Sequence[int]] = None) -> int:
        """An index for the instance.  storage_class is the DataStorageType new locations are written to (what
        GenWriteLocation picks, cache_manager.cc:786-893); weights the SelectLocationPolicy's per-type weights."""
        if instance_id in self._instances:
            return EC_OK if self._instances[instance_id].block_size == block_size else _cabi.KVCM_EC_BASE + 12
        index = BlockIndex(max_keys, self.device)
        avail = avail_mask_from_weights(weights) if weights is not None else _cabi.AVAIL_ALL
        self._instances[instance_id] = _Instance(int(block_size), index, BatchMetaSearcher(index, avail),
                                                 int(storage_class))
        return EC_OK

    def index_of(self, instance_id: str) -> BlockIndex:
        return self._instances[instance_id].index

    # ---- keys of one request on the device: given, or hashed from the tokens (GenKeyVector, :311-314,367-372) ----
    def _request_keys(self, inst: _Instance, keys, tokens) -> torch.Tensor:
        if keys is not None and len(keys) > 0:
            return torch.as_tensor(np.asarray(keys, dtype=np.int64), device=self.device)
        toks = np.asarray(tokens, dtype=np.int64)
        off = np.array([0, len(toks)], dtype=np.int64)
        ko = key_offsets(off, inst.block_size)
        return GenKeyVectorBatch(torch.from_numpy(toks).to(self.device), torch.from_numpy(off).to(self.device),
                                 inst.block_size, torch.from_numpy(ko).to(self.device), int(ko[-1]))

    def _check(self, instance_id, keys, tokens):
        """CheckInputAndGetMetaSearcher (cache_manager.cc:906-924)"""
        inst = self._instances.get(instance_id)
        if inst is None:
            return EC_INSTANCE_NOT_EXIST, None
        if (keys is None or len(keys) == 0) and (tokens is None or len(tokens) == 0):
            return EC_BADARGS, None
        return EC_OK, inst

    def GetCacheLocation(self, instance_id: str, query_type: QueryType, keys=None, tokens=None,
                         block_mask: BlockMask = 0, sw_size: int = 0) -> Tuple[int, np.ndarray]:
        """(error code, one bool per returned location: True where the location carries a URI).
        QT_PREFIX_MATCH returns the matched leading locations (all True) - keys inside block_mask are skipped, not
        returned; QT_BATCH_GET one location per key; QT_REVERSE_ROLL_SW_MATCH one per key, True on the window."""
        none = np.zeros(0, dtype=bool)
        ec, inst = self._check(instance_id, keys, tokens)
        if ec != EC_OK:
            return ec, none
        if query_type == QueryType.QT_UNSPECIFIED:
            return EC_ERROR, none
        k = self._request_keys(inst, keys, tokens)
        n = k.numel()
        off = torch.tensor([0, n], dtype=torch.int64, device=self.device)
        if query_type == QueryType.QT_PREFIX_MATCH:
            mask_off = mask_bits = None
            if isinstance(block_mask, (int, np.integer)):
                mask_off = torch.tensor([int(block_mask)], dtype=torch.int64, device=self.device)
            else:
                bits = np.zeros(n, dtype=np.uint8)
                m = np.asarray(block_mask, dtype=np.uint8)[:n]
                bits[:len(m)] = m
                mask_bits = torch.from_numpy(bits).to(self.device)
            matched = int(inst.searcher.PrefixMatch(k, off, mask_off, mask_bits).cpu()[0])
            return EC_OK, np.ones(matched, dtype=bool)
        if query_type == QueryType.QT_BATCH_GET:
            flags = inst.searcher.BatchGet(k).cpu().numpy()[:n]
            return EC_OK, (flags & _cabi.FLAG_SERVABLE) != 0
        if query_type == QueryType.QT_REVERSE_ROLL_SW_MATCH:
            # (a window of no keys never ends the reference's loop, meta_searcher.cc:196-265: refused like the rest)
            if n < sw_size or sw_size <= 0:
                return EC_BADARGS, none
            out = np.zeros(n, dtype=bool)
            base = int(inst.searcher.ReverseRollSlideWindowMatch(k, off, int(sw_size)).cpu()[0])
            if base >= 0:
                out[base:base + sw_size] = True
            return EC_OK, out
        return EC_ERROR, none

    def StartWriteCache(self, instance_id: str, keys=None, tokens=None, write_timeout_seconds: float = 1800.0
                        ) -> Tuple[int, Optional[str], BlockMask, int]:
        """(error code, write_session_id, block_mask, number of new locations).  block_mask is what FilterWriteCache
        decides (cache_manager.cc:589-635): the offset of the first key still to be written when the keys that exist
        form a prefix, else one bool per key (True = the key's location map is not empty); the keys outside it get a
        location in CLS_WRITING (MetaSearcher::BatchAddLocation) and make up the session."""
        ec, inst = self._check(instance_id, keys, tokens)
        if ec != EC_OK:
            return ec, None, 0, 0
        k = self._request_keys(inst, keys, tokens)
        n = k.numel()
        off = torch.tensor([0, n], dtype=torch.int64, device=self.device)
        offset, mask, _ = inst.searcher.FilterWriteCache(k, off)
        first = int(offset.cpu()[0])
        if first >= 0:
            block_mask: BlockMask = first
            new_keys = k[first:]
        else:
            held = mask.cpu().numpy()[:n].astype(bool)
            block_mask = held.tolist()
            new_keys = k[torch.from_numpy(np.flatnonzero(~held)).to(self.device)]
        if new_keys.numel() > 0:
            codes = inst.index.add_location(new_keys, inst.storage_class, CLS_WRITING).cpu().numpy()
            if (codes != EC_OK).any():  # a full table, as the reference's "indexer reach max key count"
                return int(codes[codes != EC_OK][0]), None, block_mask, 0
        session = secrets.token_hex(16)
        if new_keys.numel() == 0:
            write_timeout_seconds = 10.0  # nothing to write: the session is dropped soon (cache_manager.cc:387-390)
        self._sessions[session] = (instance_id, new_keys, time.monotonic() + float(write_timeout_seconds))
        return EC_OK, session, block_mask, int(new_keys.numel())

    def ExpireWriteSessions(self, now: Optional[float] = None) -> int:
        """What the reference's WriteLocationManager does when a session's write_timeout_seconds have passed: it
        finishes the session with nothing written (FinishWriteCache with an offset of 0, cache_manager.cc:400-409),
        so its locations are removed and a later FinishWriteCache of the session finds nothing.  Returns how many
        sessions went.  The reference runs this from a timer thread; here the caller decides when."""
        now = time.monotonic() if now is None else now
        late = [sid for sid, (_, _, deadline) in self._sessions.items() if deadline <= now]
        for sid in late:
            self.FinishWriteCache(self._sessions[sid][0], sid, 0)
        return len(late)

    def FinishWriteCache(self, instance_id: str, write_session_id: str, success_block_mask: BlockMask) -> int:
        """The session's keys inside success_block_mask turn CLS_SERVING (BatchUpdateLocationStatus); the locations
        of the others are deleted (the reference hands them to its reclaimer, cache_manager.cc:455-492)."""
        entry = self._sessions.pop(write_session_id, None)  # GetAndDelete: a session finishes once
        if entry is None:
            return EC_ERROR
        _, new_keys, _ = entry
        n = int(new_keys.numel())
        if not IsBlockMaskValid(success_block_mask, n):
            return EC_BADARGS
        inst = self._instances.get(instance_id)
        if inst is None:
            return EC_INSTANCE_NOT_EXIST
        if n == 0:
            return EC_OK
        ok = np.array([IsIndexInMaskRange(success_block_mask, i) for i in range(n)], dtype=bool)
        tasks = np.where(ok, status_task(inst.storage_class, None, CLS_SERVING),
                         status_task(inst.storage_class, None, None)).astype(np.int32)
        codes = inst.index.update_status(new_keys, torch.from_numpy(tasks).to(self.device)).cpu().numpy()
        failed = codes[ok] != EC_OK
        return int(codes[ok][failed][0]) if failed.any() else EC_OK

    def RemoveCache(self, instance_id: str, keys=None, tokens=None) -> int:
        """The keys (or the keys of the tokens) leave the index with all their locations (cache_manager.cc:503-526;
        the reference hands the request to its reclaimer, which deletes in the background - here it is done when the
        call returns).  Its block_mask argument is not read by the reference either."""
        if (keys is None or len(keys) == 0) and (tokens is None or len(tokens) == 0):
            return EC_BADARGS
        inst = self._instances.get(instance_id)
        if inst is None:
            return EC_INSTANCE_NOT_EXIST
        inst.index.erase(self._request_keys(inst, keys, tokens))
        return EC_OK

    def TrimCache(self, instance_id: str, remove_all: bool = True) -> int:
        """TS_REMOVE_ALL_CACHE, the one trim strategy the reference implements (cache_manager.cc:528-565)."""
        if not remove_all:
            return _cabi.KVCM_EC_BASE + 7  # EC_UNIMPLEMENTED
        inst = self._instances.get(instance_id)
        if inst is None:
            return EC_INSTANCE_NOT_EXIST
        inst.index.clear()
        return EC_OK
