"""Batched matchers over a BlockIndex: many requests per call, results as lengths / window starts.

Each method is the batched twin of one MetaSearcher operator
(kv_cache_manager/manager/meta_searcher.cc:74-310); the single-request operators of the reference
are the batch-of-one case.
"""
import enum
from typing import NamedTuple, Optional

import torch

from .. import _cabi
from .block_index import BlockIndex, _keys


class QueryType(enum.IntEnum):
    # kv_cache_manager/client/include/common.h:65-70
    QT_UNSPECIFIED = 0
    QT_BATCH_GET = 1
    QT_PREFIX_MATCH = 2
    QT_REVERSE_ROLL_SW_MATCH = 3


class WriteSessions(NamedTuple):
    """What StartWriteCache of a batch returns, and what FinishWriteCache of the same batch takes back."""
    offset: torch.Tensor    # int32 per request: BlockMaskOffset, or -1 when the answer is the vector
    mask: torch.Tensor      # uint8 per key: the BlockMaskVector (1 = location map non-empty)
    n_new: torch.Tensor     # int32 per request: keys to be written
    added: torch.Tensor     # uint8 per key: 1 = this request's session holds the key
    new_off: torch.Tensor   # int64 [n_req + 1]: session keys of the requests before
    keys: torch.Tensor
    key_off: torch.Tensor
    storage_class: int


class BatchMetaSearcher:
    def __init__(self, index: BlockIndex, avail_mask: int = _cabi.AVAIL_ALL):
        self.index = index
        self.avail_mask = avail_mask

    def PrefixMatch(self, keys: torch.Tensor, key_off: torch.Tensor, mask_off: Optional[torch.Tensor] = None,
                    mask_bits: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 matched length (in keys) per request.  mask_off: int64 per request (BlockMaskOffset);
        mask_bits: uint8 per key (BlockMaskVector padded with zeros)."""
        n_req = key_off.numel() - 1
        keys, key_off = _keys(keys, self.index.device), _keys(key_off, self.index.device)
        if out is None:
            out = torch.empty(max(n_req, 1), dtype=torch.int32, device=self.index.device)
        _cabi.call("kvcm_b200_match_prefix", self.index.handle, keys.data_ptr(), key_off.data_ptr(), n_req,
                   mask_off.data_ptr() if mask_off is not None else None,
                   mask_bits.data_ptr() if mask_bits is not None else None, self.avail_mask, out.data_ptr(),
                   self.index._s())
        return out[:n_req]

    def ReverseRollSlideWindowMatch(self, keys: torch.Tensor, key_off: torch.Tensor, sw_size: int,
                                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 per request: start of the matched window, -1 no window, -2 fewer keys than sw_size.
        Raises KvcmError(KVCM_EC_BADARGS) for sw_size <= 0."""
        n_req = key_off.numel() - 1
        keys, key_off = _keys(keys, self.index.device), _keys(key_off, self.index.device)
        if out is None:
            out = torch.empty(max(n_req, 1), dtype=torch.int32, device=self.index.device)
        _cabi.call("kvcm_b200_match_sw", self.index.handle, keys.data_ptr(), key_off.data_ptr(), n_req, sw_size,
                   self.avail_mask, out.data_ptr(), self.index._s())
        return out[:n_req]

    def BatchGet(self, keys: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """uint8 flags per key (FLAG_SERVABLE | FLAG_EXISTS | FLAG_NONEMPTY | FLAG_WRITABLE)."""
        keys = _keys(keys, self.index.device)
        if out is None:
            out = torch.empty(max(keys.numel(), 1), dtype=torch.uint8, device=self.index.device)
        _cabi.call("kvcm_b200_batch_get", self.index.handle, keys.data_ptr(), keys.numel(), self.avail_mask,
                   out.data_ptr(), self.index._s())
        return out[:keys.numel()]

    # When one batch asks both questions - how long is the cached prefix, where is the last cached window - one
    # look-up per key (BatchGet) can serve both: the two matchers below read the flag bytes instead of probing the
    # index again.  Same results as PrefixMatch / ReverseRollSlideWindowMatch on the keys.
    def PrefixMatchFromFlags(self, flags: torch.Tensor, key_off: torch.Tensor, mask_off: Optional[torch.Tensor] = None,
                             mask_bits: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        n_req = key_off.numel() - 1
        key_off = _keys(key_off, self.index.device)
        if out is None:
            out = torch.empty(max(n_req, 1), dtype=torch.int32, device=self.index.device)
        _cabi.call("kvcm_b200_match_prefix_from_flags", flags.data_ptr(), key_off.data_ptr(), n_req,
                   mask_off.data_ptr() if mask_off is not None else None,
                   mask_bits.data_ptr() if mask_bits is not None else None, out.data_ptr(), self.index._s())
        return out[:n_req]

    def ReverseRollSlideWindowMatchFromFlags(self, flags: torch.Tensor, key_off: torch.Tensor, sw_size: int,
                                             out: Optional[torch.Tensor] = None) -> torch.Tensor:
        n_req = key_off.numel() - 1
        key_off = _keys(key_off, self.index.device)
        if out is None:
            out = torch.empty(max(n_req, 1), dtype=torch.int32, device=self.index.device)
        _cabi.call("kvcm_b200_match_sw_from_flags", flags.data_ptr(), key_off.data_ptr(), n_req, sw_size,
                   out.data_ptr(), self.index._s())
        return out[:n_req]

    def FilterWriteCache(self, keys: torch.Tensor, key_off: torch.Tensor):
        """Batched CacheManager::FilterWriteCache.  Returns (offset, mask, n_new): int32 offset per request (index
        of the first key still to be written when the existing keys form a prefix, else -1), uint8 per-key mask
        (1 = location map non-empty; the BlockMaskVector for requests with offset -1), int32 keys to write."""
        n_req = key_off.numel() - 1
        keys, key_off = _keys(keys, self.index.device), _keys(key_off, self.index.device)
        dev = self.index.device
        offset = torch.empty(max(n_req, 1), dtype=torch.int32, device=dev)
        n_new = torch.empty(max(n_req, 1), dtype=torch.int32, device=dev)
        mask = torch.empty(max(keys.numel(), 1), dtype=torch.uint8, device=dev)
        _cabi.call("kvcm_b200_filter_write", self.index.handle, keys.data_ptr(), key_off.data_ptr(), n_req,
                   self.avail_mask, offset.data_ptr(), mask.data_ptr(), n_new.data_ptr(), self.index._s())
        return offset[:n_req], mask[:keys.numel()], n_new[:n_req]

    def StartWriteCache(self, keys: torch.Tensor, key_off: torch.Tensor, storage_class: int,
                        table_full: Optional[torch.Tensor] = None) -> WriteSessions:
        """CacheManager::StartWriteCache for a batch of requests (kv_cache_manager/manager/cache_manager.cc:334-430):
        FilterWriteCache and BatchAddLocation in one call, with the answers the reference gives when it serves the
        requests one after the other in batch order.  The keys a request still has to write get a location of
        `storage_class` in CLS_WRITING and form its write session; a key several requests name is written by the
        first of them."""
        n_req = key_off.numel() - 1
        dev = self.index.device
        keys, key_off = _keys(keys, dev), _keys(key_off, dev)
        need = int(_cabi.lib().kvcm_b200_start_write_workspace_bytes(keys.numel(), n_req))
        if need < 0:
            raise ValueError("too many keys for one StartWriteCache batch")
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        offset = torch.empty(max(n_req, 1), dtype=torch.int32, device=dev)
        n_new = torch.empty(max(n_req, 1), dtype=torch.int32, device=dev)
        mask = torch.empty(max(keys.numel(), 1), dtype=torch.uint8, device=dev)
        added = torch.zeros(max(keys.numel(), 1), dtype=torch.uint8, device=dev)
        new_off = torch.zeros(n_req + 1, dtype=torch.int64, device=dev)
        _cabi.call("kvcm_b200_start_write", self.index.handle, keys.data_ptr(), key_off.data_ptr(), n_req, keys.numel(),
                   self.avail_mask, int(storage_class), ws.data_ptr(), need, offset.data_ptr(), mask.data_ptr(),
                   n_new.data_ptr(), added.data_ptr(), new_off.data_ptr(),
                   table_full.data_ptr() if table_full is not None else None, self.index._s())
        ws.record_stream(torch.cuda.current_stream(dev))
        return WriteSessions(offset[:n_req], mask[:keys.numel()], n_new[:n_req], added[:keys.numel()], new_off, keys,
                             key_off, int(storage_class))

    def FinishWriteCache(self, sessions: WriteSessions, success_off: Optional[torch.Tensor] = None,
                         success_bits: Optional[torch.Tensor] = None) -> torch.Tensor:
        """CacheManager::FinishWriteCache (cache_manager.cc:432-501) for the sessions of one StartWriteCache batch:
        success_off (int64 per request, a BlockMaskOffset over the session's keys) or success_bits (uint8 per
        session key of the batch, request after request).  Session keys inside the mask turn CLS_SERVING, the
        others lose their location.  Returns the int32 result code per request."""
        n_req = sessions.key_off.numel() - 1
        dev = self.index.device
        if success_off is None and success_bits is None:
            raise ValueError("a success mask is needed: offsets per request or bits per session key")
        if success_off is not None:
            success_off = _keys(success_off, dev)
        if success_bits is not None:
            success_bits = success_bits.to(torch.uint8).contiguous()
        out = torch.zeros(max(n_req, 1), dtype=torch.int32, device=dev)
        # (a batch without a key: the flags' tensor is empty and has no address to give)
        added = sessions.added if sessions.added.numel() > 0 else torch.zeros(1, dtype=torch.uint8, device=dev)
        _cabi.call("kvcm_b200_finish_write", self.index.handle, sessions.keys.data_ptr(), sessions.key_off.data_ptr(),
                   n_req, added.data_ptr(), sessions.new_off.data_ptr(),
                   success_off.data_ptr() if success_off is not None else None,
                   success_bits.data_ptr() if success_bits is not None else None, sessions.storage_class,
                   out.data_ptr(), self.index._s())
        return out[:n_req]
