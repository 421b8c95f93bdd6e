"""Single-block gather / scatter operators and the staging-buffer allocator.

Same names and arguments as kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:
scatter_kv_caches (:110-140), gather_kv_caches (:143-172), CopyBufferAllocator (:175-252).
"""
import threading
from typing import List, Sequence, Union

import torch

from .. import _cabi
from .batch_gather_scatter_helper import _index_tensor, _stream


def _legacy(entry: str, kv_caches_ptrs: torch.Tensor, total_token_in_kvcache: int, tensor: torch.Tensor,
            token_indices: Union[Sequence[int], torch.Tensor]) -> None:
    assert kv_caches_ptrs.shape[0] == tensor.shape[0], "Number of layers mismatch"
    if not tensor.is_contiguous():
        raise ValueError("the staging tensor must be contiguous")
    idx = _index_tensor(token_indices, kv_caches_ptrs.device)
    hidden_bytes = tensor.shape[-1] * tensor.element_size()
    _cabi.bind_device(kv_caches_ptrs.device.index)
    with torch.cuda.device(kv_caches_ptrs.device):
        _cabi.call_move(entry, kv_caches_ptrs.data_ptr(), kv_caches_ptrs.shape[0], total_token_in_kvcache,
                   tensor.data_ptr(), idx.data_ptr(), idx.numel(), hidden_bytes, _stream())
    idx.record_stream(torch.cuda.current_stream())


def scatter_kv_caches(kv_caches_ptrs: torch.Tensor, total_token_in_kvcache: int, src_tensor: torch.Tensor,
                      token_indices: Union[List[int], torch.Tensor]) -> None:
    """cache_l[kv, token_indices[t], :] = src[l, kv, t, :]; cache_l is [2, total_token_in_kvcache, hidden]."""
    _legacy("kvcm_b200_scatter_legacy", kv_caches_ptrs, total_token_in_kvcache, src_tensor, token_indices)


def gather_kv_caches(kv_caches_ptrs: torch.Tensor, total_token_in_kvcache: int, dst_tensor: torch.Tensor,
                     token_indices: Union[List[int], torch.Tensor]) -> None:
    """dst[l, kv, t, :] = cache_l[kv, token_indices[t], :]."""
    _legacy("kvcm_b200_gather_legacy", kv_caches_ptrs, total_token_in_kvcache, dst_tensor, token_indices)


class CopyBufferAllocator:
    """Fixed pool of `max_count` staging blocks carved from one tensor (pinned when on the CPU).

    Indices are handed out under a condition variable; `alloc_buffer_idx_blocking` waits until
    enough blocks are free.  Staging slots are therefore arbitrary, non-contiguous indices into
    `_raw_buffer`, which is what the batched operators take as `dst_block_indices`."""

    def __init__(self, device, dtype, shape: List[int], max_count: int):
        if max_count <= 0:
            raise ValueError("max_count must be positive")
        self.max_count = max_count
        self.device = torch.device(device)
        self.dtype = dtype
        self._cond = threading.Condition()
        self._raw_buffer = torch.zeros([max_count] + list(shape), dtype=dtype, device=self.device,
                                       pin_memory=self.device.type == "cpu")
        self._free_idx_list = list(range(max_count))
        self._free_buffer_list = [self._raw_buffer[i] for i in range(max_count)]
        self.shape = self._free_buffer_list[0].shape
        self._inuse_count = 0

    def alloc_buffer_idx_blocking(self, count: int) -> List[int]:
        if count <= 0:
            raise ValueError("count must be positive")
        if count > self.max_count:
            raise ValueError(f"count ({count}) exceeds max_count ({self.max_count})")
        with self._cond:
            while self._inuse_count + count > self.max_count:
                self._cond.wait()
            self._inuse_count += count
            taken = self._free_idx_list[-count:]
            del self._free_idx_list[-count:]
            return taken

    def get_buffer_by_idx(self, indices: List[int]):
        return [self._free_buffer_list[i] for i in indices]

    def free_buffer(self, buffers: List[int]):
        if not buffers:
            return
        with self._cond:
            for idx in buffers:
                if idx >= self.max_count or idx < 0:
                    raise ValueError(f"Buffer idx {idx} wrong")
            if self._inuse_count < len(buffers):
                raise RuntimeError(f"Trying to free {len(buffers)} buffers, but only {self._inuse_count} are in use")
            self._inuse_count -= len(buffers)
            self._free_idx_list.extend(buffers)
            self._cond.notify_all()
