"""Single-block gather / scatter operators and the staging-buffer allocator.

Same names and arguments as kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:
scatter_kv_caches (:110-140), gather_kv_caches (:143-172), CopyBufferAllocator (:175-252).
"""
import collections
import threading
from typing import List, Sequence, Union

import numpy as np
import torch

from .. import _cabi
from .batch_gather_scatter_helper import _index_tensor, _stream


def _legacy(entry: str, kv_caches_ptrs: torch.Tensor, total_token_in_kvcache: int, tensor: torch.Tensor,
            token_indices: Union[Sequence[int], torch.Tensor]) -> None:
    if kv_caches_ptrs.shape[0] != tensor.shape[0]:
        raise ValueError("%d layer pointers but the staging tensor holds %d layers"
                         % (kv_caches_ptrs.shape[0], tensor.shape[0]))
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

    Public surface of the reference's allocator (kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:175-252):
    `alloc_buffer_idx_blocking`, `get_buffer_by_idx`, `free_buffer`, `_raw_buffer`, `shape`, `max_count`.  Slot
    numbers are arbitrary, non-contiguous indices into `_raw_buffer`, which is what the batched operators take as
    `dst_block_indices`.

    Bookkeeping: the free slots are a stack in a preallocated int32 array (`_stack[:_n_free]`), and one flag per
    slot says whether it is out on loan, so that a slot returned twice, or never handed out, is refused instead of
    ending up in the stack twice.  Requests are served in arrival order: a large request is not starved by a
    stream of small ones that would each fit."""

    def __init__(self, device, dtype, shape: List[int], max_count: int):
        if int(max_count) < 1:
            raise ValueError("a staging pool needs at least one block, got max_count=%r" % (max_count,))
        self.max_count = int(max_count)
        self.device = torch.device(device)
        self.dtype = dtype
        self._raw_buffer = torch.zeros([self.max_count] + list(shape), dtype=dtype, device=self.device,
                                       pin_memory=self.device.type == "cpu" and torch.cuda.is_available())
        self._views = tuple(self._raw_buffer.unbind(0))
        self.shape = self._views[0].shape
        self._stack = np.arange(self.max_count, dtype=np.int32)
        self._n_free = self.max_count
        self._on_loan = np.zeros(self.max_count, dtype=bool)
        self._lock = threading.Lock()
        self._waiters = collections.deque()  # one Event per blocked request, oldest first

    def alloc_buffer_idx_blocking(self, count: int) -> List[int]:
        """Takes `count` slots, waiting until that many are free.  Returns their indices."""
        count = int(count)
        if not 1 <= count <= self.max_count:
            raise ValueError("cannot hand out %d blocks from a pool of %d" % (count, self.max_count))
        with self._lock:
            if not self._waiters and self._n_free >= count:
                return self._pop(count)
            turn = threading.Event()
            self._waiters.append((turn, count))
        while True:
            # Only the request at the head of the queue is ever signalled, and it stays queued until it has its
            # slots; later arrivals line up behind it, so between the signal and the wake-up the free count can
            # only grow.
            turn.wait()
            with self._lock:
                if self._n_free >= count:
                    self._waiters.popleft()
                    got = self._pop(count)
                    self._signal_head()
                    return got
                turn.clear()

    def _pop(self, count: int) -> List[int]:
        top = self._n_free
        taken = self._stack[top - count:top]
        self._on_loan[taken] = True
        self._n_free = top - count
        return taken.tolist()

    def _signal_head(self) -> None:
        """With the lock held: wakes the oldest waiting request once it fits."""
        if self._waiters and self._n_free >= self._waiters[0][1]:
            self._waiters[0][0].set()

    def get_buffer_by_idx(self, indices: List[int]):
        return [self._views[i] for i in indices]

    def free_buffer(self, buffers: List[int]):
        """Returns slots to the pool.  Refuses, without changing anything, a list that names a slot outside the
        pool, a slot that is not on loan, or the same slot twice."""
        if len(buffers) == 0:
            return
        back = np.asarray(buffers, dtype=np.int64).reshape(-1)
        with self._lock:
            bad = back[(back < 0) | (back >= self.max_count)]
            if bad.size:
                raise ValueError("staging block %d is outside this pool of %d" % (int(bad[0]), self.max_count))
            if np.unique(back).size != back.size or not self._on_loan[back].all():
                raise RuntimeError("free_buffer got %d blocks of which some are not on loan (%d are)"
                                   % (back.size, self.max_count - self._n_free))
            self._on_loan[back] = False
            self._stack[self._n_free:self._n_free + back.size] = back
            self._n_free += back.size
            self._signal_head()
