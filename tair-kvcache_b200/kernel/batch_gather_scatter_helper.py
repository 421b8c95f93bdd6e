"""Batched paged-KV gather / scatter operators.

Same names, argument order and meaning as
kv_cache_manager/py_connector/kernel/batch_gather_scatter_helper.py:101-136 (batch_gather_kv_caches)
and :208-248 (batch_scatter_kv_caches); the Triton kernels behind them are replaced by the
sm_100a kernels of libkvcm_b200.so, reached through its C ABI with raw addresses and the
current CUDA stream.  torch is used only to own memory and streams.

Like the reference, the calls return as soon as the kernel is enqueued on the current stream;
callers record an event and synchronise (kv_cache_manager/py_connector/vllm/data_transfer.py:138-150).
"""
import os
from typing import Optional, Sequence, Union

import numpy as np
import torch

from .. import _cabi

IndexArg = Union[Sequence[int], torch.Tensor]
_NO_BOUND = 1 << 31  # int32 indices cannot exceed this; used when the caller gives no pool size
# Device bounce buffer of the host-staging path: blocks go through it in groups of at most this many bytes.
_BOUNCE_BYTES = 256 << 20
# KVCM_B200_HOST_STAGING=zerocopy makes the kernels read / write pinned host memory directly (no bounce
# buffer, lowest latency for small transfers); the default sends the PCIe leg through the copy engines.
_ZERO_COPY = os.environ.get("KVCM_B200_HOST_STAGING", "").lower() == "zerocopy"


def _index_tensor(values: IndexArg, device: torch.device) -> torch.Tensor:
    """int32 device tensor from a Python list (the reference's argument type) or a tensor.

    A device int32 tensor is passed through untouched, so callers that keep their block tables on
    the GPU pay no host work and no copy per call (the reference rebuilds two tensors from
    Python lists on every call, batch_gather_scatter_helper.py:118-121)."""
    if isinstance(values, torch.Tensor):
        t = values
        if t.dtype != torch.int32:
            t = t.to(torch.int32)
        if t.device != device:
            t = t.to(device, non_blocking=True)
        return t.contiguous()
    return torch.tensor(values, dtype=torch.int32, device="cpu").to(device, non_blocking=True)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _coalesce_token_runs(row_indices, slot_indices, rows_per_block: int, pool_rows: Optional[int], n_slots: int):
    """Token indices given as a host list (the reference's argument type) almost always come from a block table:
    runs of page_size consecutive tokens that start at a multiple of page_size
    (kv_cache_manager/py_connector/vllm/v1_connector.py:308-320).  Such a list is the page form with longer rows, and
    long rows move faster (one bulk copy per page instead of one vector loop per token).  Returns
    (row array, rows per block, run length) with run length g > 1 when every block splits into aligned runs of g
    tokens, else None.  Only lists whose indices and staging slots are all in range are rewritten, so that the
    counts reported in the status words cannot change."""
    if isinstance(row_indices, torch.Tensor) or rows_per_block < 2:
        return None
    arr = np.asarray(row_indices, dtype=np.int64)
    if arr.size == 0 or arr.size % rows_per_block != 0 or arr.min() < 0:
        return None
    if pool_rows is not None and arr.max() >= pool_rows:
        return None
    if slot_indices is not None and not isinstance(slot_indices, torch.Tensor):
        sl = np.asarray(slot_indices, dtype=np.int64)
        if sl.size and (sl.min() < 0 or sl.max() >= n_slots):
            return None
    elif slot_indices is not None:
        return None  # device-resident slots cannot be range-checked here without a sync
    # the first place where the list stops counting up bounds the run length; try its divisors that also divide
    # the block length, longest first
    breaks = np.flatnonzero(np.diff(arr) != 1)
    longest = int(breaks[0]) + 1 if breaks.size else arr.size
    for g in range(min(longest, rows_per_block), 1, -1):
        if rows_per_block % g or (pool_rows is not None and pool_rows % g):
            continue
        runs = arr.reshape(-1, g)
        if not (runs[:, 0] % g).any() and (np.diff(runs, axis=1) == 1).all():
            return np.ascontiguousarray(runs[:, 0] // g, dtype=np.int32), rows_per_block // g, g
    return None


def _move(entry: str, kv_caches_ptrs_tensor: torch.Tensor, staging: torch.Tensor, row_indices: IndexArg,
          slot_indices: Optional[IndexArg], rows_per_block: int, row_bytes: int, pool_rows: Optional[int],
          status: Optional[torch.Tensor], sm_count: Optional[int] = None) -> None:
    if kv_caches_ptrs_tensor.dtype != torch.int64 or not kv_caches_ptrs_tensor.is_cuda:
        raise ValueError("kv_caches_ptrs_tensor must be an int64 CUDA tensor of pool base addresses")
    if not staging.is_contiguous():
        raise ValueError("the staging tensor must be contiguous")
    if not (staging.is_cuda or staging.is_pinned()):
        raise ValueError("the staging tensor must live on the GPU or in pinned host memory")
    device = kv_caches_ptrs_tensor.device
    if entry.endswith("_tokens") and rows_per_block > 0 and row_bytes > 0:
        n_pools_ = kv_caches_ptrs_tensor.numel()
        slot_bytes_ = n_pools_ * rows_per_block * row_bytes
        merged = _coalesce_token_runs(row_indices, slot_indices, rows_per_block, pool_rows,
                                      staging.numel() * staging.element_size() // slot_bytes_ if slot_bytes_ else 0)
        if merged is not None:
            row_indices, rows_per_block, g = merged
            row_indices = torch.from_numpy(row_indices)
            row_bytes *= g
            pool_rows = None if pool_rows is None else pool_rows // g
            entry = entry.replace("_tokens", "_pages")
    rows = _index_tensor(row_indices, device)
    if rows_per_block <= 0 or rows.numel() % rows_per_block != 0:
        raise ValueError("index count %d is not a multiple of %d" % (rows.numel(), rows_per_block))
    n_blocks = rows.numel() // rows_per_block
    if not staging.is_cuda and not _ZERO_COPY and sm_count is None:
        _move_through_bounce(entry, kv_caches_ptrs_tensor, staging, rows, slot_indices, n_blocks, rows_per_block,
                             row_bytes, pool_rows, status)
        return
    slots = None
    if slot_indices is not None:
        slots = _index_tensor(slot_indices, device)
        if slots.numel() != n_blocks:
            raise ValueError("%d staging indices for %d blocks" % (slots.numel(), n_blocks))
    n_pools = kv_caches_ptrs_tensor.numel()
    slot_bytes = n_pools * rows_per_block * row_bytes
    n_slots = staging.numel() * staging.element_size() // slot_bytes if slot_bytes else 0
    _cabi.bind_device(device.index)
    with torch.cuda.device(device):
        _cabi.call_move(entry, kv_caches_ptrs_tensor.data_ptr(), n_pools, staging.data_ptr(), n_slots,
                        rows.data_ptr(), slots.data_ptr() if slots is not None else None, n_blocks, rows_per_block,
                        row_bytes, _NO_BOUND if pool_rows is None else pool_rows,
                        status.data_ptr() if status is not None else None, int(sm_count or 0), _stream())
    # keep the index tensors alive until the stream has consumed them
    rows.record_stream(torch.cuda.current_stream())
    if slots is not None:
        slots.record_stream(torch.cuda.current_stream())


def _move_through_bounce(entry, kv_caches_ptrs_tensor, staging, rows, slot_indices, n_blocks, rows_per_block,
                         row_bytes, pool_rows, status) -> None:
    """Pinned-host staging: gather into a device bounce buffer and let the copy engines cross PCIe (or the
    reverse for a load).  The staging slots are needed on the host, where the reference passes them anyway."""
    device = kv_caches_ptrs_tensor.device
    n_pools = kv_caches_ptrs_tensor.numel()
    block_bytes = n_pools * rows_per_block * row_bytes
    n_slots = staging.numel() * staging.element_size() // block_bytes if block_bytes else 0
    slots = None
    if slot_indices is not None:
        if isinstance(slot_indices, torch.Tensor):
            slots = slot_indices.detach().to("cpu", torch.int32).contiguous().numpy()
        else:
            slots = np.ascontiguousarray(slot_indices, dtype=np.int32)
        if len(slots) != n_blocks:
            raise ValueError("%d staging indices for %d blocks" % (len(slots), n_blocks))
    if n_blocks == 0:
        return
    group = max(1, min(n_blocks, _BOUNCE_BYTES // block_bytes))
    bounce = torch.empty(group * block_bytes, dtype=torch.uint8, device=device)
    name = "kvcm_b200_save_rows_to_host" if "gather" in entry else "kvcm_b200_load_rows_from_host"
    _cabi.bind_device(device.index)
    with torch.cuda.device(device):
        _cabi.call_move(name, kv_caches_ptrs_tensor.data_ptr(), n_pools, staging.data_ptr(), n_slots,
                        rows.data_ptr(), slots.ctypes.data if slots is not None else None, n_blocks, rows_per_block,
                        row_bytes, _NO_BOUND if pool_rows is None else pool_rows, bounce.data_ptr(), bounce.numel(),
                        status.data_ptr() if status is not None else None, _stream())
    rows.record_stream(torch.cuda.current_stream())
    bounce.record_stream(torch.cuda.current_stream())


def batch_gather_kv_caches(
        kv_caches_ptrs_tensor: torch.Tensor,
        dst_tensor: torch.Tensor,
        block_token_indices: IndexArg,
        dst_block_indices: IndexArg,
        num_tokens_per_block: int,
        dim_size_per_token_per_layer: int,
        sm_count: Optional[int] = None,
        total_token_in_kvcache: Optional[int] = None,
        status: Optional[torch.Tensor] = None,
) -> None:
    """dst[dst_block_indices[b], p, t, :] = pool_p[block_token_indices[b*T + t], :].

    `dst_tensor` on the GPU: one kernel at HBM speed.  `dst_tensor` in pinned host memory (the connector's
    production setting): blocks are gathered into a device bounce buffer and leave through the copy engines, so
    a save and a load on two streams use both PCIe directions at full rate.  Passing `sm_count` (the reference's
    argument, default 3 there) instead makes the kernel write host memory directly from that many SMs.  `total_token_in_kvcache` (optional) bounds the token indices; out-of-range rows are
    skipped and counted in `status` (four zeroed 32-bit words on the GPU)."""
    _move("kvcm_b200_gather_tokens", kv_caches_ptrs_tensor, dst_tensor, block_token_indices, dst_block_indices,
          num_tokens_per_block, dim_size_per_token_per_layer * dst_tensor.element_size(), total_token_in_kvcache,
          status, sm_count)


def batch_scatter_kv_caches(
        kv_caches_ptrs_tensor: torch.Tensor,
        src_tensor: torch.Tensor,
        block_token_indices: IndexArg,
        src_block_indices: IndexArg,
        num_tokens_per_block: int,
        dim_size_per_token_per_layer: int,
        sm_count: Optional[int] = None,
        total_token_in_kvcache: Optional[int] = None,
        status: Optional[torch.Tensor] = None,
) -> None:
    """pool_p[block_token_indices[b*T + t], :] = src[src_block_indices[b], p, t, :]."""
    _move("kvcm_b200_scatter_tokens", kv_caches_ptrs_tensor, src_tensor, block_token_indices, src_block_indices,
          num_tokens_per_block, dim_size_per_token_per_layer * src_tensor.element_size(), total_token_in_kvcache,
          status, sm_count)


def batch_gather_kv_pages(kv_caches_ptrs_tensor: torch.Tensor, dst_tensor: torch.Tensor, block_page_table: IndexArg,
                          dst_block_indices: Optional[IndexArg], pages_per_block: int, page_bytes: int,
                          pool_pages: Optional[int] = None, status: Optional[torch.Tensor] = None,
                          sm_count: Optional[int] = None) -> None:
    """Page-table form: the engine's block table addresses whole pages, so the per-token index
    list of generate_blocks_idx (kv_cache_manager/py_connector/vllm/v1_connector.py:308-320) is
    never built.  Byte-identical to batch_gather_kv_caches on the expanded token indices."""
    _move("kvcm_b200_gather_pages", kv_caches_ptrs_tensor, dst_tensor, block_page_table, dst_block_indices,
          pages_per_block, page_bytes, pool_pages, status, sm_count)


def batch_scatter_kv_pages(kv_caches_ptrs_tensor: torch.Tensor, src_tensor: torch.Tensor, block_page_table: IndexArg,
                           src_block_indices: Optional[IndexArg], pages_per_block: int, page_bytes: int,
                           pool_pages: Optional[int] = None, status: Optional[torch.Tensor] = None,
                           sm_count: Optional[int] = None) -> None:
    _move("kvcm_b200_scatter_pages", kv_caches_ptrs_tensor, src_tensor, block_page_table, src_block_indices,
          pages_per_block, page_bytes, pool_pages, status, sm_count)
