"""Batched paged-KV gather / scatter operators.

Same names, argument order and meaning as
kv_cache_manager/py_connector/kernel/batch_gather_scatter_helper.py:101-136 (batch_gather_kv_caches)
and :208-248 (batch_scatter_kv_caches); the Triton kernels behind them are replaced by the
sm_100a kernels of libkvcm_b200.so, reached through its C ABI with raw addresses and the
current CUDA stream.  torch is used only to own memory and streams.

Like the reference, the calls return as soon as the kernel is enqueued on the current stream;
callers record an event and synchronise (kv_cache_manager/py_connector/vllm/data_transfer.py:138-150).
"""
from typing import List, Optional, Sequence, Union

import torch

from .. import _cabi

IndexArg = Union[Sequence[int], torch.Tensor]
_NO_BOUND = 1 << 31  # int32 indices cannot exceed this; used when the caller gives no pool size


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


def _move(entry: str, kv_caches_ptrs_tensor: torch.Tensor, staging: torch.Tensor, row_indices: IndexArg,
          slot_indices: Optional[IndexArg], rows_per_block: int, row_bytes: int, pool_rows: Optional[int],
          status: Optional[torch.Tensor]) -> None:
    if kv_caches_ptrs_tensor.dtype != torch.int64 or not kv_caches_ptrs_tensor.is_cuda:
        raise ValueError("kv_caches_ptrs_tensor must be an int64 CUDA tensor of pool base addresses")
    if not staging.is_contiguous():
        raise ValueError("the staging tensor must be contiguous")
    if not (staging.is_cuda or staging.is_pinned()):
        raise ValueError("the staging tensor must live on the GPU or in pinned host memory")
    device = kv_caches_ptrs_tensor.device
    rows = _index_tensor(row_indices, device)
    if rows_per_block <= 0 or rows.numel() % rows_per_block != 0:
        raise ValueError("index count %d is not a multiple of %d" % (rows.numel(), rows_per_block))
    n_blocks = rows.numel() // rows_per_block
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
        _cabi.call(entry, kv_caches_ptrs_tensor.data_ptr(), n_pools, staging.data_ptr(), n_slots, rows.data_ptr(),
                   slots.data_ptr() if slots is not None else None, n_blocks, rows_per_block, row_bytes,
                   _NO_BOUND if pool_rows is None else pool_rows,
                   status.data_ptr() if status is not None else None, _stream())
    # keep the index tensors alive until the stream has consumed them
    rows.record_stream(torch.cuda.current_stream())
    if slots is not None:
        slots.record_stream(torch.cuda.current_stream())


def batch_gather_kv_caches(
        kv_caches_ptrs_tensor: torch.Tensor,
        dst_tensor: torch.Tensor,
        block_token_indices: IndexArg,
        dst_block_indices: IndexArg,
        num_tokens_per_block: int,
        dim_size_per_token_per_layer: int,
        sm_count: int = 3,
        total_token_in_kvcache: Optional[int] = None,
        status: Optional[torch.Tensor] = None,
) -> None:
    """dst[dst_block_indices[b], p, t, :] = pool_p[block_token_indices[b*T + t], :].

    `sm_count` is accepted for signature compatibility and ignored: the library sizes its
    persistent grid from the device.  `total_token_in_kvcache` (optional) bounds the token
    indices; out-of-range rows are skipped and counted in `status` (four zeroed 32-bit words on the GPU)."""
    del sm_count
    _move("kvcm_b200_gather_tokens", kv_caches_ptrs_tensor, dst_tensor, block_token_indices, dst_block_indices,
          num_tokens_per_block, dim_size_per_token_per_layer * dst_tensor.element_size(), total_token_in_kvcache,
          status)


def batch_scatter_kv_caches(
        kv_caches_ptrs_tensor: torch.Tensor,
        src_tensor: torch.Tensor,
        block_token_indices: IndexArg,
        src_block_indices: IndexArg,
        num_tokens_per_block: int,
        dim_size_per_token_per_layer: int,
        sm_count: int = 3,
        total_token_in_kvcache: Optional[int] = None,
        status: Optional[torch.Tensor] = None,
) -> None:
    """pool_p[block_token_indices[b*T + t], :] = src[src_block_indices[b], p, t, :]."""
    del sm_count
    _move("kvcm_b200_scatter_tokens", kv_caches_ptrs_tensor, src_tensor, block_token_indices, src_block_indices,
          num_tokens_per_block, dim_size_per_token_per_layer * src_tensor.element_size(), total_token_in_kvcache,
          status)


def batch_gather_kv_pages(kv_caches_ptrs_tensor: torch.Tensor, dst_tensor: torch.Tensor, block_page_table: IndexArg,
                          dst_block_indices: Optional[IndexArg], pages_per_block: int, page_bytes: int,
                          pool_pages: Optional[int] = None, status: Optional[torch.Tensor] = None) -> None:
    """Page-table form: the engine's block table addresses whole pages, so the per-token index
    list of generate_blocks_idx (kv_cache_manager/py_connector/vllm/v1_connector.py:308-320) is
    never built.  Byte-identical to batch_gather_kv_caches on the expanded token indices."""
    _move("kvcm_b200_gather_pages", kv_caches_ptrs_tensor, dst_tensor, block_page_table, dst_block_indices,
          pages_per_block, page_bytes, pool_pages, status)


def batch_scatter_kv_pages(kv_caches_ptrs_tensor: torch.Tensor, src_tensor: torch.Tensor, block_page_table: IndexArg,
                           src_block_indices: Optional[IndexArg], pages_per_block: int, page_bytes: int,
                           pool_pages: Optional[int] = None, status: Optional[torch.Tensor] = None) -> None:
    _move("kvcm_b200_scatter_pages", kv_caches_ptrs_tensor, src_tensor, block_page_table, src_block_indices,
          pages_per_block, page_bytes, pool_pages, status)
