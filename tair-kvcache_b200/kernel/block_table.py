"""Block-table helpers of the connector's worker side (host logic, vectorised).

generate_blocks_idx keeps the result of TairKvCacheConnector.generate_blocks_idx
(kv_cache_manager/py_connector/vllm/v1_connector.py:308-320) - the token slot of every token of every manager
block - without its Python double loop.  generate_block_page_table is what the page-table operators take
instead: one engine page id per page of a manager block, no per-token list at all.
"""
from typing import List, Sequence

import numpy as np


def generate_blocks_idx(manager_block_idxes: Sequence[int], local_block_ids: Sequence[int], manager_block_size: int,
                        local_block_size: int) -> List[List[int]]:
    """blocks_idx[b][i] = local_block_ids[(mb*M + i) // L] * L + (mb*M + i) % L for mb = manager_block_idxes[b]."""
    mb = np.asarray(manager_block_idxes, dtype=np.int64)
    ids = np.asarray(local_block_ids, dtype=np.int64)
    tok = mb[:, None] * manager_block_size + np.arange(manager_block_size, dtype=np.int64)[None, :]
    if tok.size and tok.max() // local_block_size >= len(ids):
        raise AssertionError("manager block reaches past the request's local blocks")
    return (ids[tok // local_block_size] * local_block_size + tok % local_block_size).tolist()


def generate_block_page_table(manager_block_idxes: Sequence[int], local_block_ids: Sequence[int],
                              manager_block_size: int, local_block_size: int) -> np.ndarray:
    """int32 [n_blocks, manager_block_size // local_block_size]: the engine pages of each manager block, for
    batch_gather_kv_pages / batch_scatter_kv_pages.  Needs manager_block_size % local_block_size == 0."""
    if manager_block_size % local_block_size != 0:
        raise ValueError("a manager block must be a whole number of engine pages for the page-table form")
    pages_per_block = manager_block_size // local_block_size
    mb = np.asarray(manager_block_idxes, dtype=np.int64)
    ids = np.asarray(local_block_ids, dtype=np.int64)
    page = mb[:, None] * pages_per_block + np.arange(pages_per_block, dtype=np.int64)[None, :]
    if page.size and page.max() >= len(ids):
        raise AssertionError("manager block reaches past the request's local blocks")
    return ids[page].astype(np.int32)
