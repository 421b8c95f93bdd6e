"""Host-side logic of the Python operators that needs no GPU."""
import threading
import time

import pytest
import torch

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.kernel.batch_gather_scatter_helper import _coalesce_token_runs
from tair_kvcache_b200.kernel.gather_scatter_helper import CopyBufferAllocator
from tair_kvcache_b200.kernel.block_table import generate_block_page_table, generate_blocks_idx


def _tokens(pages, page):
    return [p * page + i for p in pages for i in range(page)]


def test_block_table_lists_become_page_runs():
    # the list generate_blocks_idx (kv_cache_manager/py_connector/vllm/v1_connector.py:308-320) builds for two blocks
    # of four 16-token pages
    idx = _tokens([5, 2, 9, 7, 0, 11, 3, 8], 16)
    rows, per_block, g = _coalesce_token_runs(idx, [1, 0], 64, 12 * 16, 2)
    assert (rows.tolist(), per_block, g) == ([5, 2, 9, 7, 0, 11, 3, 8], 4, 16)
    # consecutive pages merge further: one run of 64 tokens per block
    rows, per_block, g = _coalesce_token_runs(_tokens([4, 5, 6, 7, 8, 9, 10, 11], 16), None, 64, None, 2)
    assert (rows.tolist(), per_block, g) == ([1, 2], 1, 64)
    # a block length that is not a power of two: 48 = 3 pages of 16
    rows, per_block, g = _coalesce_token_runs(_tokens([3, 1, 2], 16), None, 48, None, 1)
    assert (per_block, g) == (3, 16) and rows.tolist() == [3, 1, 2]


def test_lists_that_must_keep_the_token_path():
    idx = _tokens([5, 2, 9, 7], 16)
    assert _coalesce_token_runs(idx, [0], 64, None, 1) is not None
    swapped = list(idx)
    swapped[1], swapped[2] = swapped[2], swapped[1]
    assert _coalesce_token_runs(swapped, [0], 64, None, 1) is None            # a run out of order
    assert _coalesce_token_runs([i + 1 for i in idx], [0], 64, None, 1) is None  # runs not aligned to their length
    assert _coalesce_token_runs(idx, [0], 64, 100, 1) is None                 # an index beyond the pool
    assert _coalesce_token_runs([-1] + idx[1:], [0], 64, None, 1) is None     # a negative index
    assert _coalesce_token_runs(idx, [3], 64, None, 1) is None                # a staging slot out of range
    assert _coalesce_token_runs(idx, [0], 64, 10 * 16 + 8, 1)[2] == 8         # pool size only a multiple of 8
    assert _coalesce_token_runs([7], [0], 1, None, 1) is None                 # one token per block: nothing to merge
    assert _coalesce_token_runs([], None, 64, None, 0) is None


def test_generate_blocks_idx_matches_the_reference_loop():
    # kv_cache_manager/py_connector/vllm/v1_connector.py:308-320 restated as the double loop it is
    local_block_ids, page, T = [7, 3, 9, 1, 4, 6], 16, 32
    manager_blocks = [2, 0, 1]
    want = []
    for mb in manager_blocks:
        want.append([local_block_ids[(mb * T + i) // page] * page + (mb * T + i) % page for i in range(T)])
    assert generate_blocks_idx(manager_blocks, local_block_ids, T, page) == want
    assert generate_block_page_table(manager_blocks, local_block_ids, T, page).tolist() == [[4, 6], [7, 3], [9, 1]]
    # and the list it yields is one the operators turn back into page runs
    flat = [t for row in want for t in row]
    rows, per_block, g = _coalesce_token_runs(flat, [0, 1, 2], T, None, 3)
    assert (rows.tolist(), per_block, g) == ([4, 6, 7, 3, 9, 1], 2, 16)


def test_copy_buffer_allocator_surface_and_refusals():
    # public surface of kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:175-252
    alloc = CopyBufferAllocator(torch.device("cpu"), torch.bfloat16, [2, 4, 8], 6)
    assert alloc.max_count == 6 and tuple(alloc._raw_buffer.shape) == (6, 2, 4, 8) and tuple(alloc.shape) == (2, 4, 8)
    a = alloc.alloc_buffer_idx_blocking(4)
    b = alloc.alloc_buffer_idx_blocking(2)
    assert sorted(a + b) == list(range(6))
    views = alloc.get_buffer_by_idx(a)
    views[0].fill_(1.0)
    assert float(alloc._raw_buffer[a[0]].sum()) == 2 * 4 * 8  # the views alias the raw buffer
    for bad in (0, -1, 7):
        with pytest.raises(ValueError):
            alloc.alloc_buffer_idx_blocking(bad)
    with pytest.raises(ValueError):
        alloc.free_buffer([6])
    with pytest.raises(ValueError):
        alloc.free_buffer([-1])
    alloc.free_buffer([])  # nothing to do
    alloc.free_buffer(b)
    with pytest.raises(RuntimeError):
        alloc.free_buffer(b)           # already back in the pool
    with pytest.raises(RuntimeError):
        alloc.free_buffer([a[0], a[0]])  # the same slot twice in one call
    assert sorted(alloc.alloc_buffer_idx_blocking(2)) == sorted(b)  # the refused calls changed nothing
    with pytest.raises(ValueError):
        CopyBufferAllocator(torch.device("cpu"), torch.uint8, [1], 0)


def test_copy_buffer_allocator_blocks_until_enough_is_free():
    alloc = CopyBufferAllocator(torch.device("cpu"), torch.uint8, [16], 4)
    held = alloc.alloc_buffer_idx_blocking(3)
    got, order = {}, []

    def want(name, n):
        got[name] = alloc.alloc_buffer_idx_blocking(n)
        order.append(name)

    big = threading.Thread(target=want, args=("big", 3))
    big.start()
    time.sleep(0.1)
    small = threading.Thread(target=want, args=("small", 1))  # would fit at once, but queues behind the older request
    small.start()
    time.sleep(0.1)
    assert big.is_alive() and small.is_alive() and not got
    alloc.free_buffer(held[:1])          # 2 free: still not enough for the head of the queue
    time.sleep(0.1)
    assert big.is_alive() and small.is_alive()
    alloc.free_buffer(held[1:])          # 4 free: big takes 3, then small takes the last
    big.join(5)
    small.join(5)
    assert not big.is_alive() and not small.is_alive()
    assert order == ["big", "small"] and sorted(got["big"] + got["small"]) == [0, 1, 2, 3]
    alloc.free_buffer(got["big"])
    alloc.free_buffer(got["small"])
    assert sorted(alloc.alloc_buffer_idx_blocking(4)) == [0, 1, 2, 3]
