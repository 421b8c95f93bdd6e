"""Byte-exact parity of the CUDA gather / scatter with the CPU oracle, through the C ABI.

Shapes of the first cases follow the reference's own kernel test
(kv_cache_manager/py_connector/test/kernel/test_batch_gather_scatter.py:9-216,301-494): seed 42,
4 layers x (K,V), 10240 tokens, 16 tokens per block, hidden 1024 bf16, 128 of 1024 staging blocks,
staging in pinned host memory and on the device; its edge case is one block of one token (:221-298).
Values are random 16-bit patterns (NaN payloads included) and every comparison is on raw bytes."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi
from tair_kvcache_b200.kernel import (CopyBufferAllocator, batch_gather_kv_caches, batch_gather_kv_pages,
                                      batch_scatter_kv_caches, batch_scatter_kv_pages, gather_kv_caches,
                                      scatter_kv_caches)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True, params=["bulk", "ldg"])
def mover(request):
    """Every case runs on both gather/scatter kernels: the bulk-copy ring and the vector mover."""
    _cabi.call("kvcm_b200_set_mover", 1 if request.param == "bulk" else 0, -1)
    yield request.param
    _cabi.call("kvcm_b200_set_mover", 1, -1)


def _rand_bytes(gen, n):
    return torch.randint(0, 256, (n,), dtype=torch.uint8, generator=gen)


def _make(seed, n_pools, pool_rows, row_bytes):
    gen = torch.Generator().manual_seed(seed)
    host = [_rand_bytes(gen, pool_rows * row_bytes) for _ in range(n_pools)]
    dev = [h.to(DEV) for h in host]
    ptrs = torch.tensor([d.data_ptr() for d in dev], dtype=torch.int64, device=DEV)
    return host, dev, ptrs


def _np(ts):
    return [t.numpy() for t in ts]


@pytest.mark.parametrize("staging_on", ["pinned_host", "pinned_host_zero_copy", "device"])
def test_gather_reference_shapes(staging_on):
    torch.manual_seed(42)
    n_layers, total_tokens, T, hidden, n_blocks, n_slots = 4, 10240, 16, 1024, 128, 1024
    P, row_bytes = n_layers * 2, hidden * 2
    host, dev, ptrs = _make(42, P, total_tokens, row_bytes)
    tok = torch.cat([torch.randperm(total_tokens)[:T] for _ in range(n_blocks)]).tolist()
    slots = torch.randperm(n_slots)[:n_blocks].tolist()
    if staging_on.startswith("pinned_host"):
        dst = torch.zeros(n_slots, P, T, hidden, dtype=torch.bfloat16, pin_memory=True)
    else:
        dst = torch.zeros(n_slots, P, T, hidden, dtype=torch.bfloat16, device=DEV)
    # pinned host staging goes through a device bounce buffer and the copy engines unless an SM budget is given,
    # in which case the kernel writes host memory itself (the reference's mode of operation)
    batch_gather_kv_caches(ptrs, dst, tok, slots, T, hidden, sm_count=8 if staging_on.endswith("zero_copy") else None)
    torch.cuda.synchronize()
    want = np.zeros(n_slots * P * T * row_bytes, dtype=np.uint8)
    assert oracle.move_rows(_np(host), want, tok, slots, T, row_bytes, 0, threads=4) == 0
    got = dst.cpu().view(torch.uint8).numpy().reshape(-1)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("staging_on", ["pinned_host", "pinned_host_zero_copy", "device"])
def test_scatter_reference_shapes(staging_on):
    torch.manual_seed(42)
    n_layers, total_tokens, T, hidden, n_blocks, n_slots = 4, 10240, 16, 1024, 128, 1024
    P, row_bytes = n_layers * 2, hidden * 2
    host, dev, ptrs = _make(43, P, total_tokens, row_bytes)
    tok = torch.randperm(total_tokens)[:n_blocks * T].tolist()  # unique rows, as the reference test uses
    slots = torch.randperm(n_slots)[:n_blocks].tolist()
    gen = torch.Generator().manual_seed(7)
    src_bytes = _rand_bytes(gen, n_slots * P * T * row_bytes)
    src = src_bytes.view(torch.bfloat16).view(n_slots, P, T, hidden)
    src = src.pin_memory() if staging_on.startswith("pinned_host") else src.to(DEV)
    batch_scatter_kv_caches(ptrs, src, tok, slots, T, hidden, sm_count=8 if staging_on.endswith("zero_copy") else None)
    torch.cuda.synchronize()
    want = [h.numpy().copy() for h in host]
    oracle.move_rows(want, src_bytes.numpy(), tok, slots, T, row_bytes, 1, threads=4)
    for p in range(P):
        assert np.array_equal(dev[p].cpu().numpy(), want[p]), p


def test_single_token_single_block_edge_case():
    host, dev, ptrs = _make(1, 8, 10240, 2048)
    dst = torch.zeros(4, 8, 1, 1024, dtype=torch.bfloat16, device=DEV)
    batch_gather_kv_caches(ptrs, dst, [777], [2], 1, 1024)
    torch.cuda.synchronize()
    want = np.zeros(4 * 8 * 2048, dtype=np.uint8)
    oracle.move_rows(_np(host), want, [777], [2], 1, 2048, 0)
    assert np.array_equal(dst.cpu().view(torch.uint8).numpy().reshape(-1), want)


def test_empty_batch_is_a_no_op():
    host, dev, ptrs = _make(2, 2, 64, 64)
    dst = torch.zeros(2, 2, 4, 32, dtype=torch.bfloat16, device=DEV)
    batch_gather_kv_caches(ptrs, dst, [], [], 4, 32)
    torch.cuda.synchronize()
    assert not dst.view(torch.uint8).any()


@pytest.mark.parametrize("row_bytes,rows_per_block", [(6, 5), (2, 3), (48, 7), (4098, 2), (40000, 3), (16, 1)])
def test_ragged_row_sizes_any_alignment(row_bytes, rows_per_block):
    n_pools, pool_rows, n_blocks, n_slots = 3, 101, 9, 12
    host, dev, ptrs = _make(row_bytes, n_pools, pool_rows, row_bytes)
    rng = np.random.default_rng(row_bytes)
    rows = rng.permutation(pool_rows)[:n_blocks * rows_per_block].astype(np.int32)
    slots = rng.permutation(n_slots)[:n_blocks].astype(np.int32)
    staging = torch.zeros(n_slots * n_pools * rows_per_block * row_bytes, dtype=torch.uint8, device=DEV)
    batch_gather_kv_pages(ptrs, staging, torch.from_numpy(rows), torch.from_numpy(slots), rows_per_block, row_bytes,
                          pool_rows)
    torch.cuda.synchronize()
    want = np.zeros(staging.numel(), dtype=np.uint8)
    oracle.move_rows(_np(host), want, rows, slots, rows_per_block, row_bytes, 0)
    assert np.array_equal(staging.cpu().numpy(), want)
    # scatter the staged bytes into zeroed pools: referenced rows come back, the rest stay zero
    zero = [torch.zeros_like(d) for d in dev]
    zptrs = torch.tensor([z.data_ptr() for z in zero], dtype=torch.int64, device=DEV)
    batch_scatter_kv_pages(zptrs, staging, torch.from_numpy(rows), torch.from_numpy(slots), rows_per_block,
                           row_bytes, pool_rows)
    torch.cuda.synchronize()
    wantp = [np.zeros_like(h.numpy()) for h in host]
    oracle.move_rows(wantp, want, rows, slots, rows_per_block, row_bytes, 1)
    for p in range(n_pools):
        assert np.array_equal(zero[p].cpu().numpy(), wantp[p])


def test_unaligned_pool_base_addresses():
    row_bytes, pool_rows, T = 64, 50, 4
    gen = torch.Generator().manual_seed(5)
    raw = [_rand_bytes(gen, pool_rows * row_bytes + 16).to(DEV) for _ in range(2)]
    views = [raw[0][3:3 + pool_rows * row_bytes], raw[1][8:8 + pool_rows * row_bytes]]
    ptrs = torch.tensor([v.data_ptr() for v in views], dtype=torch.int64, device=DEV)
    rows = np.arange(12, dtype=np.int32)[::-1].copy()
    staging = torch.zeros(3 * 2 * T * row_bytes, dtype=torch.uint8, device=DEV)
    batch_gather_kv_pages(ptrs, staging, torch.from_numpy(rows), None, T, row_bytes, pool_rows)
    torch.cuda.synchronize()
    want = np.zeros(staging.numel(), dtype=np.uint8)
    oracle.move_rows([v.cpu().numpy() for v in views], want, rows, None, T, row_bytes, 0)
    assert np.array_equal(staging.cpu().numpy(), want)


def test_out_of_range_rows_and_slots_are_skipped_and_counted():
    n_pools, pool_rows, row_bytes, T = 2, 32, 256, 4
    host, dev, ptrs = _make(9, n_pools, pool_rows, row_bytes)
    rows = np.array([0, 1, 2, 3, 4, 32, -1, 7, 8, 9, 10, 11], dtype=np.int32)  # block 1 has two bad rows
    slots = np.array([1, 0, 5], dtype=np.int32)  # block 2 names a slot that does not exist
    staging = torch.zeros(3 * n_pools * T * row_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    batch_gather_kv_pages(ptrs, staging, torch.from_numpy(rows), torch.from_numpy(slots), T, row_bytes, pool_rows,
                          status=status)
    torch.cuda.synchronize()
    want = np.zeros(staging.numel(), dtype=np.uint8)
    skipped = oracle.move_rows(_np(host), want, rows, slots, T, row_bytes, 0)
    assert np.array_equal(staging.cpu().numpy(), want)
    assert status[0].item() == skipped == 2 * n_pools + T * n_pools
    assert status[1].item() == 3  # 1 + largest offending block
    assert status[2].item() == 0  # no wait ran out


def test_host_staging_in_groups_smaller_than_the_batch(monkeypatch):
    """The bounce buffer holds fewer blocks than the call moves: several gather + copy rounds, ragged last group,
    consecutive and scattered host slots."""
    from tair_kvcache_b200.kernel import batch_gather_scatter_helper as helper
    n_pools, pool_pages, page_bytes, ppb, n_blocks, n_slots = 3, 300, 4096, 2, 37, 64
    monkeypatch.setattr(helper, "_BOUNCE_BYTES", 5 * n_pools * ppb * page_bytes)
    host, dev, ptrs = _make(21, n_pools, pool_pages, page_bytes)
    rng = np.random.default_rng(21)
    table = rng.permutation(pool_pages)[:n_blocks * ppb].astype(np.int32)
    slots = np.concatenate([np.arange(10, 30), rng.permutation(np.r_[0:10, 30:64])[:17]]).astype(np.int32)
    staging = torch.zeros(n_slots * n_pools * ppb * page_bytes, dtype=torch.uint8, pin_memory=True)
    batch_gather_kv_pages(ptrs, staging, torch.from_numpy(table), slots.tolist(), ppb, page_bytes, pool_pages)
    torch.cuda.synchronize()
    want = np.zeros(staging.numel(), dtype=np.uint8)
    oracle.move_rows(_np(host), want, table, slots, ppb, page_bytes, 0)
    assert np.array_equal(staging.numpy(), want)
    zero = [torch.zeros_like(d) for d in dev]
    zptrs = torch.tensor([z.data_ptr() for z in zero], dtype=torch.int64, device=DEV)
    batch_scatter_kv_pages(zptrs, staging, torch.from_numpy(table), torch.from_numpy(slots), ppb, page_bytes,
                           pool_pages)
    torch.cuda.synchronize()
    wantp = [np.zeros_like(h.numpy()) for h in host]
    oracle.move_rows(wantp, want, table, slots, ppb, page_bytes, 1)
    for p in range(n_pools):
        assert np.array_equal(zero[p].cpu().numpy(), wantp[p])
    with pytest.raises(_cabi.KvcmError):  # a slot outside the staging tensor is refused on the host
        batch_gather_kv_pages(ptrs, staging, torch.from_numpy(table[:ppb]), [n_slots], ppb, page_bytes, pool_pages)


def test_pybind_shim_and_ctypes_routes_agree(monkeypatch):
    """The operators reach the C ABI through the pybind shim when it is built; ctypes is the same call."""
    if _cabi.shim() is None:
        pytest.skip("pybind shim not built")
    host, dev, ptrs = _make(77, 4, 512, 4096)
    table = torch.randperm(512)[:64].to(torch.int32)
    via_shim = torch.zeros(16 * 4 * 4 * 4096, dtype=torch.uint8, device=DEV)
    via_ctypes = torch.zeros_like(via_shim)
    pinned = torch.zeros(16 * 4 * 4 * 4096, dtype=torch.uint8, pin_memory=True)
    batch_gather_kv_pages(ptrs, via_shim, table, None, 4, 4096, 512)
    batch_gather_kv_pages(ptrs, pinned, table, list(range(16)), 4, 4096, 512)
    monkeypatch.setattr(_cabi, "_shim", None)
    batch_gather_kv_pages(ptrs, via_ctypes, table, None, 4, 4096, 512)
    torch.cuda.synchronize()
    assert torch.equal(via_shim, via_ctypes) and via_shim.any()
    assert torch.equal(pinned, via_shim.cpu())
    with pytest.raises(_cabi.KvcmError):
        monkeypatch.undo()
        _cabi.call_move("kvcm_b200_gather_pages", ptrs.data_ptr(), 0, via_shim.data_ptr(), 1, table.data_ptr(), None,
                        1, 1, 16, 1, None, 0, None)


def test_page_table_form_equals_token_form():
    # Llama-3-8B geometry, shrunk: page 16 tokens x 2 KiB, block = 4 pages = 64 tokens
    n_pools, pool_pages, page_tokens, tok_bytes, pages_per_block, n_blocks = 6, 256, 16, 2048, 4, 40
    host, dev, ptrs = _make(11, n_pools, pool_pages * page_tokens, tok_bytes)
    rng = np.random.default_rng(11)
    table = rng.permutation(pool_pages)[:n_blocks * pages_per_block].astype(np.int32)
    slots = rng.permutation(n_blocks).astype(np.int32)
    # what generate_blocks_idx (kv_cache_manager/py_connector/vllm/v1_connector.py:308-320) would build
    tok = (table[:, None] * page_tokens + np.arange(page_tokens, dtype=np.int32)[None, :]).reshape(-1)
    T = pages_per_block * page_tokens
    a = torch.zeros(n_blocks * n_pools * T * tok_bytes, dtype=torch.uint8, device=DEV)
    b = torch.zeros_like(a)
    batch_gather_kv_pages(ptrs, a, torch.from_numpy(table), torch.from_numpy(slots), pages_per_block,
                          page_tokens * tok_bytes, pool_pages)
    batch_gather_kv_caches(ptrs, b.view(torch.bfloat16).view(n_blocks, n_pools, T, tok_bytes // 2), tok.tolist(),
                           slots.tolist(), T, tok_bytes // 2)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    want = np.zeros(a.numel(), dtype=np.uint8)
    oracle.move_rows(_np(host), want, tok, slots, T, tok_bytes, 0, threads=4)
    assert np.array_equal(a.cpu().numpy(), want)


def test_mla_shaped_block_roundtrip():
    # DeepSeek-style latent cache: one pool per layer, 576 bf16 per token, page = block = 64 tokens
    n_pools, pool_pages, page_bytes = 5, 40, 64 * 1152
    host, dev, ptrs = _make(13, n_pools, pool_pages, page_bytes)
    table = torch.randperm(pool_pages, generator=torch.Generator().manual_seed(1))[:17].to(torch.int32)
    staging = torch.zeros(17 * n_pools * page_bytes, dtype=torch.uint8, device=DEV)
    batch_gather_kv_pages(ptrs, staging, table, None, 1, page_bytes, pool_pages)
    zero = [torch.zeros_like(d) for d in dev]
    zptrs = torch.tensor([z.data_ptr() for z in zero], dtype=torch.int64, device=DEV)
    batch_scatter_kv_pages(zptrs, staging, table, None, 1, page_bytes, pool_pages)
    torch.cuda.synchronize()
    idx = table.long().to(DEV)
    for p in range(n_pools):
        assert torch.equal(zero[p].view(pool_pages, page_bytes)[idx], dev[p].view(pool_pages, page_bytes)[idx])
        assert int(zero[p].view(pool_pages, page_bytes).any(dim=1).sum()) == 17


def test_legacy_single_block_operators():
    # kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:279-317 self-test shapes
    torch.manual_seed(42)
    n_layers, total, n_tok, hidden = 4, 128, 32, 512
    gen = torch.Generator().manual_seed(42)
    host = [_rand_bytes(gen, 2 * total * hidden * 4) for _ in range(n_layers)]
    caches = [h.to(DEV).view(torch.float32).view(2, total, hidden) for h in host]
    ptrs = torch.tensor([c.data_ptr() for c in caches], device=DEV, dtype=torch.int64)
    tok = torch.randperm(total)[:n_tok].tolist()
    tok[5] = total + 3  # past the cache: skipped by the reference kernels
    dst = torch.zeros(n_layers, 2, n_tok, hidden, dtype=torch.float32, device=DEV)
    gather_kv_caches(ptrs, total, dst, tok)
    torch.cuda.synchronize()
    want = np.zeros(dst.numel() * 4, dtype=np.uint8)
    oracle.move_legacy(_np(host), total, want, tok, hidden * 4, 0)
    assert np.array_equal(dst.cpu().view(torch.uint8).numpy().reshape(-1), want)

    src_b = _rand_bytes(gen, dst.numel() * 4)
    src = src_b.to(DEV).view(torch.float32).view(n_layers, 2, n_tok, hidden)
    scatter_kv_caches(ptrs, total, src, tok)
    torch.cuda.synchronize()
    wantc = [h.numpy().copy() for h in host]
    oracle.move_legacy(wantc, total, src_b.numpy(), tok, hidden * 4, 1)
    for l in range(n_layers):
        assert np.array_equal(caches[l].cpu().view(torch.uint8).numpy().reshape(-1), wantc[l])


def test_copy_buffer_allocator_with_gather():
    alloc = CopyBufferAllocator(torch.device(DEV), torch.bfloat16, [2, 4, 64], 8)
    idx = alloc.alloc_buffer_idx_blocking(3)
    assert len(idx) == 3 and alloc._raw_buffer.shape == (8, 2, 4, 64)
    host, dev, ptrs = _make(3, 2, 64, 128)
    tok = list(range(12))
    batch_gather_kv_caches(ptrs, alloc._raw_buffer, tok, idx, 4, 64)
    torch.cuda.synchronize()
    bufs = alloc.get_buffer_by_idx(idx)
    for b in range(3):
        for p in range(2):
            want = dev[p].view(64, 128)[b * 4:(b + 1) * 4]
            assert torch.equal(bufs[b][p].view(torch.uint8).view(4, 128), want)
    alloc.free_buffer(idx)
    with pytest.raises(RuntimeError):
        alloc.free_buffer([0])


def test_large_roundtrip_property():
    """A few GiB, larger than L2: gather -> scatter into zeroed pools restores exactly the referenced pages,
    and the staged bytes equal a torch index_select of the pools."""
    n_pools, pool_pages, page_bytes, ppb, n_blocks = 8, 4096, 32768, 4, 512
    gen = torch.Generator(device=DEV).manual_seed(99)
    dev = [torch.randint(0, 1 << 31, (pool_pages * page_bytes // 4,), dtype=torch.int32, device=DEV, generator=gen)
           for _ in range(n_pools)]
    ptrs = torch.tensor([d.data_ptr() for d in dev], dtype=torch.int64, device=DEV)
    table = torch.randperm(pool_pages, device=DEV)[:n_blocks * ppb].to(torch.int32)
    slots = torch.randperm(n_blocks, device=DEV).to(torch.int32)
    staging = torch.zeros(n_blocks, n_pools, ppb, page_bytes // 4, dtype=torch.int32, device=DEV)
    batch_gather_kv_pages(ptrs, staging, table, slots, ppb, page_bytes, pool_pages)
    torch.cuda.synchronize()
    tl = table.long().view(n_blocks, ppb)
    for p in range(n_pools):
        want = dev[p].view(pool_pages, -1)[tl]  # [n_blocks, ppb, page]
        assert torch.equal(staging[slots.long(), p], want)
    zero = [torch.zeros_like(d) for d in dev]
    zptrs = torch.tensor([z.data_ptr() for z in zero], dtype=torch.int64, device=DEV)
    batch_scatter_kv_pages(zptrs, staging, table, slots, ppb, page_bytes, pool_pages)
    torch.cuda.synchronize()
    for p in range(n_pools):
        z = zero[p].view(pool_pages, -1)
        assert torch.equal(z[table.long()], dev[p].view(pool_pages, -1)[table.long()])
        assert int((z != 0).any(dim=1).sum()) == n_blocks * ppb


def test_pageable_host_staging_is_refused_not_dereferenced():
    host, dev, ptrs = _make(31, 1, 16, 64)
    pageable = np.zeros(4096, dtype=np.uint8)
    rows = torch.arange(4, dtype=torch.int32, device=DEV)
    _cabi.bind_device(0)
    rc = _cabi.lib().kvcm_b200_gather_tokens(ptrs.data_ptr(), 1, pageable.ctypes.data, 4, rows.data_ptr(), None, 4, 1,
                                             64, 16, None, 0, None)
    assert rc == _cabi.KVCM_ER_UNSUPPORTED_MEMORY_TYPE
    torch.cuda.synchronize()
    assert not pageable.any()
    with pytest.raises(ValueError):  # the Python operator says the same before reaching the library
        batch_gather_kv_pages(ptrs, torch.from_numpy(pageable), rows, None, 1, 64, 16)


def test_bad_arguments_return_codes():
    L = _cabi.lib()
    _cabi.bind_device(0)
    t = torch.zeros(64, dtype=torch.uint8, device=DEV)
    p = t.data_ptr()
    assert L.kvcm_b200_gather_tokens(p, 0, p, 1, p, None, 1, 1, 16, 1, None, 0, None) == _cabi.KVCM_ER_INVALID_PARAMS
    assert L.kvcm_b200_gather_tokens(p, 1, p, 1, p, None, 1, 1, 0, 1, None, 0, None) == _cabi.KVCM_ER_INVALID_PARAMS
    assert L.kvcm_b200_gather_tokens(None, 1, p, 1, p, None, 1, 1, 16, 1, None, 0, None) == _cabi.KVCM_ER_INVALID_ADDRESS
    assert L.kvcm_b200_gather_tokens(p, 1, p, 1, p, None, 1, 2, 1 << 30, 1, None, 0, None) == _cabi.KVCM_ER_INVALID_PARAMS


def test_token_lists_made_of_page_runs_take_the_page_path():
    """Llama-3-70B / TP8 geometry, shrunk: 256-byte token rows in pages of 32.  Token lists built from a block table
    are moved as 8 KiB page runs; lists that do not split into aligned runs, or that hold an out-of-range index,
    keep the per-token path - bytes and status words are the same either way."""
    from tair_kvcache_b200.kernel.batch_gather_scatter_helper import _coalesce_token_runs
    n_pools, pool_pages, page_tokens, tok_bytes, pages_per_block, n_blocks = 5, 128, 32, 256, 4, 24
    T = pages_per_block * page_tokens
    host, dev, ptrs = _make(21, n_pools, pool_pages * page_tokens, tok_bytes)
    rng = np.random.default_rng(21)
    table = rng.permutation(pool_pages)[:n_blocks * pages_per_block].astype(np.int64)
    slots = rng.permutation(n_blocks).astype(np.int32)
    tok = (table[:, None] * page_tokens + np.arange(page_tokens)[None, :]).reshape(-1)
    assert _coalesce_token_runs(tok.tolist(), slots.tolist(), T, pool_pages * page_tokens, n_blocks)[1:] == (4, 32)
    broken = tok.copy()
    broken[5], broken[6] = broken[6], broken[5]  # same tokens, one run out of order: runs of 4 at best... not even
    assert _coalesce_token_runs(broken.tolist(), slots.tolist(), T, None, n_blocks) is None
    outside = tok.copy()
    outside[40] = pool_pages * page_tokens + 3
    assert _coalesce_token_runs(outside.tolist(), slots.tolist(), T, pool_pages * page_tokens, n_blocks) is None
    for name, idx, skipped in (("runs", tok, 0), ("broken", broken, 0), ("outside", outside, n_pools)):
        for staging_on in ("device", "pinned_host"):
            stage = torch.zeros(n_blocks * n_pools * T * tok_bytes, dtype=torch.uint8,
                                device=DEV if staging_on == "device" else "cpu")
            if staging_on != "device":
                stage = stage.pin_memory()
            status = torch.zeros(4, dtype=torch.int32, device=DEV)
            batch_gather_kv_caches(ptrs, stage.view(torch.bfloat16).view(n_blocks, n_pools, T, tok_bytes // 2),
                                   idx.tolist(), slots.tolist(), T, tok_bytes // 2,
                                   total_token_in_kvcache=pool_pages * page_tokens, status=status)
            torch.cuda.synchronize()
            want = np.zeros(stage.numel(), dtype=np.uint8)
            oracle.move_rows(_np(host), want, idx.astype(np.int32), slots, T, tok_bytes, 0, threads=4)
            assert np.array_equal(stage.cpu().numpy(), want), (name, staging_on)
            assert status[0].item() == skipped, (name, staging_on)
            # and back: scatter into zeroed pools restores exactly the referenced tokens
            zero = [torch.zeros_like(d) for d in dev]
            zptrs = torch.tensor([z.data_ptr() for z in zero], dtype=torch.int64, device=DEV)
            batch_scatter_kv_caches(zptrs, stage.view(torch.bfloat16).view(n_blocks, n_pools, T, tok_bytes // 2),
                                    idx.tolist(), slots.tolist(), T, tok_bytes // 2,
                                    total_token_in_kvcache=pool_pages * page_tokens)
            torch.cuda.synchronize()
            wantp = [np.zeros_like(h.numpy()) for h in host]
            oracle.move_rows(wantp, want, idx.astype(np.int32), slots, T, tok_bytes, 1, threads=4)
            for z, w in zip(zero, wantp):
                assert np.array_equal(z.cpu().numpy(), w), (name, staging_on)


def test_bounded_wait_gives_up_reports_and_leaves_the_context_usable():
    """The give-up path of the kernels' mbarrier waits, run once in a form with nothing in flight: a barrier armed
    for bytes that are never sent, polled through the shared helper with a limit of a few polls.  The call comes
    back at once with the status words set, and the next gather is bit-exact."""
    import time
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    _cabi.bind_device(0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _cabi.call("kvcm_b200_selftest_bounded_wait", 64, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert status.cpu().tolist()[:2] == [1, 64]          # gave up after exactly the polls it was allowed
    for bad in (0, 1 << 20):
        assert _cabi.lib().kvcm_b200_selftest_bounded_wait(bad, status.data_ptr(), None) == _cabi.KVCM_ER_INVALID_PARAMS
    # the context is intact: a gather on the bulk-copy ring right after it, against the oracle
    host, dev, ptrs = _make(4, 4, 64, 16 * 2048)
    table = np.random.default_rng(0).permutation(64)[:32].astype(np.int32)
    staging = torch.zeros(8 * 4 * 4 * 16 * 2048, dtype=torch.uint8, device=DEV)
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    batch_gather_kv_pages(ptrs, staging, torch.from_numpy(table), None, 4, 16 * 2048, 64, status=st)
    torch.cuda.synchronize()
    want = np.zeros(staging.numel(), dtype=np.uint8)
    oracle.move_rows(_np(host), want, table, None, 4, 16 * 2048, 0)
    assert np.array_equal(staging.cpu().numpy(), want) and st.cpu().tolist()[2] == 0


@pytest.mark.parametrize("use_mla", [False, True])
def test_trtllm_block_major_layout(use_mla):
    """The TensorRT-LLM connector's pool is ONE tensor [num_blocks, num_layers, kv_factor, block_size] with
    block_size = kv heads x head size x tokens per block and kv_factor 1 under MLA
    (kv_cache_manager/py_connector/trtllm/connector.py:173-179): a block is one contiguous row.  The reference saves
    a block as `kv_cache_tensor[block_id].cpu()` handed over as one iov and loads it with
    `kv_cache_tensor[block_id].copy_(cpu_tensor)` (:209-216, :261-279).  Here that is the page form with one pool,
    one row per block and the block ids as the page table; the staged bytes must be those very tensors."""
    num_blocks, num_layers, kv_factor = 96, 6, 1 if use_mla else 2
    block_size = (1 * 576 if use_mla else 8 * 128) * 32          # elements: heads x head size x 32 tokens per block
    gen = torch.Generator(device=DEV).manual_seed(17)
    kv_cache_tensor = torch.randint(-(1 << 15), 1 << 15, (num_blocks, num_layers, kv_factor, block_size),
                                    dtype=torch.int16, device=DEV, generator=gen).view(torch.bfloat16)
    row_bytes = num_layers * kv_factor * block_size * 2          # the connector's location_spec_size
    ptrs = torch.tensor([kv_cache_tensor.data_ptr()], dtype=torch.int64, device=DEV)
    block_ids = [77, 3, 41, 42, 0, 95, 18]
    # save: one staging slot per block, in pinned host memory
    staged = torch.zeros(len(block_ids), num_layers, kv_factor, block_size, dtype=torch.bfloat16, pin_memory=True)
    batch_gather_kv_pages(ptrs, staged, block_ids, None, 1, row_bytes, num_blocks)
    torch.cuda.synchronize()
    for slot, block_id in enumerate(block_ids):
        cpu_tensor = kv_cache_tensor[block_id].cpu()             # what the reference hands to SaveKvCaches
        assert torch.equal(staged[slot].view(torch.int16), cpu_tensor.view(torch.int16))
    # load: into an engine pool that holds other bytes, through other block ids
    target = torch.zeros_like(kv_cache_tensor)
    tptrs = torch.tensor([target.data_ptr()], dtype=torch.int64, device=DEV)
    new_ids = [5, 6, 90, 1, 50, 51, 52]
    batch_scatter_kv_pages(tptrs, staged, new_ids, None, 1, row_bytes, num_blocks)
    torch.cuda.synchronize()
    want = torch.zeros_like(kv_cache_tensor)
    for slot, block_id in enumerate(new_ids):
        want[block_id].copy_(staged[slot])                       # the reference's load
    assert torch.equal(target.view(torch.int16), want.view(torch.int16))
    # the same bytes through the oracle's index rule
    pool = kv_cache_tensor.view(torch.uint8).reshape(-1).cpu().numpy()
    ref = np.zeros(len(block_ids) * row_bytes, dtype=np.uint8)
    oracle.move_rows([pool], ref, np.array(block_ids, dtype=np.int32), None, 1, row_bytes, 0)
    assert np.array_equal(staged.view(torch.uint8).reshape(-1).numpy(), ref)
