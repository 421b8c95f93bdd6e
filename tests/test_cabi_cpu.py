"""The C-ABI library on a box without a GPU: it loads, exports every declared symbol, and refuses
to compute (no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi


def _declared_symbols():
    names = []
    inc = os.path.join(ROOT, "include")
    for fn in sorted(os.listdir(inc)):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            names += re.findall(r"KVCM_API\s+[\w\s\*]+?\b(kvcm_b200_\w+)\s*\(", text)
    return names


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 25
    L = ctypes.CDLL(_cabi.LIB_PATH)
    for name in names:
        assert hasattr(L, name), name
    # and the Python binding knows each of them
    assert set(names) == set(_cabi.SIGNATURES)


def test_abi_version_and_error_strings():
    assert _cabi.lib().kvcm_b200_abi_version() == 1
    assert "no CPU path" in _cabi.error_string(_cabi.KVCM_ER_NO_DEVICE)
    assert _cabi.error_string(_cabi.KVCM_EC_BADARGS) == "bad arguments"


def test_key_offsets_host_helper():
    from tair_kvcache_b200.manager import key_offsets
    assert key_offsets([0, 5, 64, 130, 130], 64).tolist() == [0, 0, 0, 1, 1]
    with pytest.raises(_cabi.KvcmError):
        key_offsets([0, 5], 0)


def test_iovs_to_segments_honours_ignore():
    iovs = (_cabi.Iov * 3)()
    bufs = [np.zeros(8, np.uint8), None, np.zeros(4, np.uint8)]
    for i, (b, size, ign) in enumerate([(bufs[0], 8, 0), (None, 4, 1), (bufs[2], 4, 0)]):
        iovs[i].type = 1
        iovs[i].ignore = ign
        iovs[i].base = b.ctypes.data if b is not None else None
        iovs[i].size = size
    segs = (_cabi.Seg * 3)()
    n, span = ctypes.c_int32(), ctypes.c_uint64()
    string = np.zeros(16, np.uint8)
    _cabi.call("kvcm_b200_iovs_to_segments", ctypes.addressof(iovs), 3, string.ctypes.data, 0,
               ctypes.addressof(segs), ctypes.addressof(n), ctypes.addressof(span))
    assert (n.value, span.value) == (2, 16)
    assert segs[0].dst == string.ctypes.data and segs[0].src == bufs[0].ctypes.data and segs[0].bytes == 8
    assert segs[1].dst == string.ctypes.data + 12 and segs[1].bytes == 4
    _cabi.call("kvcm_b200_iovs_to_segments", ctypes.addressof(iovs), 3, string.ctypes.data, 1,
               ctypes.addressof(segs), ctypes.addressof(n), ctypes.addressof(span))
    assert segs[1].src == string.ctypes.data + 12 and segs[1].dst == bufs[2].ctypes.data


def test_iovs_to_segments_refuses_pageable_cpu_iovs():
    """An iov of MemoryType CPU in ordinary memory (which the reference copies with std::memcpy,
    kv_cache_manager/client/src/internal/sdk/local_file_sdk.cc:231-233) never lands in a table a kernel reads."""
    iovs = (_cabi.Iov * 2)()
    gpu_like, cpu_buf = np.zeros(8, np.uint8), np.zeros(8, np.uint8)
    for i, (b, ty, ign) in enumerate([(gpu_like, 1, 0), (cpu_buf, 0, 0)]):
        iovs[i].type, iovs[i].ignore, iovs[i].base, iovs[i].size = ty, ign, b.ctypes.data, 8
    segs = (_cabi.Seg * 2)()
    n, span = ctypes.c_int32(), ctypes.c_uint64()
    string = np.zeros(16, np.uint8)
    rc = _cabi.lib().kvcm_b200_iovs_to_segments(ctypes.addressof(iovs), 2, string.ctypes.data, 0,
                                                ctypes.addressof(segs), ctypes.addressof(n), ctypes.addressof(span))
    assert rc == _cabi.KVCM_ER_UNSUPPORTED_MEMORY_TYPE
    iovs[1].ignore = 1  # moved by the caller on the host: skipped, its bytes still counted in the span
    _cabi.call("kvcm_b200_iovs_to_segments", ctypes.addressof(iovs), 2, string.ctypes.data, 0,
               ctypes.addressof(segs), ctypes.addressof(n), ctypes.addressof(span))
    assert (n.value, span.value) == (1, 16)


def test_compute_entry_points_refuse_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = _cabi.lib()
    one = ctypes.c_void_p(16)
    assert L.kvcm_b200_gather_tokens(one, 1, one, 1, one, None, 1, 1, 16, 1, None, 0, None) == _cabi.KVCM_ER_NO_DEVICE
    assert L.kvcm_b200_hash_blocks_u32(one, 4, one, 1, 1, one, one, None, 0, None) == _cabi.KVCM_ER_NO_DEVICE
    h = ctypes.c_void_p()
    assert L.kvcm_b200_index_create(10, ctypes.byref(h)) == _cabi.KVCM_ER_NO_DEVICE and not h.value
    assert L.kvcm_b200_copy_segments(one, 1, None) == _cabi.KVCM_ER_NO_DEVICE


def test_encode_locations_matches_oracle_predicates():
    from oracle import kvcm_oracle as oracle
    from tair_kvcache_b200.manager.block_index import avail_mask_from_weights, encode_locations
    rng = np.random.default_rng(0)
    for weights in [(1, 3, 3, 3, 5), (1, 0, 3, 0, 5), (0, 0, 0, 0, 0)]:
        avail = avail_mask_from_weights(weights)
        for _ in range(200):
            locs = [(int(rng.integers(0, 5)), int(rng.integers(0, 6))) for _ in range(int(rng.integers(0, 4)))]
            ix = oracle.Index()
            ix.put([7], [locs])
            f = int(ix.batch_get([7], weights=weights)[0])
            w = encode_locations(locs)
            assert bool(f & 1) == bool(w & avail & 0xFFFF)
            assert bool(f & 4) == bool(w & _cabi.VAL_NONEMPTY)
            assert bool(f & 8) == bool((w >> 16) & avail & 0xFFFF)


def test_block_table_helpers_match_the_connector_loop():
    from tair_kvcache_b200.kernel.block_table import generate_block_page_table, generate_blocks_idx

    def reference_loop(manager_block_idxes, local_block_ids, M, L):
        # the double loop of kv_cache_manager/py_connector/vllm/v1_connector.py:308-320, restated
        out = []
        for mb in manager_block_idxes:
            row = []
            for i in range(M):
                t = mb * M + i
                row.append(local_block_ids[t // L] * L + t % L)
            out.append(row)
        return out

    rng = np.random.default_rng(4)
    for M, L in [(64, 16), (16, 16), (32, 64), (48, 16)]:
        n_local = 40
        ids = rng.permutation(1000)[:n_local].tolist()
        n_manager = n_local * L // M
        mbs = rng.permutation(n_manager)[:min(7, n_manager)].tolist()
        assert generate_blocks_idx(mbs, ids, M, L) == reference_loop(mbs, ids, M, L)
        if M % L == 0:
            table = generate_block_page_table(mbs, ids, M, L)
            tok = (table[:, :, None].astype(np.int64) * L + np.arange(L)[None, None, :]).reshape(len(mbs), M)
            assert tok.tolist() == reference_loop(mbs, ids, M, L)
    with pytest.raises(ValueError):
        generate_block_page_table([0], [1, 2], 32, 64)


def test_partial_sort_restatement_matches_the_standard_library():
    """The heap-select + sort-heap routine the random_lru sweep orders its samples with, run on the host through
    the C ABI, against std::partial_sort called the way the reference calls it
    (kv_cache_manager/optimizer/eviction_policy/random_lru.cc:59-82): same order of the first k, ties included."""
    from oracle import kvcm_oracle as oracle
    rng = np.random.default_rng(21)
    for trial in range(300):
        n_blocks = int(rng.integers(1, 400))
        times = rng.integers(0, int(rng.integers(1, 12)), size=n_blocks).astype(np.int64)  # few distinct times: ties
        n = int(rng.integers(1, 300))
        k = int(rng.integers(0, n + 1))
        sample = rng.integers(0, n_blocks, size=n).astype(np.uint64)                        # with repeats
        want = oracle.partial_sort_by_time(sample, k, times)
        idx = sample.astype(np.uint32)
        t = times[sample.astype(np.int64)].copy()
        rc = _cabi.lib().kvcm_b200_selftest_partial_sort(idx.ctypes.data, t.ctypes.data, k, n)
        assert rc == _cabi.KVCM_OK
        assert np.array_equal(idx[:k].astype(np.uint64), want[:k]), (trial, n, k)
        assert np.array_equal(t[:k], times[want[:k].astype(np.int64)])
    assert _cabi.lib().kvcm_b200_selftest_partial_sort(None, None, 0, 0) == _cabi.KVCM_ER_INVALID_ADDRESS


def test_workspace_sizes_of_the_write_batch_and_the_policy_group_need_no_device():
    """Host arithmetic only: sizes grow with the batch, are 256-byte multiples, and bad arguments give -1."""
    L = _cabi.lib()
    small = L.kvcm_b200_start_write_workspace_bytes(1000, 10)
    large = L.kvcm_b200_start_write_workspace_bytes(100000, 1000)
    assert 0 < small < large and small % 256 == 0 and large % 256 == 0
    assert L.kvcm_b200_start_write_workspace_bytes(0, 0) > 0
    assert L.kvcm_b200_start_write_workspace_bytes(-1, 10) == -1
    assert L.kvcm_b200_start_write_workspace_bytes(10, -1) == -1

    size = L.kvcm_b200_replay_policy_group_workspace_bytes
    plain = np.array([_cabi.POLICY_LRU, _cabi.POLICY_LEAF_AWARE_LRU, _cabi.POLICY_LEAF_AWARE_LRU], np.uint8)
    mixed = np.array([_cabi.POLICY_LRU, _cabi.POLICY_LEAF_AWARE_LRU, _cabi.POLICY_RANDOM_LRU], np.uint8)
    a = size(1000, 10, 4, plain.ctypes.data, 3)
    b = size(1000, 10, 4, mixed.ctypes.data, 3)
    assert 0 < a < b and a % 256 == 0 and b % 256 == 0  # a sampled instance adds its block and stamp vectors
    assert size(1000, 10, 4, np.array([0, 9], np.uint8).ctypes.data, 2) == -1  # no such policy
    assert size(-1, 10, 4, mixed.ctypes.data, 3) == -1
    assert size(1000, 10, 4, None, 3) == a  # no policy bytes: no sampled instance
    assert L.kvcm_b200_replay_leaf_lru_group_workspace_bytes(1000, 10, 4, 3) == a
