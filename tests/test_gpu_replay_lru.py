"""Parity of the GPU quota sweep (LRU eviction) with the oracle's sequential radix-tree replay."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import (TRACE_DIALOG_TURN, TRACE_GET_LOCATION, TRACE_WRITE_CACHE, RunTraces,
                                         RunTracesLru, replay_lru_workspace_bytes)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
W, G, D = TRACE_WRITE_CACHE, TRACE_GET_LOCATION, TRACE_DIALOG_TURN


def _gpu(keys, off, types, quotas, mask=None, **kw):
    r = RunTracesLru(torch.tensor(keys, dtype=torch.int64, device=DEV),
                     torch.tensor(off, dtype=torch.int64, device=DEV),
                     torch.tensor(types, dtype=torch.uint8, device=DEV), quotas,
                     torch.tensor(mask, dtype=torch.int64, device=DEV) if mask is not None else None, **kw)
    torch.cuda.synchronize()
    ext, inte, wr, size, totals = [t.cpu().numpy() for t in r]
    # the totals per configuration are the sums of the per-trace records and the last cache size
    if ext.shape[1] > 0:
        assert np.array_equal(totals, np.stack([ext.sum(1), inte.sum(1), wr.sum(1), size[:, -1]], axis=1))
    return [ext, inte, wr, size]


def test_reference_policy_known_answers():
    # kv_cache_manager/optimizer/test/lru_eviction_policy_test.cc:44-65 and :67-96 as traces (see tests/test_oracle.py)
    ext, inte, wr, size = _gpu([1, 2, 1, 3, 2, 1, 3], [0, 1, 2, 3, 4, 5, 6, 7], [W, W, G, W, G, G, G], [2],
                               evict_batch=1, precise=True)
    assert wr[0].tolist() == [1, 1, 0, 1, 0, 0, 0] and ext[0].tolist() == [0, 0, 1, 0, 0, 1, 1]
    assert size[0].tolist() == [1, 2, 2, 2, 2, 2, 2]
    ext, inte, wr, size = _gpu([1, 2, 3, 1, 2, 3], [0, 1, 2, 3, 4, 5, 6], [W, W, W, G, G, G], [1], evict_batch=1,
                               precise=True)
    assert size[0].tolist() == [1] * 6 and ext[0].tolist() == [0, 0, 0, 0, 0, 1]
    # kv_cache_manager/optimizer/test/optimizer_manager_py_test.py:57-84 with room for everything
    ext, inte, wr, size = _gpu([1, 2, 3, 1, 2, 4], [0, 3, 6], [W, G], [12000])
    assert ext[0].tolist() == [0, 2] and wr[0].tolist() == [3, 0] and size[0].tolist() == [3, 3]


def test_rough_and_precise_modes():
    keys = list(range(1, 12))
    for precise, want in ((True, [7, 7]), (False, [6, 7])):
        size = _gpu(keys, [0, 10, 11], [W, W], [7], evict_batch=2, precise=precise)[3]
        assert size[0].tolist() == want
    # a batch larger than the list empties it
    ext, inte, wr, size = _gpu([1, 2, 1], [0, 1, 2, 3], [W, W, G], [1], evict_batch=10, precise=False)
    assert size[0].tolist() == [1, 0, 0] and ext[0].tolist() == [0, 0, 0]


def _workload(rng, n_traces, rw_separation, max_blocks=40):
    """Chained keys of token sequences that share prefixes with earlier ones."""
    bs = 16
    seqs, keys, off, types, mask = [], [], [0], [], []
    for t in range(n_traces):
        n = int(rng.integers(0, max_blocks)) * bs + int(rng.integers(0, bs))
        toks = rng.integers(0, 50000, size=n).astype(np.int64)
        if seqs and rng.random() < 0.8:
            src = seqs[int(rng.zipf(1.3)) % len(seqs)]
            m = int(rng.integers(0, min(len(src), n) + 1))
            toks[:m] = src[:m]
        seqs.append(toks)
        k = oracle.gen_key_vector(toks, bs)
        keys.append(k)
        off.append(off[-1] + len(k))
        ty = (G if rng.random() < 0.5 else W) if rw_separation else D
        types.append(ty)
        mask.append(int(rng.integers(0, len(k) + 2)) if ty == G and rng.random() < 0.5 else 0)
    return np.concatenate(keys + [np.zeros(0, np.int64)]), np.array(off), np.array(types, np.uint8), np.array(mask)


@pytest.mark.parametrize("rw_separation", [False, True])
@pytest.mark.parametrize("precise", [False, True])
def test_quota_sweep_against_sequential_oracle(rw_separation, precise):
    rng = np.random.default_rng(50 + 2 * rw_separation + precise)
    keys, off, types, mask = _workload(rng, 2500, rw_separation)
    quotas = [1, 7, 33, 100, 257, 1000, 5000, 1 << 40]
    batch = 1 if precise else 13
    got = _gpu(keys, off, types, quotas, mask, evict_batch=batch, precise=precise)
    evicting = 0
    for c, q in enumerate(quotas):
        want = oracle.LruReplay(q, evict_batch=batch, precise=precise).run(keys, off, types, mask)
        for name, a, b in zip(("ext", "int", "written", "cached"), want, got):
            assert np.array_equal(a, b[c]), (name, q)
        evicting += int(want[3].max() <= q + batch and q < 5000)
    assert evicting >= 5
    # with room for everything the sweep agrees with the eviction-free replay entry point
    plain = RunTraces(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                      torch.from_numpy(mask).to(DEV))
    for a, b in zip(plain, got):
        assert np.array_equal(a.cpu().numpy(), b[-1])


def test_long_requests_and_many_configurations():
    """Requests longer than one 32-key pass, more configurations than SMs, workspace reuse."""
    rng = np.random.default_rng(77)
    keys, off, types, mask = _workload(rng, 400, True, max_blocks=300)
    quotas = [int(q) for q in rng.integers(1, 20000, size=200)]
    ws = torch.empty(replay_lru_workspace_bytes(len(keys), len(quotas)), dtype=torch.uint8, device=DEV)
    ws.fill_(0xAB)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for _ in range(2):  # the second call finds the first call's leftovers in the workspace
        got = _gpu(keys, off, types, quotas, mask, evict_batch=100, precise=False, workspace=ws, status=status)
    assert status[0].item() == 0
    for c in rng.choice(len(quotas), size=12, replace=False):
        want = oracle.LruReplay(quotas[c], evict_batch=100, precise=False).run(keys, off, types, mask)
        for a, b in zip(want, got):
            assert np.array_equal(a, b[c]), quotas[c]


def test_empty_and_rejected_inputs():
    ext, inte, wr, size = _gpu([], [0, 0, 0], [W, G], [5])
    assert ext.shape == (1, 2) and size[0].tolist() == [0, 0]
    from tair_kvcache_b200 import _cabi
    with pytest.raises(_cabi.KvcmError):
        _gpu([1], [0, 1], [W], [5], evict_batch=0)
    with pytest.raises(ValueError):
        _gpu([1], [0, 1], [W], [])


def test_totals_only_sweep():
    rng = np.random.default_rng(91)
    keys, off, types, mask = _workload(rng, 800, True)
    quotas = [5, 80, 700, 1 << 40]
    full = _gpu(keys, off, types, quotas, mask, evict_batch=7)
    r = RunTracesLru(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                     quotas, torch.from_numpy(mask).to(DEV), evict_batch=7, per_trace=False)
    assert r.external_hit_blocks is None and r.current_cache_blocks is None
    want = np.stack([full[0].sum(1), full[1].sum(1), full[2].sum(1), full[3][:, -1]], axis=1)
    assert np.array_equal(r.totals.cpu().numpy(), want)


def test_vector_masks_with_holes_under_eviction():
    rng = np.random.default_rng(92)
    keys, off, types, mask = _workload(rng, 1200, True)
    bits = (rng.random(len(keys)) < 0.25).astype(np.uint8)
    quotas = [20, 300, 1 << 40]
    got = _gpu(keys, off, types, quotas, mask, evict_batch=9, mask_bits=torch.from_numpy(bits).to(DEV))
    for c, q in enumerate(quotas):
        want = oracle.LruReplay(q, evict_batch=9).run(keys, off, types, mask, mask_bits=bits)
        for a, b in zip(want, got):
            assert np.array_equal(a, b[c]), q
