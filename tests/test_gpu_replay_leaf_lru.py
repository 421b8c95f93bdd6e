"""Parity of the GPU quota sweep under the "leaf_aware_lru" policy with the oracle's sequential radix-tree replay.
The reference has no test of this policy; the known answers below are the hand-worked cases of tests/test_oracle.py."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import (TRACE_DIALOG_TURN, TRACE_GET_LOCATION, TRACE_WRITE_CACHE, RunTraces,
                                         RunTracesLru, replay_lru_workspace_bytes)
from test_gpu_replay_lru import _workload

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
W, G, D = TRACE_WRITE_CACHE, TRACE_GET_LOCATION, TRACE_DIALOG_TURN
POLICY = "leaf_aware_lru"


def _gpu(keys, off, types, quotas, mask=None, ts=None, **kw):
    r = RunTracesLru(torch.as_tensor(np.asarray(keys, dtype=np.int64), device=DEV),
                     torch.as_tensor(np.asarray(off, dtype=np.int64), device=DEV),
                     torch.as_tensor(np.asarray(types, dtype=np.uint8), device=DEV), quotas,
                     torch.as_tensor(np.asarray(mask, dtype=np.int64), device=DEV) if mask is not None else None,
                     policy=POLICY,
                     timestamps=torch.as_tensor(np.asarray(ts, dtype=np.int64), device=DEV) if ts is not None else None,
                     **kw)
    torch.cuda.synchronize()
    ext, inte, wr, size, totals = [t.cpu().numpy() for t in r]
    if ext.shape[1] > 0:
        assert np.array_equal(totals, np.stack([ext.sum(1), inte.sum(1), wr.sum(1), size[:, -1]], axis=1))
    return [ext, inte, wr, size]


def _oracle(q, keys, off, types, mask=None, ts=None, **kw):
    return oracle.LruReplay(q, policy=POLICY, **kw).run(keys, off, types, mask, timestamps=ts)


def _flat(traces):
    keys, off = [], [0]
    for k in traces:
        keys += k
        off.append(len(keys))
    return keys, off


def test_hand_worked_cases():
    # shared prefixes stay: kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:85-133
    keys, off = _flat([[1, 2, 3], [1, 2, 9], [1, 2, 3], [1, 2, 9, 10], [1, 2, 9, 10]])
    ext, inte, wr, size = _gpu(keys, off, [W, W, G, W, G], [3], ts=[0, 1, 2, 3, 4], evict_batch=1, precise=True)
    assert wr[0].tolist() == [3, 1, 0, 1, 0] and size[0].tolist() == [3] * 5 and ext[0].tolist() == [0, 0, 2, 0, 2]
    # a parent that became a data leaf is queued again by access time, ties behind their equals (:135-160)
    keys, off = _flat([[1, 2, 3], [1, 2, 9], [5], [6], [8], [1, 2], [1, 2, 3], [5], [8], [1, 2, 3]])
    ext, inte, wr, size = _gpu(keys, off, [W, W, W, W, W, G, D, G, G, G], [4], ts=list(range(10, 101, 10)),
                               evict_batch=1, precise=True)
    assert wr[0].tolist() == [3, 1, 1, 1, 1, 0, 2, 0, 0, 0]
    assert size[0].tolist() == [3, 4, 4, 4, 4, 4, 4, 4, 4, 4]
    assert ext[0].tolist() == [0, 0, 0, 0, 0, 1, 1, 0, 1, 3]


@pytest.mark.parametrize("rw_separation", [False, True])
@pytest.mark.parametrize("precise", [False, True])
def test_quota_sweep_against_sequential_oracle(rw_separation, precise):
    rng = np.random.default_rng(150 + 2 * rw_separation + precise)
    keys, off, types, mask = _workload(rng, 2500, rw_separation)
    ts = np.cumsum(rng.integers(0, 3, size=len(types)))  # equal timestamps on purpose
    quotas = [1, 7, 33, 100, 257, 1000, 5000, 1 << 40]
    batch = 1 if precise else 13
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = _gpu(keys, off, types, quotas, mask, ts, evict_batch=batch, precise=precise, status=status)
    assert status[0].item() == 0
    differs = 0
    for c, q in enumerate(quotas):
        want = _oracle(q, keys, off, types, mask, ts, evict_batch=batch, precise=precise)
        for name, a, b in zip(("ext", "int", "written", "cached"), want, got):
            assert np.array_equal(a, b[c]), (name, q)
        lru = oracle.LruReplay(q, evict_batch=batch, precise=precise).run(keys, off, types, mask)
        differs += int(not np.array_equal(lru[0], want[0]))
    assert differs >= 3  # the policy is not plain LRU on this workload
    plain = RunTraces(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                      torch.from_numpy(mask).to(DEV))
    for a, b in zip(plain, got):
        assert np.array_equal(a.cpu().numpy(), b[-1])


def test_long_requests_many_configurations_and_workspace_reuse():
    rng = np.random.default_rng(177)
    keys, off, types, mask = _workload(rng, 400, True, max_blocks=300)
    quotas = [int(q) for q in rng.integers(1, 20000, size=160)]
    need = replay_lru_workspace_bytes(len(keys), len(quotas), POLICY, len(types))
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    ws.fill_(0xAB)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for _ in range(2):  # the second call finds the first call's leftovers in the workspace
        got = _gpu(keys, off, types, quotas, mask, evict_batch=100, precise=False, workspace=ws, status=status)
    assert status[0].item() == 0
    for c in rng.choice(len(quotas), size=10, replace=False):
        want = _oracle(quotas[c], keys, off, types, mask, evict_batch=100, precise=False)
        for a, b in zip(want, got):
            assert np.array_equal(a, b[c]), quotas[c]


def test_vector_masks_totals_only_and_empty_inputs():
    rng = np.random.default_rng(192)
    keys, off, types, mask = _workload(rng, 900, True)
    bits = (rng.random(len(keys)) < 0.25).astype(np.uint8)
    quotas = [20, 300, 1 << 40]
    got = _gpu(keys, off, types, quotas, mask, evict_batch=9, mask_bits=torch.from_numpy(bits).to(DEV))
    for c, q in enumerate(quotas):
        want = oracle.LruReplay(q, evict_batch=9, policy=POLICY).run(keys, off, types, mask, mask_bits=bits)
        for a, b in zip(want, got):
            assert np.array_equal(a, b[c]), q
    r = RunTracesLru(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                     quotas, torch.from_numpy(mask).to(DEV), evict_batch=9, per_trace=False, policy=POLICY,
                     mask_bits=torch.from_numpy(bits).to(DEV))
    want = np.stack([got[0].sum(1), got[1].sum(1), got[2].sum(1), got[3][:, -1]], axis=1)
    assert r.external_hit_blocks is None and np.array_equal(r.totals.cpu().numpy(), want)
    ext, inte, wr, size = _gpu([], [0, 0, 0], [W, G], [5])
    assert ext.shape == (1, 2) and size[0].tolist() == [0, 0]
    with pytest.raises(ValueError):
        RunTracesLru(torch.zeros(1, dtype=torch.int64, device=DEV), torch.tensor([0, 1], device=DEV),
                     torch.zeros(1, dtype=torch.uint8, device=DEV), [5], policy="fifo")
