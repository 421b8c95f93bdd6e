"""Parity of the GPU "leaf_aware_lru" sweep for instance groups that share one quota with the oracle's per-instance
radix trees and leaf-aware queues.  The reference has no test of this policy; the known answer below is worked out by
hand from the cited source lines (and repeated for the oracle alone in tests/test_oracle.py)."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import (TRACE_GET_LOCATION, TRACE_WRITE_CACHE, RunTracesLru, RunTracesLruGroup)
from test_gpu_replay_lru import _workload

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
W, G = TRACE_WRITE_CACHE, TRACE_GET_LOCATION
POLICY = "leaf_aware_lru"


def _gpu(keys, off, types, inst, n_inst, quotas, mask=None, ts=None, **kw):
    r = RunTracesLruGroup(torch.as_tensor(np.asarray(keys, dtype=np.int64), device=DEV),
                          torch.as_tensor(np.asarray(off, dtype=np.int64), device=DEV),
                          torch.as_tensor(np.asarray(types, dtype=np.uint8), device=DEV),
                          torch.as_tensor(np.asarray(inst, dtype=np.int32), device=DEV), n_inst, quotas,
                          torch.as_tensor(np.asarray(mask, dtype=np.int64), device=DEV) if mask is not None else None,
                          policy=POLICY,
                          timestamps=torch.as_tensor(np.asarray(ts, dtype=np.int64), device=DEV) if ts is not None else None,
                          **kw)
    torch.cuda.synchronize()
    ext, inte, wr, size, totals, final = [t.cpu().numpy() for t in r[:6]]
    if ext.shape[1] > 0:
        assert np.array_equal(totals[:, :3], np.stack([ext.sum(1), inte.sum(1), wr.sum(1)], axis=1))
        assert np.array_equal(totals[:, 3], final.sum(1))
    out = [ext, inte, wr, size, final]
    if r.instance_blocks_per_trace is not None:
        out.append(r.instance_blocks_per_trace.cpu().numpy())
    return out


HAND_TRACES = [[1, 2, 3], [1, 2, 9], [1, 2], [1, 2, 3], [1, 2], [5], [7, 8], [1, 2, 9], [6]]
HAND_INST = [0, 0, 1, 0, 1, 0, 1, 0, 0]
HAND_TYPES = [W, W, W, G, G, W, W, G, W]


def test_two_instances_by_hand():
    # kv_cache_manager/optimizer/manager/eviction_manager.cc:86-146 over LeafAwareLruEvictionPolicy::EvictBlocks
    # (kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:85-160), quota 5, batches of 1, group rough.
    #   a writes 1 2 3, then 1 2 9 (a split: {1 2} over {3} and {9}); b writes 1 2: the group holds 6.
    #   The round asks a first: 1 and 2 sit in a node with cached children and only leave the queue, 3 goes;
    #   then b, whose {1 2} is a leaf: 1 goes.  a reads 1 2 3 -> 2 hits; b reads 1 2 -> none.
    #   a writes 5, b writes 7 8 (7 held).  a loses 9, which turns {1 2} into a data leaf: both are queued again,
    #   at the cold end behind 5 (their time, 3, is the oldest), 1 before 2; b loses 2.
    #   a reads 1 2 9 -> 2 hits and both move to the front, so a's next victim is 5; b's is 7.
    keys = [k for t in HAND_TRACES for k in t]
    off = np.cumsum([0] + [len(t) for t in HAND_TRACES])
    ext, inte, wr, size, final = _gpu(keys, off, HAND_TYPES, HAND_INST, 2, [5], ts=list(range(9)), evict_batch=1, mode=1)
    assert ext[0].tolist() == [0, 0, 0, 2, 0, 0, 0, 2, 0]
    assert wr[0].tolist() == [3, 1, 2, 0, 0, 1, 2, 0, 1]
    assert size[0].tolist() == [3, 4, 1, 3, 1, 4, 2, 3, 3] and final[0].tolist() == [3, 1]
    # from the writing instance only, b pays for its own writes and a keeps 3
    for mode in (2, 3):
        ext, inte, wr, size, final = _gpu(keys, off, HAND_TYPES, HAND_INST, 2, [5], ts=list(range(9)), evict_batch=1,
                                          mode=mode)
        assert ext[0].tolist() == [0, 0, 0, 3, 0, 0, 0, 2, 0] and final[0].tolist() == [4, 1]


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_group_sweep_against_the_oracle(mode):
    rng = np.random.default_rng(400 + mode)
    keys, off, types, mask = _workload(rng, 2000, True)
    ts = np.cumsum(rng.integers(0, 3, size=len(types)))  # equal timestamps on purpose
    n_inst = 4
    inst = rng.integers(0, n_inst, size=len(types)).astype(np.int32)
    quotas = [1, 9, 60, 250, 1200, 6000, 1 << 40]
    batch = 7
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = _gpu(keys, off, types, inst, n_inst, quotas, mask, ts, evict_batch=batch, mode=mode, status=status,
               instance_records=True)
    assert status[0].item() == 0
    differs = 0
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, n_inst, evict_batch=batch, mode=mode, policy=POLICY).run(
            keys, off, types, inst, mask, timestamps=ts, instance_records=True)
        for name, a, b in zip(("ext", "int", "written", "cached", "final", "every"), want, got):
            assert np.array_equal(a, b[c]), (name, q)
        lru = oracle.LruGroupReplay(q, n_inst, evict_batch=batch, mode=mode).run(keys, off, types, inst, mask)
        differs += int(not np.array_equal(lru[0], want[0]))
    assert differs >= 2  # the policy is not plain LRU on this workload


def test_one_instance_group_is_the_single_instance_sweep_and_bad_instances_are_counted():
    rng = np.random.default_rng(410)
    keys, off, types, mask = _workload(rng, 700, True)
    ts = np.cumsum(rng.integers(0, 2, size=len(types)))
    quotas = [15, 400]
    zeros = np.zeros(len(types), dtype=np.int32)
    for mode, precise in ((1, False), (2, False), (3, True)):
        got = _gpu(keys, off, types, zeros, 1, quotas, mask, ts, evict_batch=11, mode=mode)
        r = RunTracesLru(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV),
                         torch.from_numpy(types).to(DEV), quotas, torch.from_numpy(mask).to(DEV), evict_batch=11,
                         precise=precise, policy=POLICY, timestamps=torch.from_numpy(ts).to(DEV))
        for a, b in zip(r[:4], got):
            assert np.array_equal(a.cpu().numpy(), b)
    # a trace that names no instance of the group is counted and replayed as an empty trace
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    bad = zeros.copy()
    bad[3] = 7
    got = _gpu(keys, off, types, bad, 2, quotas, mask, ts, evict_batch=11, status=status)
    assert status[0].item() == 1
    keep = np.ones(len(types), dtype=bool)
    keep[3] = False
    lens = np.diff(off)
    off2 = np.concatenate([[0], np.cumsum(np.where(keep, lens, 0))])
    keys2 = np.concatenate([keys[off[t]:off[t + 1]] for t in range(len(types)) if keep[t]])
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, 2, evict_batch=11, mode=1, policy=POLICY).run(keys2, off2, types, zeros, mask,
                                                                                      timestamps=ts)
        for a, b in zip(want, got):
            assert np.array_equal(a, b[c]), q
    with pytest.raises(ValueError):
        _gpu(keys, off, types, zeros, 65, quotas, mask)
    with pytest.raises(ValueError):
        RunTracesLruGroup(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                          torch.from_numpy(zeros).to(DEV), 1, quotas, policy="fifo")


def test_deep_shared_prefixes_requeue_whole_nodes():
    """Few long stems with many short branches: evicting the branches keeps turning long parents into data leaves,
    whose blocks - written by one trace, so one time - go back into the queue as one piece."""
    rng = np.random.default_rng(421)
    stems = [rng.integers(0, 50000, size=16 * int(rng.integers(40, 120))).astype(np.int64) for _ in range(12)]
    traces, types = [], []
    for _ in range(1500):
        s = stems[int(rng.integers(len(stems)))]
        cut = 16 * int(rng.integers(1, len(s) // 16 + 1))
        tail = rng.integers(0, 50000, size=16 * int(rng.integers(0, 6))).astype(np.int64)
        traces.append(oracle.gen_key_vector(np.concatenate([s[:cut], tail]), 16))
        types.append(G if rng.random() < 0.3 else W)
    keys = np.concatenate(traces)
    off = np.concatenate([[0], np.cumsum([len(t) for t in traces])]).astype(np.int64)
    types = np.asarray(types, dtype=np.uint8)
    n_inst = 3
    inst = rng.integers(0, n_inst, size=len(types)).astype(np.int32)
    ts = np.cumsum(rng.integers(0, 2, size=len(types)))
    quotas = [30, 200, 700, 1500, 4000]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for mode, batch in ((1, 5), (3, 40)):
        got = _gpu(keys, off, types, inst, n_inst, quotas, None, ts, evict_batch=batch, mode=mode, status=status)
        assert status[0].item() == 0
        for c, q in enumerate(quotas):
            want = oracle.LruGroupReplay(q, n_inst, evict_batch=batch, mode=mode, policy=POLICY).run(
                keys, off, types, inst, timestamps=ts)
            for name, a, b in zip(("ext", "int", "written", "cached", "final"), want, got):
                assert np.array_equal(a, b[c]), (name, q, mode)
    # one instance, through the single-instance entry point
    for c, q in enumerate(quotas):
        r = RunTracesLru(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                         [q], evict_batch=9, policy=POLICY, timestamps=torch.from_numpy(ts).to(DEV), status=status)
        want = oracle.LruReplay(q, evict_batch=9, policy=POLICY).run(keys, off, types, timestamps=ts)
        for a, b in zip(want, r[:4]):
            assert np.array_equal(a, b.cpu().numpy()[0]), q
    assert status[0].item() == 0


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_a_group_that_mixes_lru_and_leaf_aware_instances(mode):
    """EvictionPolicyFactory::CreatePolicy runs per instance (kv_cache_manager/optimizer/manager/
    eviction_manager.cc:22-55), so one group may hold instances of different policies; the reference tests none."""
    rng = np.random.default_rng(430 + mode)
    keys, off, types, mask = _workload(rng, 1800, True)
    ts = np.cumsum(rng.integers(0, 3, size=len(types)))
    each = ["lru", POLICY, "lru", POLICY, POLICY]
    inst = rng.integers(0, len(each), size=len(types)).astype(np.int32)
    quotas = [5, 40, 300, 1500, 1 << 40]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    r = RunTracesLruGroup(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                          torch.from_numpy(inst).to(DEV), len(each), quotas, torch.from_numpy(mask).to(DEV), evict_batch=6,
                          mode=mode, policy=each, timestamps=torch.from_numpy(ts).to(DEV), status=status,
                          instance_records=True)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    got = [t.cpu().numpy() for t in (r[0], r[1], r[2], r[3], r[5], r[6])]
    same_as_all_leaf = 0
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, len(each), evict_batch=6, mode=mode, policy=each).run(
            keys, off, types, inst, mask, timestamps=ts, instance_records=True)
        for name, a, b in zip(("ext", "int", "written", "cached", "final", "every"), want, got):
            assert np.array_equal(a, b[c]), (name, q)
        leaf = oracle.LruGroupReplay(q, len(each), evict_batch=6, mode=mode, policy=POLICY).run(
            keys, off, types, inst, mask, timestamps=ts)
        same_as_all_leaf += int(np.array_equal(leaf[0], want[0]))
    assert same_as_all_leaf < len(quotas)  # the "lru" instances do behave differently


def test_lru_instances_in_the_tree_kernel_equal_the_lru_group_sweep():
    rng = np.random.default_rng(440)
    keys, off, types, mask = _workload(rng, 1200, True)
    n_inst = 3
    inst = rng.integers(0, n_inst, size=len(types)).astype(np.int32)
    quotas = [12, 150, 900]
    args = [torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
            torch.from_numpy(inst).to(DEV)]
    for mode in (1, 3):
        plain = RunTracesLruGroup(*args, n_inst, quotas, torch.from_numpy(mask).to(DEV), evict_batch=5, mode=mode)
        # one more instance, leaf-aware and without a trace, sends the same group through the kernel that keeps trees
        tree = RunTracesLruGroup(*args, n_inst + 1, quotas, torch.from_numpy(mask).to(DEV), evict_batch=5, mode=mode,
                                 policy=["lru"] * n_inst + [POLICY])
        for a, b in zip(plain[:5], tree[:5]):
            assert np.array_equal(a.cpu().numpy(), b.cpu().numpy())
        assert np.array_equal(plain.instance_blocks.cpu().numpy(), tree.instance_blocks.cpu().numpy()[:, :n_inst])
    with pytest.raises(ValueError):
        RunTracesLruGroup(*args, n_inst, quotas, policy=["lru", "lru"])
