"""Parity of the GPU quota sweep under the "random_lru" eviction policy with the oracle's sequential radix-tree
replay, whose evictions call std::partial_sort the way the reference does
(kv_cache_manager/optimizer/eviction_policy/random_lru.cc:38-82).  The reference has no test of this policy; the
oracle is pinned to records of the reference's own Optimizer (tests/test_optimizer_reference_pins.py), and
tests/test_gpu_optimizer_pins.py replays those records on the GPU."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi
from tair_kvcache_b200.optimizer import (TRACE_DIALOG_TURN, TRACE_GET_LOCATION, TRACE_WRITE_CACHE, RunTracesLru,
                                         replay_lru_workspace_bytes)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
W, G, D = TRACE_WRITE_CACHE, TRACE_GET_LOCATION, TRACE_DIALOG_TURN
POLICY = "random_lru"


def _workload(rng, n_traces, rw_separation, max_blocks=40):
    """Chained keys of token sequences that share prefixes with earlier ones, and timestamps that repeat (several
    traces per microsecond), so that many sampled blocks are equally old."""
    bs = 16
    seqs, keys, off, types, mask, ts = [], [], [0], [], [], []
    now = 1_700_000_000_000_000
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
        now += int(rng.integers(0, 3))
        ts.append(now)
    return (np.concatenate(keys + [np.zeros(0, np.int64)]), np.array(off), np.array(types, np.uint8), np.array(mask),
            np.array(ts, np.int64))


def _gpu(keys, off, types, quotas, mask, ts, **kw):
    r = RunTracesLru(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                     quotas, torch.from_numpy(mask).to(DEV), policy=POLICY,
                     timestamps=torch.from_numpy(ts).to(DEV) if ts is not None else None, **kw)
    torch.cuda.synchronize()
    ext, inte, wr, size, totals = [t.cpu().numpy() for t in r]
    assert np.array_equal(totals, np.stack([ext.sum(1), inte.sum(1), wr.sum(1), size[:, -1]], axis=1))
    return [ext, inte, wr, size]


@pytest.mark.parametrize("rw_separation", [False, True])
@pytest.mark.parametrize("precise,batch,rate", [(False, 13, 0.1), (True, 1, 0.05), (False, 40, 1.0), (True, 25, 0.0)])
def test_quota_sweep_against_sequential_oracle(rw_separation, precise, batch, rate):
    rng = np.random.default_rng(150 + 2 * rw_separation + precise + batch)
    keys, off, types, mask, ts = _workload(rng, 1500, rw_separation)
    quotas = [1, 7, 33, 100, 257, 1000, 5000, 1 << 40]
    got = _gpu(keys, off, types, quotas, mask, ts, evict_batch=batch, precise=precise, sample_rate=rate)
    evicting = 0
    for c, q in enumerate(quotas):
        want = oracle.LruReplay(q, evict_batch=batch, precise=precise, policy=POLICY, sample_rate=rate).run(
            keys, off, types, mask, timestamps=ts)
        for name, a, b in zip(("ext", "int", "written", "cached"), want, got):
            assert np.array_equal(a, b[c]), (name, q)
        evicting += int(q < 5000)
    assert evicting >= 5
    # the policies differ: under the same quota plain LRU keeps other blocks
    lru = oracle.LruReplay(100, evict_batch=batch, precise=precise).run(keys, off, types, mask)
    assert not np.array_equal(lru[0], got[0][3])


@pytest.mark.parametrize("batch,rate", [(32, 0.25), (33, 0.1), (64, 0.5), (100, 0.05), (127, 0.1), (128, 0.25),
                                        (129, 0.1), (300, 0.2)])
def test_batches_around_the_shared_sift_s_limits(batch, rate):
    """Heaps of 32 to 128 samples take the sift that the warp shares (heap-select phase), smaller and larger ones the
    one-lane routines: the same victims either way, with timestamps that repeat (every block of a trace shares one,
    and neighbouring traces do too), so that the order std::partial_sort leaves equal times in decides who goes."""
    rng = np.random.default_rng(900 + batch)
    keys, off, types, mask, ts = _workload(rng, 1200, False, max_blocks=120)
    n_keys = len(np.unique(keys))
    quotas = [batch + 3, n_keys // 20, n_keys // 5, n_keys // 2]
    for precise in (False, True):
        got = _gpu(keys, off, types, quotas, mask, ts, evict_batch=batch, precise=precise, sample_rate=rate)
        for c, q in enumerate(quotas):
            want = oracle.LruReplay(q, evict_batch=batch, precise=precise, policy=POLICY, sample_rate=rate).run(
                keys, off, types, mask, timestamps=ts)
            for name, a, b in zip(("ext", "int", "written", "cached"), want, got):
                assert np.array_equal(a, b[c]), (name, q, precise)
        assert got[2][0].sum() > 20 * batch  # many rounds of evictions at the smallest quota


def test_trace_number_as_time_many_configurations_and_workspace_reuse():
    rng = np.random.default_rng(177)
    keys, off, types, mask, _ = _workload(rng, 300, True, max_blocks=200)
    quotas = [int(q) for q in rng.integers(1, 12000, size=160)]
    ws = torch.empty(replay_lru_workspace_bytes(len(keys), len(quotas), POLICY), dtype=torch.uint8, device=DEV)
    ws.fill_(0xAB)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for _ in range(2):  # the second call finds the first call's leftovers in the workspace
        got = _gpu(keys, off, types, quotas, mask, None, evict_batch=100, precise=False, sample_rate=0.1,
                   workspace=ws, status=status)
    assert status[0].item() == 0
    for c in rng.choice(len(quotas), size=10, replace=False):
        want = oracle.LruReplay(quotas[c], evict_batch=100, precise=False, policy=POLICY, sample_rate=0.1).run(
            keys, off, types, mask)
        for a, b in zip(want, got):
            assert np.array_equal(a, b[c]), quotas[c]


def test_limits_and_empty_input():
    z = torch.zeros(1, dtype=torch.int64, device=DEV)
    off = torch.tensor([0, 1], dtype=torch.int64, device=DEV)
    ty = torch.zeros(1, dtype=torch.uint8, device=DEV)
    with pytest.raises(_cabi.KvcmError) as e:   # 600 blocks per round: more than the kernel's victim table
        RunTracesLru(z, off, ty, [5], evict_batch=600, policy=POLICY, sample_rate=1.0)
    assert e.value.code == _cabi.KVCM_EC_OUT_OF_LIMIT
    with pytest.raises(_cabi.KvcmError) as e:   # 100 / 0.01 = 10,000 samples per round: more than shared memory holds
        RunTracesLru(z, off, ty, [5], evict_batch=100, policy=POLICY, sample_rate=0.01)
    assert e.value.code == _cabi.KVCM_EC_OUT_OF_LIMIT
    r = RunTracesLru(torch.zeros(0, dtype=torch.int64, device=DEV), torch.zeros(3, dtype=torch.int64, device=DEV),
                     torch.tensor([W, G], dtype=torch.uint8, device=DEV), [5], policy=POLICY)
    assert r.current_cache_blocks.cpu().tolist() == [[0, 0]]


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_group_of_sampling_instances_against_the_oracle(mode):
    """Several "random_lru" instances share a quota (OptEvictionManager::EvictByGroupRough / EvictByInstanceRough /
    EvictByInstancePrecise, kv_cache_manager/optimizer/manager/eviction_manager.cc:86-239): every instance keeps its
    own generator and sampling size, and a group-rough round draws in each of them in turn."""
    from tair_kvcache_b200.optimizer import RunTracesLruGroup
    rng = np.random.default_rng(700 + mode)
    keys, off, types, mask, ts = _workload(rng, 1500, True)
    rates = [0.1, 0.5, 0.0, 1.0]
    n_inst = len(rates)
    inst = rng.integers(0, n_inst, size=len(types)).astype(np.int32)
    quotas = [3, 40, 300, 2000, 1 << 40]
    batch = 9
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    r = RunTracesLruGroup(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                          torch.from_numpy(inst).to(DEV), n_inst, quotas, torch.from_numpy(mask).to(DEV),
                          evict_batch=batch, mode=mode, policy=POLICY, sample_rate=rates,
                          timestamps=torch.from_numpy(ts).to(DEV), status=status, instance_records=True)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    got = [t.cpu().numpy() for t in (r[0], r[1], r[2], r[3], r[5], r[6])]
    assert np.array_equal(r.totals.cpu().numpy()[:, 3], got[4].sum(1))
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, n_inst, evict_batch=batch, mode=mode, policy=POLICY, sample_rate=rates).run(
            keys, off, types, inst, mask, timestamps=ts, instance_records=True)
        for name, a, b in zip(("ext", "int", "written", "cached", "final", "every"), want, got):
            assert np.array_equal(a, b[c]), (name, q)


def test_one_sampling_instance_as_a_group_and_refused_arguments():
    from tair_kvcache_b200.optimizer import RunTracesLruGroup
    rng = np.random.default_rng(710)
    keys, off, types, mask, ts = _workload(rng, 600, True)
    quotas = [10, 200]
    zeros = torch.zeros(len(types), dtype=torch.int32, device=DEV)
    args = [torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV)]
    for mode, precise in ((1, False), (2, False), (3, True)):
        one = _gpu(keys, off, types, quotas, mask, ts, evict_batch=7, precise=precise, sample_rate=0.2)
        grp = RunTracesLruGroup(*args, zeros, 1, quotas, torch.from_numpy(mask).to(DEV), evict_batch=7, mode=mode,
                                policy=POLICY, sample_rate=0.2, timestamps=torch.from_numpy(ts).to(DEV))
        for a, b in zip(one, grp[:4]):
            assert np.array_equal(a, b.cpu().numpy())
    with pytest.raises(ValueError):  # a policy the reference's factory does not know
        RunTracesLruGroup(*args, zeros, 2, quotas, policy=["fifo", POLICY])
    with pytest.raises(_cabi.KvcmError) as e:  # the sample of one of the instances would not fit shared memory
        RunTracesLruGroup(*args, zeros, 2, quotas, evict_batch=300, policy=POLICY, sample_rate=[0.5, 0.1])
    assert e.value.code == _cabi.KVCM_EC_OUT_OF_LIMIT
