"""Parity of the GPU LRU sweep for instance groups that share one quota with the oracle's per-instance radix trees."""
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


def _gpu(keys, off, types, inst, n_inst, quotas, mask=None, **kw):
    r = RunTracesLruGroup(torch.as_tensor(np.asarray(keys, dtype=np.int64), device=DEV),
                          torch.as_tensor(np.asarray(off, dtype=np.int64), device=DEV),
                          torch.as_tensor(np.asarray(types, dtype=np.uint8), device=DEV),
                          torch.as_tensor(np.asarray(inst, dtype=np.int32), device=DEV), n_inst, quotas,
                          torch.as_tensor(np.asarray(mask, dtype=np.int64), device=DEV) if mask is not None else None,
                          **kw)
    torch.cuda.synchronize()
    ext, inte, wr, size, totals, final = [t.cpu().numpy() for t in r[:6]]
    if r.instance_blocks_per_trace is not None:
        every = r.instance_blocks_per_trace.cpu().numpy()
        assert every.shape == (len(quotas), ext.shape[1], n_inst)
        if ext.shape[1] > 0:  # the trace's own instance is one of them, and the last record is the final usage
            own = np.take_along_axis(every, np.asarray(inst, dtype=np.int64)[None, :, None].repeat(len(quotas), 0), 2)
            assert np.array_equal(own[:, :, 0], size) and np.array_equal(every[:, -1, :], final)
    if ext.shape[1] > 0:
        assert np.array_equal(totals[:, :3], np.stack([ext.sum(1), inte.sum(1), wr.sum(1)], axis=1))
        assert np.array_equal(totals[:, 3], final.sum(1))
    return [ext, inte, wr, size, final]


def test_two_instances_share_a_quota_by_hand():
    # kv_cache_manager/optimizer/manager/eviction_manager.cc:86-146 by hand: the instances a and b write the same
    # keys (separate trees: nothing is shared), quota 4, batches of 1.
    #   a writes 1 2 3 (a: 3), b writes 1 2 (b: 2; the group holds 5, one over)
    #   GROUP_ROUGH: one round takes a block from a (key 1) AND from b (key 1) -> a: 2, b: 1
    #   INSTANCE modes: only the writer b loses a block (key 1) -> a: 3, b: 1
    keys, off, types, inst = [1, 2, 3, 1, 2, 1, 2, 3, 1, 2], [0, 3, 5, 8, 10], [W, W, G, G], [0, 1, 0, 1]
    ext, inte, wr, size, final = _gpu(keys, off, types, inst, 2, [4], evict_batch=1, mode=1)
    assert wr[0].tolist() == [3, 2, 0, 0] and size[0].tolist() == [3, 1, 2, 1] and final[0].tolist() == [2, 1]
    assert ext[0].tolist() == [0, 0, 0, 0]  # both lost key 1, the head of their chains
    for mode in (2, 3):
        ext, inte, wr, size, final = _gpu(keys, off, types, inst, 2, [4], evict_batch=1, mode=mode)
        assert size[0].tolist() == [3, 1, 3, 1] and final[0].tolist() == [3, 1] and ext[0].tolist() == [0, 0, 3, 0]


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_group_sweep_against_the_oracle(mode):
    rng = np.random.default_rng(300 + mode)
    keys, off, types, mask = _workload(rng, 2000, True)
    n_inst = 5
    inst = rng.integers(0, n_inst, size=len(types)).astype(np.int32)
    quotas = [1, 9, 60, 250, 1200, 6000, 1 << 40]
    batch = 7
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = _gpu(keys, off, types, inst, n_inst, quotas, mask, evict_batch=batch, mode=mode, status=status)
    assert status[0].item() == 0
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, n_inst, evict_batch=batch, mode=mode).run(keys, off, types, inst, mask)
        for name, a, b in zip(("ext", "int", "written", "cached", "final"), want, got):
            assert np.array_equal(a, b[c]), (name, q)
    # the instances do not share blocks: the same traces in one instance hit more
    one = RunTracesLru(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                       [1 << 40], torch.from_numpy(mask).to(DEV))
    assert int(one.totals[0, 0]) > int(got[0][-1].sum())


def test_one_instance_group_is_the_plain_sweep_and_bad_instances_are_counted():
    rng = np.random.default_rng(310)
    keys, off, types, mask = _workload(rng, 700, True)
    quotas = [15, 400]
    zeros = np.zeros(len(types), dtype=np.int32)
    for mode, precise in ((1, False), (2, False), (3, True)):
        got = _gpu(keys, off, types, zeros, 1, quotas, mask, evict_batch=11, mode=mode)
        r = RunTracesLru(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV),
                         torch.from_numpy(types).to(DEV), quotas, torch.from_numpy(mask).to(DEV), evict_batch=11,
                         precise=precise)
        for a, b in zip(r[:4], got):
            assert np.array_equal(a.cpu().numpy(), b)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    bad = zeros.copy()
    bad[3] = 7
    _gpu(keys, off, types, bad, 2, quotas, mask, status=status)
    assert status[0].item() == 1
    with pytest.raises(ValueError):
        _gpu(keys, off, types, zeros, 65, quotas, mask)


@pytest.mark.parametrize("mode", [1, 3])
def test_usage_of_every_instance_after_each_trace(mode):
    """ReadRecord::blocks_per_instance (kv_cache_manager/optimizer/manager/optimizer_runner.cc:116-124): under
    group-rough eviction a write of one instance shrinks the others too, so the column cannot be derived from the
    per-trace usage of the trace's own instance."""
    rng = np.random.default_rng(330 + mode)
    keys, off, types, mask = _workload(rng, 900, True)
    n_inst = 4
    inst = rng.integers(0, n_inst, size=len(types)).astype(np.int32)
    quotas = [40, 300, 1 << 40]
    r = RunTracesLruGroup(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                          torch.from_numpy(inst).to(DEV), n_inst, quotas, torch.from_numpy(mask).to(DEV), evict_batch=5,
                          mode=mode, instance_records=True)
    got = r.instance_blocks_per_trace.cpu().numpy()
    changed_others = 0
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, n_inst, evict_batch=5, mode=mode).run(keys, off, types, inst, mask,
                                                                              instance_records=True)
        assert np.array_equal(want[5], got[c]), q
        d = np.diff(want[5], axis=0)
        others = d.copy()
        others[np.arange(len(d)), inst[1:]] = 0
        changed_others += int((others != 0).sum())
    assert (changed_others > 0) == (mode == 1)
    _gpu(keys, off, types, inst, n_inst, quotas, mask, evict_batch=5, mode=mode, instance_records=True)
