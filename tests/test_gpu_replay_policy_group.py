"""Groups whose instances mix all three eviction policies - "lru", "leaf_aware_lru" and "random_lru" - under one
quota (kvcm_b200_replay_policy_group), against the oracle's per-instance trees and policy objects.  The reference
makes one policy per instance through EvictionPolicyFactory::CreatePolicy
(kv_cache_manager/optimizer/manager/eviction_manager.cc:21-60) and has no test of a mixed group; what its Optimizer
records for such groups is in tests/golden/optimizer_ref_kat.json (tests/test_gpu_optimizer_pins.py replays it), and
tests/test_optimizer_reference_pins.py compares the oracle with the compiled reference on larger mixed groups."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi
from tair_kvcache_b200.optimizer import RunTracesLruGroup
from test_gpu_replay_random_lru import _workload

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("ext", "int", "written", "cached", "final", "every")


def _gpu(keys, off, types, inst, each, quotas, mask, ts, rates, bits=None, **kw):
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    r = RunTracesLruGroup(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                          torch.from_numpy(inst).to(DEV), len(each), quotas,
                          torch.from_numpy(mask).to(DEV) if mask is not None else None, policy=each, sample_rate=rates,
                          mask_bits=torch.from_numpy(bits).to(DEV) if bits is not None else None,
                          timestamps=torch.from_numpy(ts).to(DEV), status=status, instance_records=True, **kw)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    got = [t.cpu().numpy() for t in (r[0], r[1], r[2], r[3], r[5], r[6])]
    assert np.array_equal(r.totals.cpu().numpy()[:, 3], got[4].sum(1))
    assert np.array_equal(r.totals.cpu().numpy()[:, 2], got[2].sum(1))
    return got


@pytest.mark.parametrize("mode", [1, 2, 3])
@pytest.mark.parametrize("each,rates", [
    (["random_lru", "lru", "leaf_aware_lru"], [0.25, 0.0, 0.0]),
    (["leaf_aware_lru", "random_lru", "random_lru", "lru", "leaf_aware_lru"], [0.0, 0.1, 1.0, 0.0, 0.0])])
def test_mixed_group_against_the_oracle(mode, each, rates):
    rng = np.random.default_rng(900 + 10 * len(each) + mode)
    keys, off, types, mask, ts = _workload(rng, 1800, True)
    inst = rng.integers(0, len(each), size=len(types)).astype(np.int32)
    quotas = [4, 35, 260, 1400, 7000, 1 << 40]
    batch = 8
    got = _gpu(keys, off, types, inst, each, quotas, mask, ts, rates, evict_batch=batch, mode=mode)
    differs = 0
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, len(each), evict_batch=batch, mode=mode, policy=each, sample_rate=rates).run(
            keys, off, types, inst, mask, timestamps=ts, instance_records=True)
        for name, a, b in zip(NAMES, want, got):
            assert np.array_equal(a, b[c]), (name, q)
        plain = oracle.LruGroupReplay(q, len(each), evict_batch=batch, mode=mode,
                                      policy=["lru" if e == "random_lru" else e for e in each]).run(
            keys, off, types, inst, mask, timestamps=ts)
        differs += int(not np.array_equal(plain[0], want[0]))
    assert differs > 0  # the sampling instances do pick other victims than a queue would


def test_dialog_turns_vector_masks_and_an_idle_sampling_instance():
    rng = np.random.default_rng(940)
    each, rates = ["leaf_aware_lru", "random_lru", "random_lru"], [0.0, 0.5, 0.1]
    for rw in (False, True):
        keys, off, types, mask, ts = _workload(rng, 900, rw)
        inst = rng.integers(0, 2, size=len(types)).astype(np.int32)  # the third instance gets no trace
        bits = (rng.random(len(keys)) < 0.2).astype(np.uint8) if rw else None
        quotas = [9, 120, 800]
        got = _gpu(keys, off, types, inst, each, quotas, None if rw else mask, ts, rates, bits, evict_batch=5, mode=1)
        for c, q in enumerate(quotas):
            want = oracle.LruGroupReplay(q, 3, evict_batch=5, mode=1, policy=each, sample_rate=rates).run(
                keys, off, types, inst, None if rw else mask, bits, timestamps=ts, instance_records=True)
            for name, a, b in zip(NAMES, want, got):
                assert np.array_equal(a, b[c]), (rw, name, q)
            assert got[4][c][2] == 0


def test_sampling_instances_alone_take_either_kernel_and_limits_hold():
    """A group of sampling instances goes through the kernel without trees; with one more instance of a queue policy
    that no trace names it goes through the kernel that keeps trees: same records."""
    rng = np.random.default_rng(950)
    keys, off, types, mask, ts = _workload(rng, 1000, True)
    rates = [0.2, 1.0]
    inst = rng.integers(0, 2, size=len(types)).astype(np.int32)
    quotas = [15, 300, 2500]
    for mode in (1, 2, 3):
        alone = _gpu(keys, off, types, inst, ["random_lru"] * 2, quotas, mask, ts, rates, evict_batch=6, mode=mode)
        beside = _gpu(keys, off, types, inst, ["random_lru"] * 2 + ["leaf_aware_lru"], quotas, mask, ts, rates + [0.0],
                      evict_batch=6, mode=mode)
        for name, a, b in zip(NAMES[:4], alone, beside):
            assert np.array_equal(a, b), (mode, name)
        assert np.array_equal(alone[4], beside[4][:, :2]) and np.array_equal(alone[5], beside[5][:, :, :2])
    lib = _cabi.lib()
    two = (ctypes.c_uint8 * 2)(_cabi.POLICY_LEAF_AWARE_LRU, _cabi.POLICY_RANDOM_LRU)
    plain = (ctypes.c_uint8 * 2)(_cabi.POLICY_LEAF_AWARE_LRU, _cabi.POLICY_LRU)
    cast = lambda a: ctypes.cast(a, ctypes.c_void_p)
    # the block vectors are added to the workspace only when a sampling instance is present
    assert lib.kvcm_b200_replay_policy_group_workspace_bytes(1000, 10, 4, cast(two), 2) > \
        lib.kvcm_b200_replay_policy_group_workspace_bytes(1000, 10, 4, cast(plain), 2) == \
        lib.kvcm_b200_replay_leaf_lru_group_workspace_bytes(1000, 10, 4, 2)
    bad = (ctypes.c_uint8 * 2)(0, 3)
    assert lib.kvcm_b200_replay_policy_group_workspace_bytes(1000, 10, 4, cast(bad), 2) == -1
    args = [torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
            torch.from_numpy(inst).to(DEV)]
    with pytest.raises(_cabi.KvcmError) as e:  # the sample of the sampling instance would not fit shared memory
        RunTracesLruGroup(*args, 2, quotas, evict_batch=300, policy=["lru", "random_lru"], sample_rate=[0.0, 0.1])
    assert e.value.code == _cabi.KVCM_EC_OUT_OF_LIMIT
    # the same batch size is fine for the queue policies alone
    RunTracesLruGroup(*args, 2, quotas, evict_batch=300, policy=["lru", "leaf_aware_lru"])
    torch.cuda.synchronize()


def test_sixty_four_instances_and_the_call_without_an_instance_array():
    rng = np.random.default_rng(960)
    keys, off, types, mask, ts = _workload(rng, 1500, True)
    each = [("random_lru", "lru", "leaf_aware_lru")[j % 3] for j in range(64)]   # the most one group may hold
    rates = [0.5] * 64
    inst = rng.integers(0, 64, size=len(types)).astype(np.int32)
    quotas = [50, 900]
    got = _gpu(keys, off, types, inst, each, quotas, mask, ts, rates, evict_batch=4, mode=1)
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, 64, evict_batch=4, mode=1, policy=each, sample_rate=rates).run(
            keys, off, types, inst, mask, timestamps=ts, instance_records=True)
        for name, a, b in zip(NAMES, want, got):
            assert np.array_equal(a, b[c]), (name, q)
    with pytest.raises(ValueError):
        RunTracesLruGroup(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                          torch.from_numpy(inst).to(DEV), 65, quotas, policy=["lru"] * 64 + ["random_lru"])
    # one sampling instance through the group entry, no instance array: the single-instance sweep
    from tair_kvcache_b200.optimizer import RunTracesLru
    one = RunTracesLru(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                       quotas, torch.from_numpy(mask).to(DEV), evict_batch=5, precise=True, policy="random_lru",
                       sample_rate=0.25, timestamps=torch.from_numpy(ts).to(DEV))
    lib = _cabi.lib()
    policy = (ctypes.c_uint8 * 1)(_cabi.POLICY_RANDOM_LRU)
    rate = (ctypes.c_double * 1)(0.25)
    cast = lambda a: ctypes.cast(a, ctypes.c_void_p)
    n_tr = len(types)
    need = lib.kvcm_b200_replay_policy_group_workspace_bytes(len(keys), n_tr, 2, cast(policy), 1)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    dq = torch.tensor(quotas, dtype=torch.int64, device=DEV)
    outs = [torch.empty((2, n_tr), dtype=torch.int32, device=DEV) for _ in range(3)]
    size = torch.empty((2, n_tr), dtype=torch.int64, device=DEV)
    totals = torch.zeros((2, 4), dtype=torch.int64, device=DEV)
    dk, do, dt, dm, dts = (torch.from_numpy(a).to(DEV) for a in (keys, off, types, mask, ts))
    _cabi.call("kvcm_b200_replay_policy_group", dk.data_ptr(), do.data_ptr(), dt.data_ptr(), dm.data_ptr(), None,
               dts.data_ptr(), None, cast(policy), cast(rate), 1, n_tr, len(keys), dq.data_ptr(), 2, 5, 3,
               ws.data_ptr(), need, outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), size.data_ptr(),
               totals.data_ptr(), None, None, None, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for a, b in zip(one[:4], outs + [size]):
        assert np.array_equal(a.cpu().numpy(), b.cpu().numpy())
