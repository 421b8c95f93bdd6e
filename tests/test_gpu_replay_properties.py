"""Property tests of the eviction-aware replay kernels against the oracle (which tests/test_optimizer_properties.py
holds against the reference's own Optimizer with the same strategy): hypothesis draws small instance groups with any
mix of the three policies, short traces over a tiny alphabet - prefixes shared, split, evicted and re-written all the
time - tied timestamps, offset and vector masks, small quotas and batches, the three eviction modes.  Several quota
points go through one launch, so the warps of one launch must not disturb each other either."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings

from oracle import kvcm_oracle as oracle
from strategies import replay_cases

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import RunTracesLru, RunTracesLruGroup

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("external_hit_blocks", "internal_hit_blocks", "write_blocks", "instance_blocks", "blocks_of_every_instance")


def _dev(a):
    return torch.from_numpy(a).to(DEV) if a is not None else None


def _group_parity(case):
    quotas = [case["quota"], case["quota"] + 6, 1 << 40]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    k = len(case["policies"])
    r = RunTracesLruGroup(_dev(case["keys"]), _dev(case["key_off"]), _dev(case["types"]), _dev(case["instance"]), k,
                          quotas, _dev(case["mask_off"]), evict_batch=case["evict_batch"], mode=case["mode"],
                          status=status, mask_bits=_dev(case["mask_bits"]), instance_records=True,
                          policy=case["policies"], timestamps=_dev(case["timestamps"]),
                          sample_rate=case["sample_rates"])
    torch.cuda.synchronize()
    assert status[0].item() == 0
    got = [t.cpu().numpy() for t in (r[0], r[1], r[2], r[3], r[6])]
    final = r.instance_blocks.cpu().numpy()
    for c, q in enumerate(quotas):
        want = oracle.LruGroupReplay(q, k, evict_batch=case["evict_batch"], mode=case["mode"], policy=case["policies"],
                                     sample_rate=case["sample_rates"]).run(
            case["keys"], case["key_off"], case["types"], case["instance"], case["mask_off"], case["mask_bits"],
            timestamps=case["timestamps"], instance_records=True)
        for name, a, b in zip(NAMES, (want[0], want[1], want[2], want[3], want[5]), got):
            assert np.array_equal(a, b[c]), (name, q)
        assert np.array_equal(want[4], final[c])


@settings(max_examples=250, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(replay_cases())
def test_groups_of_any_mix_of_policies(case):
    _group_parity(case)


@settings(max_examples=120, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(replay_cases(policies=("leaf_aware_lru", "lru"), max_traces=40, max_blocks=9))
def test_tree_kernel_on_longer_traces(case):
    _group_parity(case)


@settings(max_examples=150, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(replay_cases(max_instances=1, max_traces=30))
def test_single_instance_sweeps(case):
    policy = case["policies"][0]
    precise = case["mode"] == 3
    quotas = [case["quota"], case["quota"] + 4]
    kw = dict(sample_rate=case["sample_rates"][0]) if policy == "random_lru" else {}
    mask = case["mask_off"] if case["mask_off"] is not None else np.zeros(len(case["types"]), np.int64)
    r = RunTracesLru(_dev(case["keys"]), _dev(case["key_off"]), _dev(case["types"]), quotas, _dev(mask),
                     evict_batch=case["evict_batch"], precise=precise, mask_bits=_dev(case["mask_bits"]), policy=policy,
                     timestamps=_dev(case["timestamps"]), **kw)
    torch.cuda.synchronize()
    for c, q in enumerate(quotas):
        want = oracle.LruReplay(q, evict_batch=case["evict_batch"], precise=precise, policy=policy, **kw).run(
            case["keys"], case["key_off"], case["types"], mask, mask_bits=case["mask_bits"],
            timestamps=case["timestamps"])
        for name, a, b in zip(NAMES, want, r[:4]):
            assert np.array_equal(a, b.cpu().numpy()[c]), (policy, name, q)


@settings(max_examples=150, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(replay_cases())
def test_groups_against_the_compiled_reference_itself(case):
    """The same draws against the reference's own Optimizer (compiled from its sources, where that library has
    travelled with the build), with no oracle in between."""
    from oracle import ref_optimizer as ref
    if not ref.available():
        pytest.skip("oracle/_ref/libkvcm_ref_optimizer.so not built")
    k = len(case["policies"])
    want = ref.RefOptimizer([dict(quota_capacity=case["quota"],
                                  instances=[(str(j), p, case["sample_rates"][j])
                                             for j, p in enumerate(case["policies"])])],
                            evict_batch=case["evict_batch"], mode=case["mode"]).run(
        case["keys"], case["key_off"], case["types"], case["instance"], case["mask_off"], case["mask_bits"],
        case["timestamps"])
    r = RunTracesLruGroup(_dev(case["keys"]), _dev(case["key_off"]), _dev(case["types"]), _dev(case["instance"]), k,
                          [case["quota"]], _dev(case["mask_off"]), evict_batch=case["evict_batch"], mode=case["mode"],
                          mask_bits=_dev(case["mask_bits"]), instance_records=True, policy=case["policies"],
                          timestamps=_dev(case["timestamps"]), sample_rate=case["sample_rates"])
    torch.cuda.synchronize()
    for name, a, b in zip(NAMES, want, (r[0], r[1], r[2], r[3], r[6])):
        assert np.array_equal(a, b.cpu().numpy()[0]), name
