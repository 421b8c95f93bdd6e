"""Property test of the oracle's Optimizer restatement against the REFERENCE's own Optimizer (compiled in place into
oracle/_ref/libkvcm_ref_optimizer.so; skipped where that library is absent): hypothesis draws small groups of
instances with any mix of the three eviction policies, short traces over a tiny alphabet (so prefixes are shared,
split and re-written all the time), tied timestamps, offset and vector masks, small quotas and batches, all three
eviction modes - and every per-trace record must agree.  A failing example shrinks to a few traces that can be
followed by hand."""
import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings

from oracle import kvcm_oracle as oracle
from oracle import ref_optimizer as ref
from strategies import replay_cases

NAMES = ("external_hit_blocks", "internal_hit_blocks", "write_blocks", "instance_blocks", "blocks_of_every_instance")


def oracle_records(case):
    got = oracle.LruGroupReplay(case["quota"], len(case["policies"]), evict_batch=case["evict_batch"], mode=case["mode"],
                                policy=case["policies"], sample_rate=case["sample_rates"]).run(
        case["keys"], case["key_off"], case["types"], case["instance"], case["mask_off"], case["mask_bits"],
        timestamps=case["timestamps"], instance_records=True)
    return got[0], got[1], got[2], got[3], got[5]


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref/libkvcm_ref_optimizer.so not built (reference tree absent)")
@settings(max_examples=300, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(replay_cases())
def test_oracle_equals_the_compiled_reference(case):
    want = ref.RefOptimizer([dict(quota_capacity=case["quota"],
                                  instances=[(str(j), p, case["sample_rates"][j])
                                             for j, p in enumerate(case["policies"])])],
                            evict_batch=case["evict_batch"], mode=case["mode"]).run(
        case["keys"], case["key_off"], case["types"], case["instance"], case["mask_off"], case["mask_bits"],
        case["timestamps"])
    for name, a, b in zip(NAMES, want, oracle_records(case)):
        assert np.array_equal(a, b), name


@settings(max_examples=100, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(replay_cases(max_instances=1))
def test_single_instance_class_equals_the_group_class(case):
    """LruReplay (what the single-instance GPU sweeps are compared with) is the one-instance group."""
    if case["mode"] == 1:
        case["mode"] = 2
    policy = case["policies"][0]
    kw = dict(sample_rate=case["sample_rates"][0]) if policy == "random_lru" else {}
    got = oracle.LruReplay(case["quota"], evict_batch=case["evict_batch"], precise=case["mode"] == 3, policy=policy,
                           **kw).run(case["keys"], case["key_off"], case["types"],
                                     case["mask_off"] if case["mask_off"] is not None else np.zeros(len(case["types"]), np.int64),
                                     mask_bits=case["mask_bits"], timestamps=case["timestamps"])
    for name, a, b in zip(NAMES[:4], oracle_records(case), got):
        assert np.array_equal(a, b), name
