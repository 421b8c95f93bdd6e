"""The CUDA replay kernels and the trace runner against what the REFERENCE's own Optimizer recorded.

The fixtures (tests/golden/optimizer_ref_kat.json, optimizer_ref_csv.json) were written by
tests/golden/make_optimizer_golden.py from the reference's optimizer sources compiled in place; tests/
test_optimizer_reference_pins.py replays them against the oracle on any box, this file against the GPU: every
eviction policy alone and in groups of instances, the three eviction modes, offset and vector masks, a hierarchical
group - and the three trace-file formats end to end, down to the bytes of the hit-rate CSV files."""
import json

import numpy as np
import pytest
import torch

from conftest import load_golden
from test_optimizer_reference_pins import NAMES, compare_with_reference_files

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import RunTracesLru, RunTracesLruGroup, runner

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev(a, dtype):
    return torch.as_tensor(np.asarray(a, dtype=dtype), device=DEV)


def test_group_kernels_replay_what_the_reference_recorded():
    cases = load_golden("optimizer_ref_kat.json")["cases"]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for case in cases:
        quotas = [run["quota"] for run in case["runs"]]
        policies = case["policies"]
        r = RunTracesLruGroup(
            _dev(case["keys"], np.int64), _dev(case["key_off"], np.int64), _dev(case["types"], np.uint8),
            _dev(case["instance"], np.int32), len(policies), quotas,
            _dev(case["mask_off"], np.int64) if case["mask_off"] is not None else None,
            evict_batch=case["evict_batch"], mode=case["mode"], status=status,
            mask_bits=_dev(case["mask_bits"], np.uint8) if case["mask_bits"] is not None else None,
            instance_records=True, policy=policies if len(set(policies)) > 1 else policies[0],
            timestamps=_dev(case["timestamps"], np.int64), sample_rate=case["sample_rates"])
        torch.cuda.synchronize()
        got = [t.cpu().numpy() for t in (r[0], r[1], r[2], r[3], r[6])]
        for c, run in enumerate(case["runs"]):
            for name, g in zip(NAMES, got):
                assert np.array_equal(np.asarray(run[name]), g[c]), (case["name"], run["quota"], name)
    assert status[0].item() == 0


def test_single_instance_kernels_replay_what_the_reference_recorded():
    n = 0
    for case in load_golden("optimizer_ref_kat.json")["cases"]:
        if len(case["policies"]) != 1 or case["mode"] == 1:
            continue
        quotas = [run["quota"] for run in case["runs"]]
        r = RunTracesLru(
            _dev(case["keys"], np.int64), _dev(case["key_off"], np.int64), _dev(case["types"], np.uint8), quotas,
            _dev(case["mask_off"], np.int64) if case["mask_off"] is not None else None,
            evict_batch=case["evict_batch"], precise=case["mode"] == 3,
            mask_bits=_dev(case["mask_bits"], np.uint8) if case["mask_bits"] is not None else None,
            policy=case["policies"][0], timestamps=_dev(case["timestamps"], np.int64),
            sample_rate=case["sample_rates"][0])
        torch.cuda.synchronize()
        for c, run in enumerate(case["runs"]):
            for name, g in zip(NAMES, r[:4]):
                assert np.array_equal(np.asarray(run[name]), g.cpu().numpy()[c]), (case["name"], run["quota"], name)
        n += 1
    assert n >= 12


def test_trace_files_give_the_reference_csv_files(tmp_path):
    for n, case in enumerate(load_golden("optimizer_ref_csv.json")["cases"]):
        work = tmp_path / ("case%d" % n)
        work.mkdir()
        (work / "trace.jsonl").write_text(case["trace_text"])
        config = json.loads(json.dumps(case["config"]))
        config["trace_file_path"] = str(work / "trace.jsonl")
        config["output_result_path"] = str(work / "out")
        runner.run_startup_config(config, device=DEV)
        compare_with_reference_files(case, str(work / "out"))


@pytest.mark.parametrize("trace_type", ["optimizer_schema", "qwen_bailian", "publisher_log"])
def test_larger_trace_files_against_the_compiled_reference(tmp_path, trace_type):
    """Where the reference's Optimizer is present as a built library (it travels with the other built files), a
    few thousand traces per format go through its optimizer_main path and through the GPU runner: same CSV files."""
    from oracle import ref_optimizer as ref
    if not ref.available():
        pytest.skip("oracle/_ref/libkvcm_ref_optimizer.so not built")
    from golden.make_optimizer_golden import trace_files
    rng = np.random.default_rng(0xB2000009)
    text = trace_files(rng, scale=40)[trace_type]
    (tmp_path / "trace.jsonl").write_text(text)
    plans = {"optimizer_schema": ([[("inst_a", "leaf_aware_lru"), ("idle", "lru")], [("inst_b", "random_lru")]], 1, 300),
             "qwen_bailian": ([[("instance", "leaf_aware_lru")]], 2, 400),
             "publisher_log": ([[("inst_a", "lru"), ("inst_b", "leaf_aware_lru")]], 1, 500)}
    groups, mode, quota = plans[trace_type]
    files = {}
    for who in ("reference", "gpu"):
        out = tmp_path / who
        out.mkdir()
        config = ref.startup_config([dict(quota_capacity=quota, instances=[(i, p, 0.1) for i, p in members])
                                     for members in groups], evict_batch=16, mode=mode,
                                    trace_file_path=str(tmp_path / "trace.jsonl"), trace_type=trace_type,
                                    output_result_path=str(out))
        if who == "reference":
            ref.optimizer_main(config)
        else:
            runner.run_startup_config(config, device=DEV)
        files[who] = {p.name: p.read_text() for p in sorted(out.iterdir())}
    assert sum(len(t.splitlines()) for t in files["reference"].values()) > 1500
    compare_with_reference_files(dict(trace_type=trace_type, files=files["reference"]), str(tmp_path / "gpu"))


def test_large_eviction_batches_against_the_compiled_reference():
    """Batches of 32 to 128 blocks per round (the fixtures above use up to 8): the sizes at which the sampling
    policy's heap-select runs its warp-shared sift, in groups of up to three instances that mix the policies."""
    from oracle import ref_optimizer as ref
    if not ref.available():
        pytest.skip("oracle/_ref/libkvcm_ref_optimizer.so not built")
    from test_gpu_replay_random_lru import _workload
    compared = 0
    for seed in range(8):
        rng = np.random.default_rng(5000 + seed)
        keys, off, types, mask, ts = _workload(rng, 700, bool(seed % 2), max_blocks=100)
        k = int(rng.integers(1, 4))
        policies = ["random_lru"] + [str(rng.choice(["random_lru", "lru", "leaf_aware_lru"])) for _ in range(k - 1)]
        inst = rng.integers(0, k, size=len(types)).astype(np.int32)
        batch = int(rng.choice([32, 48, 64, 100, 128]))
        rates = [float(x) for x in rng.choice([0.1, 0.25, 0.5], size=k)]
        mode = int(rng.integers(1, 4))
        n_keys = len(np.unique(keys))
        quotas = [batch + 5, n_keys // 10, n_keys // 3]
        r = RunTracesLruGroup(_dev(keys, np.int64), _dev(off, np.int64), _dev(types, np.uint8), _dev(inst, np.int32), k,
                              quotas, _dev(mask, np.int64), evict_batch=batch, mode=mode, instance_records=True,
                              policy=policies, timestamps=_dev(ts, np.int64), sample_rate=rates)
        torch.cuda.synchronize()
        got = [t.cpu().numpy() for t in (r[0], r[1], r[2], r[3], r[6])]
        for c, quota in enumerate(quotas):
            want = ref.RefOptimizer([dict(quota_capacity=quota,
                                          instances=[(str(j), p, rates[j]) for j, p in enumerate(policies)])],
                                    evict_batch=batch, mode=mode).run(keys, off, types, inst, mask, None, ts)
            for name, a, b in zip(NAMES, want, got):
                assert np.array_equal(a, b[c]), (seed, policies, batch, mode, quota, name)
            compared += 1
    assert compared == 24
