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
