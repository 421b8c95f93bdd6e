"""The oracle's Optimizer restatement and the host side of the trace runner against the REFERENCE's own Optimizer.

tests/golden/optimizer_ref_kat.json and optimizer_ref_csv.json were written by tests/golden/make_optimizer_golden.py
from the reference's optimizer sources compiled in place (oracle/_ref/libkvcm_ref_optimizer.so): per-trace records of
its runner for the three eviction policies, instance groups in the three eviction modes, groups that mix two or all
three policies, offset and vector masks, a hierarchical group; and the CSV files its optimizer_main path writes for small trace files in the
three input formats.  The reference's own tests cover none of this beyond plain LRU with one instance, so these
fixtures are what pins the oracle (and, through it and directly, the GPU kernels: tests/test_gpu_optimizer_pins.py).
Where the compiled reference is present (a container that holds the reference tree), the oracle is also compared
with it live on larger random traces.  No GPU: the runner's device calls are replaced by the oracle here.
"""
import json
import os

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import kvcm_oracle as oracle
from oracle import ref_optimizer as ref

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import runner
from tair_kvcache_b200.optimizer.replay import LruGroupSweepResult, LruSweepResult

NAMES = ("external_hit_blocks", "internal_hit_blocks", "write_blocks", "instance_blocks", "blocks_of_every_instance")


def oracle_group(case, quota):
    k = len(case["policies"])
    return oracle.LruGroupReplay(quota, k, evict_batch=case["evict_batch"], mode=case["mode"], policy=case["policies"],
                                 sample_rate=case["sample_rates"]).run(
        case["keys"], case["key_off"], case["types"], case["instance"], case["mask_off"], case["mask_bits"],
        timestamps=case["timestamps"], instance_records=True)


def test_oracle_replays_what_the_reference_recorded():
    kat = load_golden("optimizer_ref_kat.json")
    assert len(kat["cases"]) >= 60
    seen = set()
    for case in kat["cases"]:
        for run in case["runs"]:
            ext, inte, wr, cached, final, every = oracle_group(case, run["quota"])
            for name, got in zip(NAMES, (ext, inte, wr, cached, every)):
                assert np.array_equal(np.asarray(run[name]), got), (case["name"], run["quota"], name)
            seen.add((tuple(case["policies"]), case["mode"]))
            assert max(run["instance_blocks"]) > 0
    # every policy alone and in groups, the policies mixed in one group, all three eviction modes
    for policies in (("lru",), ("leaf_aware_lru",), ("random_lru",), ("lru",) * 3, ("leaf_aware_lru",) * 3,
                     ("lru", "leaf_aware_lru", "lru"), ("random_lru",) * 2, ("random_lru", "lru", "leaf_aware_lru"),
                     ("leaf_aware_lru", "random_lru"), ("random_lru", "lru", "random_lru", "leaf_aware_lru")):
        for mode in (1, 2, 3):
            assert (policies, mode) in seen


def test_single_instance_oracle_classes_agree_with_the_fixture():
    """LruReplay (what the single-instance GPU sweeps are compared with) on the one-instance cases."""
    for case in load_golden("optimizer_ref_kat.json")["cases"]:
        if len(case["policies"]) != 1 or case["mode"] == 1:
            continue
        for run in case["runs"]:
            kw = dict(sample_rate=case["sample_rates"][0]) if case["policies"][0] == "random_lru" else {}
            got = oracle.LruReplay(run["quota"], evict_batch=case["evict_batch"], precise=case["mode"] == 3,
                                   policy=case["policies"][0], **kw).run(
                case["keys"], case["key_off"], case["types"], case["mask_off"], mask_bits=case["mask_bits"],
                timestamps=case["timestamps"])
            for name, g in zip(NAMES, got):
                assert np.array_equal(np.asarray(run[name]), g), (case["name"], name)


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref/libkvcm_ref_optimizer.so not built (reference tree absent)")
@pytest.mark.parametrize("policies", [["lru"], ["leaf_aware_lru"], ["random_lru"], ["leaf_aware_lru"] * 3,
                                      ["lru", "leaf_aware_lru", "lru"], ["random_lru", "random_lru"],
                                      ["random_lru", "lru", "leaf_aware_lru"]])
def test_oracle_against_the_compiled_reference(policies):
    from golden.make_optimizer_golden import workload
    rng = np.random.default_rng(len(policies) * 31 + len(policies[0]))
    k = len(policies)
    for mode in (1, 2, 3):
        for rw in (True, False):
            keys, off, types, mask, ts = workload(rng, 500, rw, max_blocks=40)
            inst = rng.integers(0, k, size=len(types)).astype(np.int32)
            rates = [float(r) for r in rng.choice([0.1, 0.25, 1.0], size=k)]
            bits = (rng.random(len(keys)) < 0.2).astype(np.uint8) if rw and mode == 2 else None
            for quota in (int(rng.integers(3, 40)), int(rng.integers(100, 2000))):
                want = ref.RefOptimizer([dict(quota_capacity=quota,
                                              instances=[(str(j), p, rates[j]) for j, p in enumerate(policies)])],
                                        evict_batch=6, mode=mode).run(keys, off, types, inst,
                                                                      None if bits is not None else mask, bits, ts)
                got = oracle.LruGroupReplay(quota, k, evict_batch=6, mode=mode, policy=policies,
                                            sample_rate=rates).run(keys, off, types, inst,
                                                                   None if bits is not None else mask, bits,
                                                                   timestamps=ts, instance_records=True)
                for name, a, b in zip(NAMES, want, (got[0], got[1], got[2], got[3], got[5])):
                    assert np.array_equal(a, b), (policies, mode, rw, quota, name)


# ---- the runner's host side (trace readers, grouping, CSV writer) on the reference's trace-file cases ------------

def _standins(monkeypatch):
    """The runner's device calls, answered by the oracle on CPU tensors."""
    def apply_prefix_hash(keys, off):
        out = np.concatenate([oracle.apply_prefix_hash(keys.numpy()[int(a):int(b)])
                              for a, b in zip(off.numpy()[:-1], off.numpy()[1:])] + [np.zeros(0, np.int64)])
        return torch.from_numpy(out)

    def run_traces_lru(keys, off, kind, quotas, mask, evict_batch, precise, mask_bits=None, policy="lru",
                       sample_rate=0.0, timestamps=None):
        kw = dict(sample_rate=sample_rate) if policy == "random_lru" else {}
        res = [oracle.LruReplay(q, evict_batch=evict_batch, precise=precise, policy=policy, **kw).run(
            keys.numpy(), off.numpy(), kind.numpy(), mask.numpy(),
            mask_bits=None if mask_bits is None else mask_bits.numpy(), timestamps=timestamps.numpy())
            for q in quotas]
        cols = [torch.from_numpy(np.stack([r[i] for r in res])) for i in range(4)]
        return LruSweepResult(*cols, None)

    def run_traces_lru_group(keys, off, kind, inst, n_inst, quotas, mask, evict_batch, mode, mask_bits=None,
                             instance_records=False, policy="lru", timestamps=None, sample_rate=0.0):
        r = oracle.LruGroupReplay(quotas[0], n_inst, evict_batch=evict_batch, mode=mode, policy=policy,
                                  sample_rate=sample_rate).run(
            keys.numpy(), off.numpy(), kind.numpy(), inst.numpy(), mask.numpy(),
            None if mask_bits is None else mask_bits.numpy(),
            timestamps=None if timestamps is None else timestamps.numpy(), instance_records=True)
        ext, inte, wr, size = [torch.from_numpy(x)[None] for x in r[:4]]
        return LruGroupSweepResult(ext, inte, wr, size, None, None, torch.from_numpy(r[5])[None])

    monkeypatch.setattr(runner, "ApplyPrefixHashBatch", apply_prefix_hash)
    monkeypatch.setattr(runner, "RunTracesLru", run_traces_lru)
    monkeypatch.setattr(runner, "RunTracesLruGroup", run_traces_lru_group)


def csv_rows(text):
    """Header and rows of a hit-rate CSV; the per-instance column as a sorted tuple (the reference lists the
    instances in the order of an unordered_map, which a replay cannot reproduce)."""
    lines = text.splitlines()
    rows = []
    for line in lines[1:]:
        cells = line.split(", ")
        cells[2] = tuple(sorted(int(x) for x in cells[2].split(";")))
        rows.append(tuple(cells))
    return lines[0], rows


def compare_with_reference_files(case, out_dir):
    assert sorted(os.listdir(out_dir)) == sorted(case["files"]), case["trace_type"]
    for name, want in case["files"].items():
        with open(os.path.join(out_dir, name)) as f:
            got = f.read()
        want_header, want_rows = csv_rows(want)
        got_header, got_rows = csv_rows(got)
        assert got_header == want_header
        assert got_rows == want_rows, (case["trace_type"], name)
        if ";" not in want:  # one instance in the configuration: byte for byte
            assert got == want


def test_trace_files_give_the_reference_csv_files(tmp_path, monkeypatch):
    _standins(monkeypatch)
    cases = load_golden("optimizer_ref_csv.json")["cases"]
    assert {c["trace_type"] for c in cases} == {"optimizer_schema", "qwen_bailian", "publisher_log"}
    for n, case in enumerate(cases):
        work = tmp_path / ("case%d" % n)
        work.mkdir()
        (work / "trace.jsonl").write_text(case["trace_text"])
        config = json.loads(json.dumps(case["config"]))
        config["trace_file_path"] = str(work / "trace.jsonl")
        config["output_result_path"] = str(work / "out")
        runner.run_startup_config(config, device="cpu")
        compare_with_reference_files(case, str(work / "out"))


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref/libkvcm_ref_optimizer.so not built (reference tree absent)")
@pytest.mark.parametrize("trace_type", ["optimizer_schema", "qwen_bailian", "publisher_log"])
def test_readers_give_the_reference_loader_s_traces_in_its_order(tmp_path, trace_type):
    """Trace by trace against OptimizerLoader::LoadTrace on a few thousand lines per format: kinds, instances,
    timestamps, keys, the keys a dialog turn replays, masks - and the ORDER, which for equal timestamps is that of
    the reference's std::sort over a list whose tail comes out of a std::unordered_map."""
    from golden.make_optimizer_golden import trace_files
    from tair_kvcache_b200.optimizer import trace_reader as tr
    (tmp_path / "trace.jsonl").write_text(trace_files(np.random.default_rng(0xB200000A), scale=40)[trace_type])
    instances = [("instance", "lru")] if trace_type == "qwen_bailian" else [("inst_a", "lru"), ("inst_b", "lru")]
    config = ref.startup_config([dict(quota_capacity=100, instances=instances)],
                                trace_file_path=str(tmp_path / "trace.jsonl"), trace_type=trace_type)
    want = ref.load_traces(config)
    got = tr.load_traces(str(tmp_path / "trace.jsonl"), trace_type, {i: 16 for i, _ in instances})
    assert len(got) == len(want) > 2000
    ties = 0
    for n, ((kind, doc), t) in enumerate(zip(want, got)):
        assert (kind, doc["instance_id"], doc["timestamp_us"]) == (t.kind, t.instance_id, t.timestamp_us), n
        keys = t.keys if not t.needs_prefix_hash else oracle.apply_prefix_hash(t.keys).tolist()
        assert doc["keys"] == keys, n
        if kind == tr.DIALOG_TURN:
            total = t.replay_keys() if not t.needs_prefix_hash else keys
            assert doc["total_keys"] == total and (doc["input_len"], doc["output_len"]) == (t.input_len, t.output_len), n
        if kind != tr.WRITE_CACHE and trace_type != "qwen_bailian":
            mask = doc["block_mask"]
            assert (mask == t.block_mask) or (mask == [] and t.block_mask in ([], None)), n
        ties += n > 0 and want[n - 1][1]["timestamp_us"] == doc["timestamp_us"]
    assert ties > 50  # equal timestamps are there to be ordered
