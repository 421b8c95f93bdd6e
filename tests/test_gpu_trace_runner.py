"""Trace file -> GPU replay -> hit-rate CSV, against the sequential oracle replay of the same traces."""
import json

import numpy as np
import pytest

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import run_trace_file, trace_reader as tr
from tair_kvcache_b200.optimizer.runner import CSV_HEADER

pytestmark = pytest.mark.gpu


def _write_qwen_trace(path, rng, n):
    """Dialog turns whose per-block ids share prefixes with earlier turns."""
    seqs = []
    with open(path, "w") as f:
        for i in range(n):
            ids = rng.integers(1, 1 << 40, size=int(rng.integers(0, 30))).tolist()
            if seqs and rng.random() < 0.7:
                src = seqs[int(rng.integers(0, len(seqs)))]
                m = int(rng.integers(0, min(len(src), len(ids)) + 1))
                ids[:m] = src[:m]
            seqs.append(ids)
            f.write(json.dumps({"timestamp": float(n - i) + 0.5, "hash_ids": ids, "input_length": len(ids) * 16,
                                "output_length": 1}) + "\n")  # descending timestamps: the loader must sort
    return seqs


def test_qwen_bailian_file_end_to_end(tmp_path):
    rng = np.random.default_rng(8)
    path = tmp_path / "trace.jsonl"
    seqs = _write_qwen_trace(path, rng, 400)
    out = run_trace_file(str(path), "qwen_bailian", str(tmp_path / "out"), device="cuda:0")
    rec = out["instance"]
    # oracle: ApplyPrefixHash per turn, turns in timestamp order (= reversed file order), sequential replay
    ordered = seqs[::-1]
    keys = [oracle.apply_prefix_hash(s) for s in ordered]
    off = np.zeros(len(keys) + 1, dtype=np.int64)
    np.cumsum([len(k) for k in keys], out=off[1:])
    want = oracle.Replay().run(np.concatenate(keys), off, np.zeros(len(keys), dtype=np.uint8))
    assert np.array_equal(rec["external_hit_blocks"], want[0]) and np.array_equal(rec["write_blocks"], want[2])
    assert np.array_equal(rec["current_cache_blocks"], want[3]) and want[0].sum() > 0
    lines = (tmp_path / "out" / "instance_hit_rates.csv").read_text().splitlines()
    assert lines[0] + "\n" == CSV_HEADER and len(lines) == 401
    # last line: accumulated external hit rate = all hits / all reads, printed like a C++ double
    acc = want[0].sum() / sum(len(s) for s in seqs)
    assert lines[-1].split(", ")[-1] == "%g" % acc and lines[-1].split(", ")[0] == "400500000"


def test_publisher_log_file_in_both_replay_modes(tmp_path):
    def ev(kind, ts, **kw):
        return json.dumps(dict(type=kind, source="i1", trigger_time_us=ts, **kw))
    path = tmp_path / "pub.log"
    path.write_text("\n".join([
        ev("GetCacheLocation", 10, query_type="prefix_match", keys=[1, 2, 3, 4], block_mask=0),
        ev("StartWriteCache", 20, write_session_id="a", keys=[1, 2, 3, 4, 5]),
        ev("FinishWriteCache", 30, write_session_id="a"),
        ev("GetCacheLocation", 40, query_type="prefix_match", keys=[1, 2, 3, 9], block_mask=1),
        ev("StartWriteCache", 50, write_session_id="b", keys=[1, 2, 3, 9, 10]),
        ev("FinishWriteCache", 60, write_session_id="b")]))
    # dialog-turn mode: turn 1 writes 5 blocks, turn 2 hits [1,2,3] and writes [9,10]
    rec = run_trace_file(str(path), "publisher_log", str(tmp_path / "o1"), "cuda:0", {"i1": 64})["i1"]
    assert rec["kind"].tolist() == [tr.DIALOG_TURN, tr.DIALOG_TURN]
    assert rec["external_hit_blocks"].tolist() == [0, 3] and rec["write_blocks"].tolist() == [5, 2]
    assert rec["external_read_blocks"].tolist() == [4, 4] and rec["current_cache_blocks"].tolist() == [5, 7]
    # read/write-separation mode: Get(10) misses, Write(30) writes 5, Get(40) masks key 1 (internal) and hits 2,3
    rec = run_trace_file(str(path), "publisher_log", str(tmp_path / "o2"), "cuda:0", {"i1": 64}, rw_separation=True)["i1"]
    assert rec["kind"].tolist() == [tr.GET_LOCATION, tr.WRITE_CACHE, tr.GET_LOCATION, tr.WRITE_CACHE]
    assert rec["external_hit_blocks"].tolist() == [0, 0, 2, 0] and rec["internal_hit_blocks"].tolist() == [0, 0, 1, 0]
    assert rec["write_blocks"].tolist() == [0, 5, 0, 2] and rec["internal_read_blocks"].tolist() == [0, 0, 1, 0]
    csv = (tmp_path / "o2" / "i1_hit_rates.csv").read_text().splitlines()
    assert len(csv) == 3 and csv[2] == "40, 5, 5, 5, 1, 3, 4, 1, 0.25, 2, 0.5, 0.75, 0.125, 0.25, 0.375"


def test_qwen_bailian_file_with_lru_quota_sweep(tmp_path):
    from tair_kvcache_b200.optimizer import tradeoff_curve
    rng = np.random.default_rng(9)
    path = tmp_path / "trace.jsonl"
    seqs = _write_qwen_trace(path, rng, 600)
    quotas = [10, 50, 200, 1000, 100000]
    out = run_trace_file(str(path), "qwen_bailian", str(tmp_path / "out"), device="cuda:0", quota_blocks=quotas,
                         evict_batch=5)
    recs = out["instance"]
    ordered = seqs[::-1]
    keys = [oracle.apply_prefix_hash(s) for s in ordered]
    off = np.zeros(len(keys) + 1, dtype=np.int64)
    np.cumsum([len(k) for k in keys], out=off[1:])
    flat, kinds = np.concatenate(keys), np.zeros(len(keys), dtype=np.uint8)
    rates = tradeoff_curve(recs)
    for c, q in enumerate(quotas):
        want = oracle.LruReplay(q, evict_batch=5).run(flat, off, kinds)
        assert np.array_equal(recs[c]["external_hit_blocks"], want[0])
        assert np.array_equal(recs[c]["write_blocks"], want[2])
        assert np.array_equal(recs[c]["current_cache_blocks"], want[3])
        assert rates[c, 1] == want[0].sum() / sum(len(s) for s in seqs) and rates[c, 0] == 0
        lines = (tmp_path / "out" / ("instance_quota%d_hit_rates.csv" % q)).read_text().splitlines()
        assert len(lines) == 601 and lines[-1].split(", ")[-1] == "%g" % rates[c, 2]
    assert rates[0, 2] < rates[2, 2] <= rates[4, 2]  # a larger cache never hurts this trace
    # the same curve from the totals-only sweep
    from tair_kvcache_b200.optimizer import sweep_hit_rates
    light = sweep_hit_rates(tr.load_traces(str(path), "qwen_bailian"), "cuda:0", quotas, evict_batch=5)
    assert np.array_equal(light, rates)
    # a single quota gives one record and the plain file name
    rec = run_trace_file(str(path), "qwen_bailian", str(tmp_path / "one"), device="cuda:0", quota_blocks=50,
                         evict_batch=5)["instance"]
    assert np.array_equal(rec["external_hit_blocks"], recs[1]["external_hit_blocks"])
    assert (tmp_path / "one" / "instance_hit_rates.csv").exists()


def test_startup_config_drives_a_publisher_log_replay_with_eviction(tmp_path):
    """The reference's `optimizer_main <config>` flow: configuration file -> trace -> per-instance CSV, with a group
    quota small enough to evict.  Expected numbers are worked out by hand from the LRU rules."""
    from tair_kvcache_b200.optimizer import run_startup_config

    def ev(kind, ts, **kw):
        return json.dumps(dict(type=kind, source="i1", trigger_time_us=ts, **kw))
    path = tmp_path / "pub.log"
    path.write_text("\n".join([
        ev("StartWriteCache", 10, write_session_id="a", keys=[1, 2, 3]),
        ev("FinishWriteCache", 11, write_session_id="a"),                       # cache: 1 2 3
        ev("GetCacheLocation", 20, query_type="prefix_match", keys=[1, 2, 3], block_mask=0),  # hit 3, all refreshed
        ev("StartWriteCache", 30, write_session_id="b", keys=[7, 8]),
        ev("FinishWriteCache", 31, write_session_id="b"),                       # 5 cached > 4: one batch of 2 evicts 1, 2
        ev("GetCacheLocation", 40, query_type="prefix_match", keys=[1, 2, 3], block_mask=0),  # 1 is gone: no hit
        ev("GetCacheLocation", 50, query_type="prefix_match", keys=[7, 8, 9], block_mask=1)]))  # 7 masked, 8 hit
    cfg = {"trace_file_path": str(path), "trace_type": "publisher_log", "output_result_path": str(tmp_path / "out"),
           "eviction_params": {"eviction_mode": 2, "eviction_batch_size_per_instance": 2},
           "instance_groups": [{"group_name": "g", "quota_capacity": 8, "used_percentage": 0.5,
                                "hierarchical_eviction_enabled": False, "storages": [],
                                "instances": [{"instance_id": "i1", "block_size": 64, "eviction_policy_type": "lru",
                                               "eviction_policy_params": {"sample_rate": 0.1}}]}]}
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(cfg))
    rec = run_startup_config(str(cfg_path), device="cuda:0")["i1"]
    assert rec["kind"].tolist() == [tr.WRITE_CACHE, tr.GET_LOCATION, tr.WRITE_CACHE, tr.GET_LOCATION, tr.GET_LOCATION]
    assert rec["write_blocks"].tolist() == [3, 0, 2, 0, 0]
    assert rec["external_hit_blocks"].tolist() == [0, 3, 0, 0, 1]
    assert rec["internal_hit_blocks"].tolist() == [0, 0, 0, 0, 1]
    assert rec["current_cache_blocks"].tolist() == [3, 3, 3, 3, 3]
    # the same through the oracle's radix tree
    keys, off = [1, 2, 3, 1, 2, 3, 7, 8, 1, 2, 3, 7, 8, 9], [0, 3, 6, 8, 11, 14]
    want = oracle.LruReplay(4, evict_batch=2).run(keys, off, rec["kind"], [0, 0, 0, 0, 1])
    assert np.array_equal(want[0], rec["external_hit_blocks"]) and np.array_equal(want[3], rec["current_cache_blocks"])
    assert len((tmp_path / "out" / "i1_hit_rates.csv").read_text().splitlines()) == 4
    # the same file under the instance's other policy: the configuration picks the kernel, the event times reach it
    cfg["instance_groups"][0]["instances"][0]["eviction_policy_type"] = "leaf_aware_lru"
    rec = run_startup_config(cfg, device="cuda:0")["i1"]
    want = oracle.LruReplay(4, evict_batch=2, policy="leaf_aware_lru").run(keys, off, rec["kind"], [0, 0, 0, 0, 1],
                                                                           timestamps=rec["timestamp_us"])
    for name, w in zip(("external_hit_blocks", "internal_hit_blocks", "write_blocks", "current_cache_blocks"), want):
        assert np.array_equal(w, rec[name]), name


def test_optimizer_schema_query_with_a_holey_vector_mask(tmp_path):
    """GetLocation traces of the optimizer schema carry block_mask as an offset or as a bool vector; a vector with
    holes reaches the GPU as one byte per key."""
    path = tmp_path / "schema.jsonl"
    path.write_text("\n".join([
        json.dumps({"instance_id": "i", "trace_id": "w", "timestamp_us": 1, "tokens": [], "keys": [1, 2, 3, 4]}),
        json.dumps({"instance_id": "i", "trace_id": "g", "timestamp_us": 2, "tokens": [], "keys": [1, 2, 3, 4, 5],
                    "query_type": "prefix_match", "block_mask": [False, True, False, True, True], "sw_size": 0,
                    "location_spec_names": []})]))
    rec = run_trace_file(str(path), "optimizer_schema", str(tmp_path / "out"), device="cuda:0", rw_separation=True)["i"]
    assert rec["kind"].tolist() == [tr.WRITE_CACHE, tr.GET_LOCATION]
    assert rec["external_hit_blocks"].tolist() == [0, 2] and rec["internal_hit_blocks"].tolist() == [0, 2]
    assert rec["internal_read_blocks"].tolist() == [0, 3] and rec["external_read_blocks"].tolist() == [0, 2]


def test_two_instances_of_one_group_share_the_quota(tmp_path):
    """The startup configuration names two "lru" instances in one group: they are replayed together against the
    shared quota (kv_cache_manager/optimizer/manager/eviction_manager.cc:86-146), each gets its own CSV."""
    from tair_kvcache_b200.optimizer import run_startup_config
    path = tmp_path / "schema.jsonl"

    def line(inst, ts, keys, query=False):
        d = {"instance_id": inst, "trace_id": "t%d" % ts, "timestamp_us": ts, "tokens": [], "keys": keys}
        if query:
            d.update(query_type="prefix_match", block_mask=0, sw_size=0, location_spec_names=[])
        return json.dumps(d)
    path.write_text("\n".join([line("a", 1, [1, 2, 3]), line("b", 2, [1, 2]), line("a", 3, [1, 2, 3], True),
                               line("b", 4, [1, 2], True)]))
    cfg = {"trace_file_path": str(path), "trace_type": "optimizer_schema", "output_result_path": str(tmp_path / "out"),
           "eviction_params": {"eviction_mode": 1, "eviction_batch_size_per_instance": 1},
           "instance_groups": [{"group_name": "g", "quota_capacity": 4, "used_percentage": 1.0,
                                "hierarchical_eviction_enabled": False, "storages": [],
                                "instances": [{"instance_id": "a", "block_size": 16, "eviction_policy_type": "lru"},
                                              {"instance_id": "b", "block_size": 16, "eviction_policy_type": "lru"}]}]}
    recs = run_startup_config(cfg, device="cuda:0", rw_separation=True)
    # 5 blocks against a quota of 4: one round takes block 1 from a and from b (see tests/test_oracle.py)
    assert recs["a"]["current_cache_blocks"].tolist() == [3, 2] and recs["a"]["external_hit_blocks"].tolist() == [0, 0]
    assert recs["b"]["current_cache_blocks"].tolist() == [1, 1] and recs["b"]["write_blocks"].tolist() == [2, 0]
    assert (tmp_path / "out" / "a_hit_rates.csv").exists() and (tmp_path / "out" / "b_hit_rates.csv").exists()
    cfg["eviction_params"]["eviction_mode"] = 2  # only the writer b pays
    recs = run_startup_config(cfg, device="cuda:0", rw_separation=True)
    assert recs["a"]["current_cache_blocks"].tolist() == [3, 3] and recs["a"]["external_hit_blocks"].tolist() == [0, 3]
