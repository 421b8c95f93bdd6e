"""The trace-file readers (host logic) on hand-made lines that exercise the rules of the reference's converters."""
import json

import numpy as np
import pytest

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import trace_reader as tr


def _lines(*docs):
    return [json.dumps(d) for d in docs]


def test_qwen_bailian_lines_become_dialog_turns_with_raw_ids():
    t = tr.read_qwen_bailian(_lines({"timestamp": 1.5, "hash_ids": [100, 200, 300], "input_length": 48,
                                     "output_length": 7}, {"timestamp": 0.25, "hash_ids": []}) + ["not json", ""])
    assert [x.kind for x in t] == [tr.DIALOG_TURN, tr.DIALOG_TURN]
    assert t[0].timestamp_us == 1500000 and t[0].keys == [100, 200, 300] and t[0].needs_prefix_hash
    assert t[0].instance_id == "instance" and t[0].input_len == 48 and t[0].output_len == 7
    assert t[1].timestamp_us == 250000 and t[1].keys == []


def test_optimizer_schema_type_is_inferred_from_the_fields():
    t = tr.read_optimizer_schema(_lines(
        {"instance_id": "a", "timestamp_us": 3, "keys": [1, 2], "query_type": "prefix_match", "block_mask": 1,
         "sw_size": 0, "input_len": 128, "output_len": 64, "total_keys": [1, 2, 3]},
        {"instance_id": "a", "timestamp_us": 1, "keys": [1, 2], "query_type": "prefix_match",
         "block_mask": [True, False]},
        {"instance_id": "b", "timestamp_us": 2, "keys": [9]}))
    assert [x.kind for x in t] == [tr.DIALOG_TURN, tr.GET_LOCATION, tr.WRITE_CACHE]
    assert t[0].total_keys == [1, 2, 3] and t[0].block_mask == 1 and t[0].replay_keys() == [1, 2, 3]
    assert t[1].block_mask == [True, False] and t[2].instance_id == "b"


def test_publisher_log_events_are_paired_like_the_reference():
    lines = _lines(
        {"type": "GetCacheLocation", "source": "i1", "trigger_time_us": 10, "query_type": "prefix_match",
         "keys": [1, 2, 3, 99], "block_mask": 1, "sw_size": -1},
        {"type": "GetCacheLocation", "source": "other", "trigger_time_us": 11, "keys": [5]},       # unknown instance
        {"type": "StartWriteCache", "source": "i1", "trigger_time_us": 20, "write_session_id": "s1",
         "keys": [1, 2, 3, 4, 5]},                                                                # opens with [1,2,3]
        {"type": "FinishWriteCache", "source": "i1", "trigger_time_us": 30, "write_session_id": "s1",
         "success_block": 5},
        {"type": "StartWriteCache", "source": "i1", "trigger_time_us": 40, "write_session_id": "s2", "keys": [7, 8]},
        {"type": "GetCacheLocation", "source": "i1", "trigger_time_us": 50, "query_type": "prefix_match",
         "keys": [7, 8, 9], "block_mask": [True, False, False]},
        {"type": "FinishWriteCache", "source": "i1", "trigger_time_us": 60, "write_session_id": "nope"})
    t = tr.read_publisher_log(lines, {"i1": 64})
    kinds = [(x.kind, x.timestamp_us) for x in t]
    # the first Get, its dialog turn (keeps the Get's timestamp), the finished write (finish time), then what was
    # left pending: the unfinished write (+100 ms) and the unmatched Get as a dialog turn over its own keys
    assert kinds == [(tr.GET_LOCATION, 10), (tr.DIALOG_TURN, 10), (tr.WRITE_CACHE, 30), (tr.GET_LOCATION, 50),
                     (tr.WRITE_CACHE, 100040), (tr.DIALOG_TURN, 50)]
    turn = t[1]
    assert turn.keys == [1, 2, 3, 99] and turn.total_keys == [1, 2, 3, 4, 5]
    assert turn.input_len == 4 * 64 and turn.output_len == (5 - 3) * 64 and turn.block_mask == 1
    assert t[5].total_keys == [7, 8, 9] and t[5].output_len == 0


def test_load_traces_sorts_by_timestamp_and_csr_layout(tmp_path):
    p = tmp_path / "schema.jsonl"
    p.write_text("\n".join(_lines(
        {"instance_id": "a", "timestamp_us": 30, "keys": [1, 2, 4], "query_type": "prefix_match", "block_mask": 1},
        {"instance_id": "a", "timestamp_us": 10, "keys": [1, 2, 3]})))
    t = tr.load_traces(str(p), "optimizer_schema")
    assert [x.timestamp_us for x in t] == [10, 30]
    keys, off, kind, mask, read = tr.to_csr(t)
    assert keys.tolist() == [1, 2, 3, 1, 2, 4] and off.tolist() == [0, 3, 6]
    assert kind.tolist() == [tr.WRITE_CACHE, tr.GET_LOCATION] and mask.tolist() == [0, 1] and read.tolist() == [0, 3]
    with pytest.raises(ValueError):
        tr.load_traces(str(p), "nonsense")


def test_mask_offset_rules():
    assert tr.mask_offset(None, 5) == 0 and tr.mask_offset(3, 5) == 3 and tr.mask_offset(9, 5) == 5
    assert tr.mask_offset([True, True, False], 3) == 2 and tr.mask_offset([], 3) == 0
    # a vector with holes: the leading run is the offset, the rest travels as one byte per key
    assert tr.mask_offset([True, False, True], 3) == 1 and tr.masked_count([True, False, True], 3) == 2
    traces = [tr.Trace(kind=tr.GET_LOCATION, keys=[1, 2, 3], block_mask=[True, False, True]),
              tr.Trace(kind=tr.WRITE_CACHE, keys=[4, 5]),
              tr.Trace(kind=tr.GET_LOCATION, keys=[6, 7], block_mask=[True, True])]
    keys, off, kind, mask, read = tr.to_csr(traces)
    assert mask.tolist() == [1, 0, 2]
    assert tr.mask_bits(traces, off).tolist() == [1, 0, 1, 0, 0, 0, 0]
    assert tr.mask_bits(traces[1:], tr.to_csr(traces[1:])[1]) is None  # no holes: nothing to pass


def test_startup_config_of_the_reference_is_understood():
    """The shipped example (kv_cache_manager/optimizer/optimizer_startup_config_load.json), transcribed: one group,
    quota 12000 x 1.0, rough group eviction in batches of 100, one "lru" instance with block size 16."""
    import pytest
    from tair_kvcache_b200.optimizer.runner import parse_startup_config
    cfg = {"trace_file_path": "/data/event_publisher.log", "trace_type": "publisher_log",
           "output_result_path": "/data/out",
           "eviction_params": {"eviction_mode": 1, "eviction_batch_size_per_instance": 100},
           "instance_groups": [{"group_name": "instance_group_01", "quota_capacity": 12000, "used_percentage": 1.0,
                                "hierarchical_eviction_enabled": False,
                                "storages": [{"unique_name": "pace_00", "storage_type": "pace", "capacity": 100000}],
                                "instances": [{"instance_id": "3780643326877293460", "block_size": 16,
                                               "eviction_policy_type": "lru",
                                               "eviction_policy_params": {"sample_rate": 0.1}}]}]}
    c = parse_startup_config(cfg)
    assert c["quota_blocks"] == {"3780643326877293460": 12000} and c["block_sizes"] == {"3780643326877293460": 16}
    assert c["evict_batch"] == 100 and c["precise"] is False and c["trace_type"] == "publisher_log"
    cfg["instance_groups"][0]["used_percentage"] = 0.75
    cfg["eviction_params"]["eviction_mode"] = 3
    c = parse_startup_config(cfg)
    assert c["quota_blocks"]["3780643326877293460"] == 9000 and c["precise"] is True
    # hierarchical eviction: the first tier's capacity takes the place of quota_capacity
    # (kv_cache_manager/optimizer/manager/eviction_manager.cc:247-258); nothing else changes for a replay
    cfg["instance_groups"][0]["hierarchical_eviction_enabled"] = True
    assert parse_startup_config(cfg)["quota_blocks"]["3780643326877293460"] == 75000
    cfg["instance_groups"][0]["hierarchical_eviction_enabled"] = False
    # what the GPU replay does not reproduce is refused, not approximated
    cfg["instance_groups"][0]["instances"][0]["eviction_policy_type"] = "leaf_aware_lru"
    assert parse_startup_config(cfg)["policies"] == {"3780643326877293460": "leaf_aware_lru"}
    cfg["instance_groups"][0]["instances"][0]["eviction_policy_type"] = "random_lru"
    c = parse_startup_config(cfg)
    assert c["policies"] == {"3780643326877293460": "random_lru"} and c["sample_rates"] == {"3780643326877293460": 0.1}
    cfg["instance_groups"][0]["instances"][0]["eviction_policy_type"] = "fifo"
    with pytest.raises(NotImplementedError):
        parse_startup_config(cfg)
    cfg["instance_groups"][0]["instances"][0]["eviction_policy_type"] = "lru"
    cfg["instance_groups"][0]["instances"].append({"instance_id": "b", "block_size": 16, "eviction_policy_type": "lru"})
    c = parse_startup_config(cfg)  # two "lru" instances share the quota: replayed together
    assert c["groups"] == [dict(group_name=cfg["instance_groups"][0]["group_name"],
                                instances=["3780643326877293460", "b"], quota=9000, policy="lru")]
    assert c["quota_blocks"] == {} and c["mode"] == 3
    cfg["instance_groups"][0]["instances"][1]["eviction_policy_type"] = "leaf_aware_lru"
    assert parse_startup_config(cfg)["groups"][0]["policy"] == ["lru", "leaf_aware_lru"]  # one name per instance
    cfg["instance_groups"][0]["instances"][0]["eviction_policy_type"] = "leaf_aware_lru"
    assert parse_startup_config(cfg)["groups"][0]["policy"] == "leaf_aware_lru"  # the same policy throughout
    cfg["instance_groups"][0]["instances"][1]["eviction_policy_type"] = "random_lru"
    g = parse_startup_config(cfg)["groups"][0]  # a sampling instance beside a queueing one in a shared quota
    assert g["policy"] == ["leaf_aware_lru", "random_lru"] and g["sample_rate"] == [0.1, 0.0]
    cfg["instance_groups"][0]["instances"][0]["eviction_policy_type"] = "random_lru"
    g = parse_startup_config(cfg)["groups"][0]  # sampling instances only: replayed, each with its own rate
    assert g["policy"] == "random_lru" and g["sample_rate"] == [0.1, 0.0]
    cfg["eviction_params"]["eviction_mode"] = 0  # no eviction is ever performed: any grouping replays
    assert parse_startup_config(cfg)["quota_blocks"] == {}


def test_shared_quota_groups_host_side(tmp_path, monkeypatch):
    """The runner's handling of a group whose instances share a quota, without a GPU: the device call is replaced by
    the oracle, so this covers the grouping of traces by instance, the per-instance records and the CSV files."""
    import json

    import numpy as np
    import torch

    from oracle import kvcm_oracle as oracle
    from tair_kvcache_b200.optimizer import runner

    from tair_kvcache_b200.optimizer.replay import LruGroupSweepResult

    def stand_in(keys, off, kind, inst, n_inst, quotas, mask, evict_batch, mode, mask_bits=None,
                 instance_records=False, policy="lru", timestamps=None, sample_rate=0.0):
        assert (timestamps is not None) == (policy != "lru")
        r = oracle.LruGroupReplay(quotas[0], n_inst, evict_batch=evict_batch, mode=mode, policy=policy).run(
            keys.numpy(), off.numpy(), kind.numpy(), inst.numpy(), mask.numpy(), instance_records=True,
            timestamps=None if timestamps is None else timestamps.numpy())
        ext, inte, wr, size = [torch.from_numpy(x)[None] for x in r[:4]]
        return LruGroupSweepResult(ext, inte, wr, size, None, None, torch.from_numpy(r[5])[None])

    monkeypatch.setattr(runner, "RunTracesLruGroup", stand_in)

    def line(inst, ts, keys, query=False):
        d = {"instance_id": inst, "trace_id": "t%d" % ts, "timestamp_us": ts, "tokens": [], "keys": keys}
        if query:
            d.update(query_type="prefix_match", block_mask=0, sw_size=0, location_spec_names=[])
        return json.dumps(d)
    path = tmp_path / "schema.jsonl"
    path.write_text("\n".join([line("a", 1, [1, 2, 3]), line("b", 2, [1, 2]), line("a", 3, [1, 2, 3], True),
                               line("b", 4, [1, 2], True)]))
    cfg = {"trace_file_path": str(path), "trace_type": "optimizer_schema", "output_result_path": str(tmp_path / "out"),
           "eviction_params": {"eviction_mode": 1, "eviction_batch_size_per_instance": 1},
           "instance_groups": [{"group_name": "g", "quota_capacity": 4, "used_percentage": 1.0,
                                "hierarchical_eviction_enabled": False, "storages": [],
                                "instances": [{"instance_id": "a", "block_size": 16, "eviction_policy_type": "lru"},
                                              {"instance_id": "b", "block_size": 16, "eviction_policy_type": "lru"}]}]}
    recs = runner.run_startup_config(cfg, device="cpu", rw_separation=True)
    assert recs["a"]["current_cache_blocks"].tolist() == [3, 2] and recs["b"]["current_cache_blocks"].tolist() == [1, 1]
    assert recs["a"]["timestamp_us"].tolist() == [1, 3] and recs["b"]["write_blocks"].tolist() == [2, 0]
    rows = (tmp_path / "out" / "a_hit_rates.csv").read_text().splitlines()
    # CachedBlocksCurrentInstance, CachedBlocksPerInstance (a;b), CachedBlocksAllInstance: after b's write the group
    # held 5 blocks, one round of group-rough eviction took one from each
    assert len(rows) == 2 and rows[1].startswith("3, 2, 2;1, 3, 0, 3, 3, 0, ")
    assert recs["b"]["blocks_per_instance"].tolist() == [[2, 1], [2, 1]]
    cfg["eviction_params"]["eviction_mode"] = 2
    recs = runner.run_startup_config(cfg, device="cpu", rw_separation=True)
    assert recs["a"]["external_hit_blocks"].tolist() == [0, 3] and np.array_equal(recs["a"]["kind"], [2, 1])
    # the same group under "leaf_aware_lru": the policy and the traces' timestamps reach the group replay
    for i in cfg["instance_groups"][0]["instances"]:
        i["eviction_policy_type"] = "leaf_aware_lru"
    cfg["eviction_params"]["eviction_mode"] = 1
    recs = runner.run_startup_config(cfg, device="cpu", rw_separation=True)
    assert recs["a"]["current_cache_blocks"].tolist() == [3, 2] and recs["b"]["blocks_per_instance"].tolist() == [[2, 1]] * 2
    cfg["instance_groups"][0]["instances"][0]["eviction_policy_type"] = "lru"  # a mixed group: one name per instance
    recs = runner.run_startup_config(cfg, device="cpu", rw_separation=True)
    assert recs["a"]["current_cache_blocks"].tolist() == [3, 2] and recs["b"]["write_blocks"].tolist() == [2, 0]


def test_a_key_repeated_inside_a_trace_is_found_before_any_launch():
    import pytest
    from tair_kvcache_b200.optimizer import trace_reader as tr
    keys = np.array([5, 6, 7, 5, 8, 9, 8, 10, 6], dtype=np.int64)
    assert tr.first_repeat_within_a_trace(keys, np.array([0, 3, 6, 9])) is None      # repeats only across traces
    assert tr.first_repeat_within_a_trace(keys, np.array([0, 3, 7, 9])) == 1         # 8 twice in the second trace
    assert tr.first_repeat_within_a_trace(keys[:1], np.array([0, 1])) is None
    verbatim = [tr.Trace(kind=tr.GET_LOCATION, keys=[1, 2, 3]), tr.Trace(kind=tr.GET_LOCATION, keys=[4, 5, 4])]
    k, off = tr.to_csr(verbatim)[:2]
    with pytest.raises(NotImplementedError):
        tr.require_no_repeats(verbatim, k, off)
    hashed = [tr.Trace(kind=tr.DIALOG_TURN, keys=[4, 5, 4], needs_prefix_hash=True)]
    k, off = tr.to_csr(hashed)[:2]
    tr.require_no_repeats(hashed, k, off)  # ids that repeat are chained into distinct keys before the replay
