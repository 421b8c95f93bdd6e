"""Generates tests/golden/optimizer_ref_kat.json and tests/golden/optimizer_ref_csv.json from the reference's OWN
Optimizer.

Run in a container that holds the reference tree: `make -C oracle KVCM_REF_DIR=<tree>` compiles the reference's
optimizer sources in place into oracle/_ref/libkvcm_ref_optimizer.so (oracle/ref_optimizer_driver.cc wraps it), and
this script feeds it seeded traces.  The committed JSON files are what travels: the tests replay them against the
oracle restatement (any box) and against the CUDA kernels (GPU box), so eviction policies, instance groups, trace
readers and the hit-rate CSV are pinned to the reference's answers where the reference has no tests of its own.

    python tests/golden/make_optimizer_golden.py
"""
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import kvcm_oracle as oracle  # noqa: E402
from oracle import ref_optimizer as ref  # noqa: E402

W, G, D = 2, 1, 0  # WriteCache, GetLocation, DialogTurn


def workload(rng, n_traces, rw_separation, max_blocks=12):
    """Chained keys of token sequences that share prefixes with earlier ones; timestamps that repeat."""
    bs = 16
    seqs, keys, off, types, mask, ts = [], [], [0], [], [], []
    now = 1_700_000_000_000_000
    for _ in range(n_traces):
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


def replay_cases():
    cases = []
    rng = np.random.default_rng(0xB2000007)
    layouts = [(["lru"], "one lru instance"), (["leaf_aware_lru"], "one leaf_aware_lru instance"),
               (["random_lru"], "one random_lru instance"), (["lru"] * 3, "three lru instances"),
               (["leaf_aware_lru"] * 3, "three leaf_aware_lru instances"),
               (["lru", "leaf_aware_lru", "lru"], "lru and leaf_aware_lru instances mixed"),
               (["random_lru"] * 2, "two random_lru instances")]

    def record(layouts):
        for policies, what in layouts:
            for mode in (1, 2, 3):
                for rw in (True, False):
                    keys, off, types, mask, ts = workload(rng, 70, rw)
                    k = len(policies)
                    inst = rng.integers(0, k, size=len(types)).astype(np.int32)
                    rates = [float(r) for r in rng.choice([0.1, 0.25, 0.5, 1.0], size=k)]
                    use_bits = bool(rng.random() < 0.3) and rw
                    bits = (rng.random(len(keys)) < 0.25).astype(np.uint8) if use_bits else None
                    batch = int(rng.integers(1, 9))
                    runs = []
                    for quota in (int(rng.integers(3, 25)), int(rng.integers(40, 200))):
                        r = ref.RefOptimizer([dict(quota_capacity=quota,
                                                   instances=[(str(j), p, rates[j]) for j, p in enumerate(policies)])],
                                             evict_batch=batch, mode=mode)
                        ext, inte, wr, cached, every = r.run(keys, off, types, inst, None if use_bits else mask, bits, ts)
                        runs.append(dict(quota=quota, external_hit_blocks=ext.tolist(), internal_hit_blocks=inte.tolist(),
                                         write_blocks=wr.tolist(), instance_blocks=cached.tolist(),
                                         blocks_of_every_instance=every.tolist()))
                    cases.append(dict(name="%s, mode %d, %s" % (what, mode, "read/write" if rw else "turns"),
                                      policies=policies, sample_rates=rates, mode=mode, evict_batch=batch,
                                      keys=keys.tolist(), key_off=off.tolist(), types=types.tolist(),
                                      instance=inst.tolist(), mask_off=None if use_bits else mask.tolist(),
                                      mask_bits=bits.tolist() if use_bits else None, timestamps=ts.tolist(), runs=runs))

    record(layouts)
    # hierarchical eviction: the first tier's capacity x used_percentage is the quota
    keys, off, types, mask, ts = workload(rng, 120, False)
    r = ref.RefOptimizer([dict(quota_capacity=10 ** 9, hierarchical=True, tier_capacity=120, used_percentage=0.5,
                               instances=[("0", "leaf_aware_lru")])], evict_batch=4, mode=2)
    ext, inte, wr, cached, every = r.run(keys, off, types, None, mask, None, ts)
    cases.append(dict(name="hierarchical group: 0.5 of a first tier of 120 blocks", policies=["leaf_aware_lru"],
                      sample_rates=[0.1], mode=2, evict_batch=4, keys=keys.tolist(), key_off=off.tolist(),
                      types=types.tolist(), instance=[0] * len(types), mask_off=mask.tolist(), mask_bits=None,
                      timestamps=ts.tolist(),
                      runs=[dict(quota=60, external_hit_blocks=ext.tolist(), internal_hit_blocks=inte.tolist(),
                                 write_blocks=wr.tolist(), instance_blocks=cached.tolist(),
                                 blocks_of_every_instance=every.tolist())],
                      startup_group=dict(quota_capacity=10 ** 9, used_percentage=0.5,
                                         hierarchical_eviction_enabled=True, storages=[dict(capacity=120)])))
    # sampling instances beside queueing ones in one group (recorded after the cases above so that those keep their
    # workloads)
    record([(["random_lru", "lru", "leaf_aware_lru"], "all three policies mixed"),
            (["leaf_aware_lru", "random_lru"], "leaf_aware_lru and random_lru instances"),
            (["random_lru", "lru", "random_lru", "leaf_aware_lru"], "two random_lru instances among four")])
    return cases


def trace_files(rng, scale=1):
    """One small trace file per input format the reference reads, as text (scale: times as many traces)."""
    files = {}
    bs = 16

    def chained(n_traces, max_blocks=10):
        seqs, out = [], []
        for _ in range(n_traces):
            n = int(rng.integers(1, max_blocks)) * bs
            toks = rng.integers(0, 50000, size=n).astype(np.int64)
            if seqs and rng.random() < 0.8:
                src = seqs[int(rng.zipf(1.3)) % len(seqs)]
                m = int(rng.integers(0, min(len(src), n) + 1))
                toks[:m] = src[:m]
            seqs.append(toks)
            out.append(oracle.gen_key_vector(toks, bs).tolist())
        return out

    # optimizer_schema: one JSON object per line (kv_cache_manager/optimizer/trace_converter/optimizer_schema_trace.h);
    # dialog turns are replayed, the read and the write line in between are not (this format runs without read/write
    # separation, kv_cache_manager/optimizer/trace_converter/converter_factory.cc:17-29)
    lines, now = [], 1_700_000_000_000_000
    for t, total in enumerate(chained(70 * scale)):
        now += int(rng.integers(0, 3))
        n_in = int(rng.integers(0, len(total) + 1))
        inst = "inst_a" if t % 3 else "inst_b"
        lines.append(json.dumps({"instance_id": inst, "trace_id": "trace_%d" % t, "timestamp_us": now, "tokens": [],
                                 "keys": total[:n_in], "query_type": "prefix_match", "block_mask": 0, "sw_size": 0,
                                 "location_spec_names": [], "input_len": n_in * bs,
                                 "output_len": (len(total) - n_in) * bs, "total_keys": total}))
        if t == 20:
            lines.append(json.dumps({"instance_id": inst, "trace_id": "read", "timestamp_us": now, "tokens": [],
                                     "keys": total, "query_type": "prefix_match", "block_mask": 1, "sw_size": 0,
                                     "location_spec_names": []}))
            lines.append(json.dumps({"instance_id": inst, "trace_id": "write", "timestamp_us": now, "tokens": [],
                                     "keys": total}))
    rng.shuffle(lines)  # the loader sorts by timestamp (stable)
    files["optimizer_schema"] = "\n".join(lines) + "\n"

    # qwen_bailian: chat turns with hash_ids per block (trace_converter/qwen_bailian_converter.cc)
    lines, chats = [], {}
    for t in range(60 * scale):
        chat = int(rng.integers(0, 8 * scale))
        ids = chats.get(chat, []) + rng.integers(1, 1 << 30, size=int(rng.integers(1, 6))).tolist()
        chats[chat] = ids
        lines.append(json.dumps({"chat_id": chat, "parent_chat_id": -1, "timestamp": 1000.0 + 0.5 * (t // 2),
                                 "input_length": 16 * len(ids), "output_length": 16, "type": "text", "turn": t,
                                 "hash_ids": ids}))
    files["qwen_bailian"] = "\n".join(lines) + "\n"

    # publisher_log: the events the manager publishes (trace_converter/publisher_log_converter.cc:34-267): reads,
    # writes opened and finished (or never finished), an event of an instance the configuration does not know
    lines, now, session = [], 1_700_000_000_000_000, 0
    for t, total in enumerate(chained(60 * scale)):
        inst = "inst_a" if t % 2 else "inst_b"
        now += int(rng.integers(1, 50))
        n_in = int(rng.integers(1, len(total) + 1))
        mask = int(rng.integers(0, n_in + 1)) if rng.random() < 0.5 else [bool(b) for b in rng.random(n_in) < 0.3]
        lines.append(json.dumps({"type": "GetCacheLocation", "source": inst, "trigger_time_us": now,
                                 "query_type": "prefix_match", "keys": total[:n_in], "block_mask": mask,
                                 "sw_size": -1, "location_spec_names": []}))
        if rng.random() < 0.85:
            session += 1
            now += int(rng.integers(1, 50))
            lines.append(json.dumps({"type": "StartWriteCache", "source": inst, "trigger_time_us": now,
                                     "write_session_id": "s%d" % session, "keys": total}))
            if rng.random() < 0.8:
                now += int(rng.integers(1, 50))
                lines.append(json.dumps({"type": "FinishWriteCache", "source": inst, "trigger_time_us": now,
                                         "write_session_id": "s%d" % session,
                                         "success_block": int(rng.integers(0, len(total) + 1))}))
        if t == 30:
            lines.append(json.dumps({"type": "GetCacheLocation", "source": "stranger", "trigger_time_us": now,
                                     "query_type": "prefix_match", "keys": total, "block_mask": 0}))
            lines.append("not json at all")
    files["publisher_log"] = "\n".join(lines) + "\n"
    return files


def csv_cases():
    """The reference's optimizer_main path on small trace files: what it writes per instance."""
    rng = np.random.default_rng(0xB2000008)
    files = trace_files(rng)
    out = []
    plans = [("optimizer_schema", [("inst_a", "lru"), ("inst_b", "leaf_aware_lru")], 1, 30),
             ("optimizer_schema", [("inst_a", "leaf_aware_lru"), ("inst_b", "leaf_aware_lru")], 3, 12),
             ("qwen_bailian", [("instance", "lru")], 2, 25),
             ("qwen_bailian", [("instance", "random_lru")], 3, 10),
             ("publisher_log", [("inst_a", "lru"), ("inst_b", "lru")], 1, 40),
             ("publisher_log", [("inst_a", "leaf_aware_lru"), ("inst_b", "lru")], 2, 15)]
    # the last two plans put the instances into groups of their own (usage of the other group's instance still
    # shows in every record), one of them with an instance that no trace names
    plans += [("publisher_log", [[("inst_a", "lru")], [("inst_b", "leaf_aware_lru")]], 3, 20),
              ("optimizer_schema", [[("inst_a", "leaf_aware_lru"), ("idle", "lru")], [("inst_b", "random_lru")]], 1, 18)]
    # a sampling instance and a queueing one share a quota
    plans += [("optimizer_schema", [("inst_a", "random_lru"), ("inst_b", "leaf_aware_lru")], 1, 20),
              ("publisher_log", [("inst_a", "lru"), ("inst_b", "random_lru")], 2, 15)]
    for trace_type, instances, mode, quota in plans:
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "trace.jsonl")
            with open(path, "w") as f:
                f.write(files[trace_type])
            grouped = instances if isinstance(instances[0], list) else [instances]
            config = ref.startup_config([dict(quota_capacity=quota, instances=[(i, p, 0.1) for i, p in members])
                                         for members in grouped],
                                        evict_batch=3, mode=mode, trace_file_path=path, trace_type=trace_type,
                                        output_result_path=os.path.join(tmp, "out"))
            os.makedirs(os.path.join(tmp, "out"), exist_ok=True)
            ref.optimizer_main(config)
            written = {}
            for name in sorted(os.listdir(os.path.join(tmp, "out"))):
                with open(os.path.join(tmp, "out", name)) as f:
                    written[name] = f.read()
            config["trace_file_path"] = "trace.jsonl"
            config["output_result_path"] = "out"
            out.append(dict(trace_type=trace_type, trace_text=files[trace_type], config=config, files=written))
    return out


def main():
    if not ref.available():
        raise SystemExit("oracle/_ref/libkvcm_ref_optimizer.so not built: the reference tree is needed")
    cases = replay_cases()
    with open(os.path.join(HERE, "optimizer_ref_kat.json"), "w") as f:
        json.dump({"generator": "tests/golden/make_optimizer_golden.py",
                   "source": "the reference's Optimizer compiled from its own sources (oracle/_ref)",
                   "trace_types": {"dialog_turn": D, "get_location": G, "write_cache": W}, "cases": cases}, f,
                  separators=(",", ":"))
    csvs = csv_cases()
    with open(os.path.join(HERE, "optimizer_ref_csv.json"), "w") as f:
        json.dump({"generator": "tests/golden/make_optimizer_golden.py",
                   "source": "the reference's optimizer_main path compiled from its own sources (oracle/_ref)",
                   "cases": csvs}, f, separators=(",", ":"))
    print("%d replay workloads (%d runs), %d trace-file cases" % (len(cases), sum(len(c["runs"]) for c in cases),
                                                                 len(csvs)))


if __name__ == "__main__":
    main()
