"""Trace file -> per-instance replay on the GPU -> hit-rate table, the shape of OptimizerRunner::Run followed by
HitAnalysis::Analyze (kv_cache_manager/optimizer/manager/optimizer_runner.cc:13-68,
kv_cache_manager/optimizer/analysis/result_analysis.cc:10-113): without eviction, or with the "lru" or "leaf_aware_lru" policy at
one or many quota points (the tradeoff curves of kv_cache_manager/optimizer/analysis/script/
tradeoff_curve_by_instances.py)."""
import json
import os
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..manager.hash_util import ApplyPrefixHashBatch
from . import trace_reader as tr
from .replay import RunTraces, RunTracesLru, RunTracesLruGroup

CSV_HEADER = ("TimestampUs,CachedBlocksCurrentInstance,CachedBlocksPerInstance,CachedBlocksAllInstance,"
              "InternalReadBlocks,ExternalReadBlocks,TotalReadBlocks,InternalHitBlocks,"
              "InternalHitRate,ExternalHitBlocks,ExternalHitRate,HitRate,AccInternalHitRate,AccExternalHitRate,"
              "AccHitRate\n")


def _g(x: float) -> str:
    """A double as a C++ ostream prints it by default (6 significant digits)."""
    return "%g" % x


def replay_instance(traces: List[tr.Trace], device, rw_separation: bool = False,
                    quota_blocks: Union[None, int, Sequence[int]] = None, evict_batch: int = 100,
                    precise: bool = False, policy: str = "lru", sample_rate: float = 0.0):
    """Replays the traces of one instance.  As OptimizerRunner::RunTrace does, only prefix_match queries are
    replayed, dialog turns are skipped in read/write-separation mode and Get/Write traces are skipped otherwise.
    quota_blocks = None: nothing is ever evicted; an int: eviction under `policy` ("lru", "leaf_aware_lru" or
    "random_lru" with its `sample_rate`: the instance's eviction_policy_type and eviction_policy_params) at that quota (quota_capacity *
    used_percentage, in blocks); a sequence: one record per quota, all replayed in one launch.  evict_batch and
    precise are eviction_batch_size_per_instance and the eviction mode (False = the rough modes)."""
    keep = _kept(traces, rw_separation)
    keys, off, kind, mask, read = tr.to_csr(keep)
    d_keys, d_off = torch.from_numpy(keys).to(device), torch.from_numpy(off).to(device)
    if any(t.needs_prefix_hash for t in keep):  # Qwen-Bailian ids: chain them first
        d_keys = ApplyPrefixHashBatch(d_keys, d_off)
    ts = np.array([t.timestamp_us for t in keep], dtype=np.int64)
    bits = tr.mask_bits(keep, off)
    d_bits = torch.from_numpy(bits).to(device) if bits is not None else None
    # GetLocation: masked keys are internal reads; a dialog turn reads its query keys externally and replays total_keys
    internal_read = np.array([tr.masked_count(t.block_mask, len(t.keys)) if t.kind == tr.GET_LOCATION else 0
                              for t in keep], dtype=np.int64)
    external_read = np.where(kind == tr.WRITE_CACHE, 0, read - internal_read)

    order = np.array([t.order for t in keep], dtype=np.int64)

    def record(ext, inte, wr, size):
        return dict(timestamp_us=ts, kind=kind, order=order, external_read_blocks=external_read,
                    internal_read_blocks=internal_read, external_hit_blocks=ext, internal_hit_blocks=inte,
                    write_blocks=wr, current_cache_blocks=size)

    d_kind, d_mask = torch.from_numpy(kind).to(device), torch.from_numpy(mask).to(device)
    if quota_blocks is None:
        return record(*(x.cpu().numpy() for x in RunTraces(d_keys, d_off, d_kind, d_mask, mask_bits=d_bits)))
    quotas = [int(quota_blocks)] if np.isscalar(quota_blocks) else [int(q) for q in quota_blocks]
    tr.require_no_repeats(keep, keys, off)
    res = [x.cpu().numpy() for x in RunTracesLru(d_keys, d_off, d_kind, quotas, d_mask, evict_batch, precise,
                                                 mask_bits=d_bits, policy=policy, sample_rate=sample_rate,
                                                 timestamps=torch.from_numpy(ts).to(device))[:4]]
    recs = [record(*(x[c] for x in res)) for c in range(len(quotas))]
    return recs[0] if np.isscalar(quota_blocks) else recs


def _kept(traces: List[tr.Trace], rw_separation: bool) -> List[tr.Trace]:
    """The traces OptimizerRunner::RunTrace replays in the given mode (optimizer_runner.cc:34-68)."""
    keep = []
    for t in traces:
        if t.kind != tr.WRITE_CACHE and t.query_type != "prefix_match":
            continue
        if (t.kind == tr.DIALOG_TURN) == rw_separation:
            continue
        keep.append(t)
    return keep


def replay_group(traces: List[tr.Trace], instance_ids: Sequence[str], device, quota_blocks: int,
                 rw_separation: bool = False, evict_batch: int = 100, mode: int = 1,
                 policy="lru", sample_rate=0.0, timeline: Optional[list] = None) -> Dict[str, Dict[str, np.ndarray]]:
    """Replays the traces of the instances of ONE group that share a quota (every instance under `policy`, or one
    name per instance in the order of `instance_ids`, in any mix; `sample_rate` is one number or one per instance,
    read for "random_lru" instances), in the order given (all instances together, by timestamp), and returns one record per
    instance as replay_instance does.  mode is the configuration's eviction_mode (1 group rough, 2 instance rough, 3 instance precise;
    kv_cache_manager/optimizer/manager/eviction_manager.cc:57-239).  current_cache_blocks is the usage of the
    trace's own instance; blocks_per_instance [record, instance] is the usage of every instance of the group at
    that moment, in the order of `instance_ids` (ReadRecord::blocks_per_instance).  timeline (optional list)
    receives (instance_ids, replay position of every trace of the group, usage of every instance after it)."""
    index = {iid: j for j, iid in enumerate(instance_ids)}
    keep = [t for t in _kept(traces, rw_separation) if t.instance_id in index]
    keys, off, kind, mask, read = tr.to_csr(keep)
    d_keys, d_off = torch.from_numpy(keys).to(device), torch.from_numpy(off).to(device)
    if any(t.needs_prefix_hash for t in keep):
        d_keys = ApplyPrefixHashBatch(d_keys, d_off)
    inst = np.array([index[t.instance_id] for t in keep], dtype=np.int32)
    ts = np.array([t.timestamp_us for t in keep], dtype=np.int64)
    order = np.array([t.order for t in keep], dtype=np.int64)
    bits = tr.mask_bits(keep, off)
    tr.require_no_repeats(keep, keys, off)
    res = RunTracesLruGroup(d_keys, d_off, torch.from_numpy(kind).to(device), torch.from_numpy(inst).to(device),
                            len(instance_ids), [int(quota_blocks)], torch.from_numpy(mask).to(device), evict_batch,
                            mode, mask_bits=torch.from_numpy(bits).to(device) if bits is not None else None,
                            instance_records=True, policy=policy,
                            timestamps=torch.from_numpy(ts).to(device) if policy != "lru" else None,
                            sample_rate=sample_rate)
    ext, inte, wr, size = (x[0].cpu().numpy() for x in res[:4])
    every = res.instance_blocks_per_trace[0].cpu().numpy()  # [trace, instance], instances in the order of instance_ids
    if timeline is not None:
        timeline.append((list(instance_ids), order, every))
    internal_read = np.array([tr.masked_count(t.block_mask, len(t.keys)) if t.kind == tr.GET_LOCATION else 0
                              for t in keep], dtype=np.int64)
    external_read = np.where(kind == tr.WRITE_CACHE, 0, read - internal_read)
    out = {}
    for iid, j in index.items():
        m = inst == j
        out[iid] = dict(timestamp_us=ts[m], kind=kind[m], order=order[m], external_read_blocks=external_read[m],
                        internal_read_blocks=internal_read[m], external_hit_blocks=ext[m],
                        internal_hit_blocks=inte[m], write_blocks=wr[m], current_cache_blocks=size[m],
                        blocks_per_instance=every[m])
    return out


def sweep_hit_rates(traces: List[tr.Trace], device, quota_blocks: Sequence[int], rw_separation: bool = False,
                    evict_batch: int = 100, precise: bool = False, policy: str = "lru") -> np.ndarray:
    """The points of a tradeoff curve without the per-trace records: rows of accumulated (internal, external, total)
    hit rates, one per quota, the same numbers tradeoff_curve() computes from full records."""
    keep = _kept(traces, rw_separation)
    keys, off, kind, mask, read = tr.to_csr(keep)
    d_keys, d_off = torch.from_numpy(keys).to(device), torch.from_numpy(off).to(device)
    if any(t.needs_prefix_hash for t in keep):
        d_keys = ApplyPrefixHashBatch(d_keys, d_off)
    bits = tr.mask_bits(keep, off)
    tr.require_no_repeats(keep, keys, off)
    res = RunTracesLru(d_keys, d_off, torch.from_numpy(kind).to(device), [int(q) for q in quota_blocks],
                       torch.from_numpy(mask).to(device), evict_batch, precise, per_trace=False,
                       mask_bits=torch.from_numpy(bits).to(device) if bits is not None else None, policy=policy,
                       timestamps=torch.from_numpy(np.array([t.timestamp_us for t in keep], dtype=np.int64)).to(device))
    totals = res.totals.cpu().numpy()
    total_read = int(read[kind != tr.WRITE_CACHE].sum())
    out = np.zeros((totals.shape[0], 3))
    if total_read:
        out[:, 0] = totals[:, 1] / total_read
        out[:, 1] = totals[:, 0] / total_read
    out[:, 2] = out[:, 0] + out[:, 1]
    return out


def tradeoff_curve(recs: Sequence[Dict[str, np.ndarray]]) -> np.ndarray:
    """Accumulated hit rates at the end of each replay: rows of (internal, external, total), the three numbers the
    reference's tradeoff scripts read from the last line of every run's CSV
    (kv_cache_manager/optimizer/analysis/script/optimizer_analysis_utils.py:207-270)."""
    out = np.zeros((len(recs), 3))
    for c, rec in enumerate(recs):
        reads = rec["kind"] != tr.WRITE_CACHE
        total = int((rec["internal_read_blocks"][reads] + rec["external_read_blocks"][reads]).sum())
        if total:
            out[c, 0] = int(rec["internal_hit_blocks"][reads].sum()) / total
            out[c, 1] = int(rec["external_hit_blocks"][reads].sum()) / total
        out[c, 2] = out[c, 0] + out[c, 1]
    return out


def export_hit_rates(path: str, rec: Dict[str, np.ndarray]) -> None:
    """`<instance>_hit_rates.csv` of HitAnalysis::ExportHitRates (result_analysis.cc:64-113): one line per read
    record, same columns, separators and number formatting.  A record without blocks_per_instance (an instance
    replayed alone through replay_instance) holds that instance's cached blocks in all three cached-blocks columns;
    with it (run_trace_file, replay_group) CachedBlocksPerInstance lists every instance's usage, ';'-separated, and
    CachedBlocksAllInstance their sum."""
    reads = rec["kind"] != tr.WRITE_CACHE
    acc_total = acc_ext = acc_int = 0
    with open(path, "w") as f:
        f.write(CSV_HEADER)
        for i in np.nonzero(reads)[0]:
            ir, er = int(rec["internal_read_blocks"][i]), int(rec["external_read_blocks"][i])
            ih, eh = int(rec["internal_hit_blocks"][i]), int(rec["external_hit_blocks"][i])
            total = ir + er
            ext_rate = eh / total if total else 0.0
            int_rate = ih / total if total else 0.0
            acc_total, acc_ext, acc_int = acc_total + total, acc_ext + eh, acc_int + ih
            acc_e = acc_ext / acc_total if acc_total else 0.0
            acc_i = acc_int / acc_total if acc_total else 0.0
            cached = int(rec["current_cache_blocks"][i])
            per, total_cached = str(cached), str(cached)
            if "blocks_per_instance" in rec:  # a group of several instances: every instance's usage, ';'-separated
                row = [int(x) for x in rec["blocks_per_instance"][i]]
                per, total_cached = ";".join(str(x) for x in row), str(sum(row))
            f.write(", ".join([str(int(rec["timestamp_us"][i])), str(cached), per, total_cached, str(ir),
                               str(er), str(total), str(ih), _g(int_rate), str(eh), _g(ext_rate),
                               _g(int_rate + ext_rate), _g(acc_i), _g(acc_e), _g(acc_i + acc_e)]) + "\n")


def run_trace_file(trace_path: str, trace_type: str, output_dir: str, device=None,
                   block_sizes: Optional[Dict[str, int]] = None, rw_separation: bool = False,
                   quota_blocks: Union[None, int, Sequence[int], Dict[str, Union[int, Sequence[int]]]] = None,
                   evict_batch: int = 100, precise: bool = False,
                   policy: Union[str, Dict[str, str]] = "lru",
                   groups: Optional[Sequence[dict]] = None, mode: int = 1,
                   sample_rate: Union[float, Dict[str, float]] = 0.0):
    """Loads a trace file, replays every instance on the GPU and writes `<instance>_hit_rates.csv` per instance
    (`<instance>_quota<q>_hit_rates.csv` per instance and quota when quota_blocks is a sequence).  Every instance is
    replayed on its own, except the instances of a group in `groups` (dicts with "instances" = the ids and "quota" =
    the shared quota in blocks, "policy" = the eviction policy of all of them or one per instance, "lru" when
    absent, "sample_rate" = the rates of "random_lru" instances, as parse_startup_config returns them), which are replayed together against their
    shared quota under eviction `mode` (replay_group).  As in the reference, the CachedBlocksPerInstance column of
    every CSV lists the usage of EVERY instance of the configuration at the moment of the record, whichever group it
    belongs to (ReadRecord::blocks_per_instance, kv_cache_manager/optimizer/manager/optimizer_runner.cc:116-124) -
    here in the order of block_sizes (the configuration's order; instance ids sorted when block_sizes is not given),
    in the reference in the order of an unordered_map.  Quota sweeps (a sequence of quotas per instance), which the
    reference does not have, keep the instance's own usage in that column."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    traces = tr.load_traces(trace_path, trace_type, block_sizes)
    by_instance: Dict[str, List[tr.Trace]] = {}
    for t in traces:
        by_instance.setdefault(t.instance_id, []).append(t)
    os.makedirs(output_dir, exist_ok=True)
    out, names, timeline, swept = {}, {}, [], False
    for group in groups or []:
        recs = replay_group(traces, group["instances"], device, group["quota"], rw_separation, evict_batch, mode,
                            group.get("policy", "lru"), group.get("sample_rate", 0.0), timeline)
        for instance_id, r in recs.items():
            by_instance.pop(instance_id, None)
            out[instance_id] = r
            names[instance_id] = [instance_id + "_hit_rates.csv"]
    for instance_id, ts in sorted(by_instance.items()):
        # a dict gives every instance its own quota (or quotas); instances it does not name are never evicted
        quota = quota_blocks.get(instance_id) if isinstance(quota_blocks, dict) else quota_blocks
        sweep = quota is not None and not np.isscalar(quota)
        swept = swept or sweep
        # policy: one name for all instances, or a dict by instance ("lru" for instances it does not name)
        pol = policy.get(instance_id, "lru") if isinstance(policy, dict) else policy
        rate = sample_rate.get(instance_id, 0.0) if isinstance(sample_rate, dict) else sample_rate
        rec = replay_instance(ts, device, rw_separation, quota, evict_batch, precise, pol, rate)
        out[instance_id] = rec
        names[instance_id] = ["%s_quota%d_hit_rates.csv" % (instance_id, int(q)) for q in quota] if sweep else \
            [instance_id + "_hit_rates.csv"]
        if not sweep:
            timeline.append(([instance_id], rec["order"], np.asarray(rec["current_cache_blocks"])[:, None]))
    every = list(block_sizes) if block_sizes else []
    every += [i for i in sorted(out) if i not in every]
    if len(every) > 1 and not swept:
        _usage_of_every_instance(out, timeline, every)
    for instance_id, rec in out.items():
        for name, r in zip(names[instance_id], rec if isinstance(rec, list) else [rec]):
            if (r["kind"] != tr.WRITE_CACHE).any():
                export_hit_rates(os.path.join(output_dir, name), r)
    return out


def _usage_of_every_instance(records: Dict[str, Dict[str, np.ndarray]], timeline, every: List[str]) -> None:
    """Fills blocks_per_instance of every record with the usage of every instance of the configuration at that
    moment: its own replay unit's row, and for the other units (instances replayed alone, groups replayed together)
    the row of their latest trace that was replayed before it.  timeline: (instance ids of a unit, replay positions
    of its traces, usage of its instances after each of them)."""
    column = {iid: k for k, iid in enumerate(every)}
    for rec in records.values():
        rows = np.zeros((len(rec["order"]), len(every)), dtype=np.int64)
        for members, order, usage in timeline:
            at = np.searchsorted(order, rec["order"], side="right") - 1
            seen = np.where(at[:, None] >= 0, np.asarray(usage)[np.maximum(at, 0)], 0)
            for m, iid in enumerate(members):
                rows[:, column[iid]] = seen[:, m]
        rec["blocks_per_instance"] = rows


EVICTION_MODE_UNSPECIFIED, EVICTION_MODE_GROUP_ROUGH, EVICTION_MODE_INSTANCE_ROUGH, EVICTION_MODE_INSTANCE_PRECISE = \
    0, 1, 2, 3  # kv_cache_manager/optimizer/config/types.h


def parse_startup_config(config: Union[str, dict]) -> dict:
    """The Optimizer's startup configuration (kv_cache_manager/optimizer/optimizer_startup_config_load.json, read
    by kv_cache_manager/optimizer/config/optimizer_config.cc:4-12, instance_group_config.cc:5-12,
    instance_config.cc:6-22, eviction_config.cc:5-8) reduced to what the GPU replay needs.  Groups of several
    instances that share a quota come back under "groups", with one policy name for all or one per instance (any
    mix of the three policies).  Raises NotImplementedError for an eviction policy the reference's factory does not
    know either.
    hierarchical_eviction_enabled: the reference creates an eviction policy for the FIRST storage tier only (later
    tiers never evict, kv_cache_manager/optimizer/manager/eviction_manager.cc:26-39), every block gets its location
    on that tier alone (kv_cache_manager/optimizer/index/radix_tree_index.cc:327-353), so erasing that location on
    eviction empties the block as in the shared case; what changes is the capacity the usage is held against:
    storages[0].capacity instead of quota_capacity (eviction_manager.cc:247-258).  That is what is replayed."""
    if isinstance(config, str):
        with open(config) as f:
            config = json.load(f)
    ev = config.get("eviction_params", {})
    mode = int(ev.get("eviction_mode", EVICTION_MODE_UNSPECIFIED))
    if mode not in (EVICTION_MODE_UNSPECIFIED, EVICTION_MODE_GROUP_ROUGH, EVICTION_MODE_INSTANCE_ROUGH,
                    EVICTION_MODE_INSTANCE_PRECISE):
        raise ValueError("unknown eviction_mode %r" % mode)
    quotas, block_sizes, policies, sample_rates, shared = {}, {}, {}, {}, []
    for group in config.get("instance_groups", []):
        instances = group.get("instances", [])
        capacity = group.get("quota_capacity", 0)
        if group.get("hierarchical_eviction_enabled", False):
            if not group.get("storages"):
                raise ValueError("group %r: hierarchical eviction without a storage tier" % group.get("group_name"))
            capacity = group["storages"][0].get("capacity", 0)
        group_quota = int(capacity * float(group.get("used_percentage", 1.0)))
        together = len(instances) > 1 and mode != EVICTION_MODE_UNSPECIFIED
        used = [i.get("eviction_policy_type", "lru") for i in instances]
        if together:
            shared.append(dict(group_name=group.get("group_name"), instances=[str(i["instance_id"]) for i in instances],
                               quota=group_quota, policy=used[0] if len(set(used)) == 1 else used))
            if "random_lru" in used:
                shared[-1]["sample_rate"] = [float((i.get("eviction_policy_params") or {}).get("sample_rate", 0.0))
                                             for i in instances]
        for inst in instances:
            policy = inst.get("eviction_policy_type", "lru")
            if policy not in ("lru", "leaf_aware_lru", "random_lru") and mode != EVICTION_MODE_UNSPECIFIED:
                raise NotImplementedError("instance %r: eviction policy %r is not replayed (\"lru\", "
                                          "\"leaf_aware_lru\" and \"random_lru\" are)"
                                          % (inst.get("instance_id"), policy))
            iid = str(inst["instance_id"])
            policies[iid] = policy
            # RandomLruParams (kv_cache_manager/optimizer/config/instance_config.cc:18-22, eviction_config.h:20-29)
            sample_rates[iid] = float((inst.get("eviction_policy_params") or {}).get("sample_rate", 0.0))
            block_sizes[iid] = int(inst.get("block_size", 16))
            # eviction_manager.cc:249-266: quota = size_t(quota_capacity * used_percentage); an unspecified mode
            # never evicts (:60-63)
            if mode != EVICTION_MODE_UNSPECIFIED and not together:
                quotas[iid] = group_quota
    return dict(trace_file_path=config.get("trace_file_path"), trace_type=config.get("trace_type"),
                output_result_path=config.get("output_result_path"), quota_blocks=quotas, block_sizes=block_sizes,
                evict_batch=int(ev.get("eviction_batch_size_per_instance", 100)),
                precise=mode == EVICTION_MODE_INSTANCE_PRECISE, policies=policies, sample_rates=sample_rates,
                groups=shared, mode=mode)


def run_startup_config(config: Union[str, dict], device=None, rw_separation: Optional[bool] = None):
    """What `optimizer_main <config>` does (kv_cache_manager/optimizer/main.cc; OptimizerRunner::Run +
    HitAnalysis), on the GPU: load the trace the configuration names, replay every instance with its group's
    quota and write `<instance>_hit_rates.csv` under output_result_path.  As the reference's converter factory
    decides it (kv_cache_manager/optimizer/trace_converter/converter_factory.cc:19-28), publisher logs are
    replayed with reads and writes separate and the two dialog-turn formats are not."""
    c = parse_startup_config(config)
    if rw_separation is None:
        rw_separation = c["trace_type"] == "publisher_log"
    return run_trace_file(c["trace_file_path"], c["trace_type"], c["output_result_path"], device, c["block_sizes"],
                          rw_separation, c["quota_blocks"] or None, c["evict_batch"], c["precise"], c["policies"],
                          c["groups"], c["mode"] or 1, c["sample_rates"])
