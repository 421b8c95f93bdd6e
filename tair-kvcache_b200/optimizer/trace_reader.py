"""Readers of the Optimizer's trace files (host logic) - the formats around the replay loop.

Each reader follows one converter of the reference and yields `Trace` records; `load_traces` then sorts them by
timestamp as OptimizerLoader::LoadTrace does (kv_cache_manager/optimizer/manager/optimizer_loader.cc:14-20).
The reference sorts with std::sort, which is not stable: the library's host helper runs the same routine, so traces
of equal timestamps are replayed in the reference's order too (replay_order below).

  read_qwen_bailian      kv_cache_manager/optimizer/trace_converter/qwen_bailian_converter.cc:10-146
                         (every line is a dialog turn; hash_ids are per-block ids that still need ApplyPrefixHash)
  read_optimizer_schema  kv_cache_manager/optimizer/trace_converter/optimizer_schema_converter.cc:22-78
                         (type inferred from which fields a line has)
  read_publisher_log     kv_cache_manager/optimizer/trace_converter/publisher_log_converter.cc:11-267
                         (GetCacheLocation / StartWriteCache / FinishWriteCache events paired into traces)
"""
import json
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Union

import numpy as np

from .. import _cabi

DIALOG_TURN, GET_LOCATION, WRITE_CACHE = 0, 1, 2  # = TRACE_* of the replay entry point

BlockMask = Union[int, List[bool], None]


@dataclass
class Trace:
    kind: int
    instance_id: str = ""
    timestamp_us: int = 0
    keys: List[int] = field(default_factory=list)         # the keys of the query (reads) or of the write
    total_keys: Optional[List[int]] = None                 # dialog turns: keys replayed (prompt + generated blocks)
    block_mask: BlockMask = None
    query_type: str = "prefix_match"
    needs_prefix_hash: bool = False                        # keys are raw per-block ids (Qwen-Bailian)
    input_len: int = 0
    output_len: int = 0
    order: int = 0                                         # position in the file's replay order (load_traces)

    def replay_keys(self) -> List[int]:
        return self.total_keys if (self.kind == DIALOG_TURN and self.total_keys is not None) else self.keys


def _int_list(value) -> List[int]:
    return [v for v in value if isinstance(v, int) and not isinstance(v, bool)] if isinstance(value, list) else []


def _mask(value) -> BlockMask:
    if isinstance(value, list):
        return [v for v in value if isinstance(v, bool)]
    if isinstance(value, int) and not isinstance(value, bool):
        return value
    return []


def _json_lines(lines: Iterable[str]):
    for line in lines:
        line = line.strip()
        if not line:
            continue
        try:
            doc = json.loads(line)
        except ValueError:
            continue  # the reference logs a warning and skips the line
        if isinstance(doc, dict):
            yield doc


def read_qwen_bailian(lines: Iterable[str]) -> List[Trace]:
    out = []
    for doc in _json_lines(lines):
        ts = doc.get("timestamp")
        out.append(Trace(kind=DIALOG_TURN, instance_id="instance",
                         timestamp_us=int(ts * 1000000) if isinstance(ts, float) else 0,
                         keys=_int_list(doc.get("hash_ids")), needs_prefix_hash=True, block_mask=[],
                         input_len=doc.get("input_length", 0) if isinstance(doc.get("input_length"), int) else 0,
                         output_len=doc.get("output_length", 0) if isinstance(doc.get("output_length"), int) else 0))
    return out


def read_optimizer_schema(lines: Iterable[str]) -> List[Trace]:
    out = []
    for doc in _json_lines(lines):
        base = dict(instance_id=doc.get("instance_id", ""), timestamp_us=doc.get("timestamp_us", 0),
                    keys=_int_list(doc.get("keys", [])))
        if "input_len" in doc and "output_len" in doc and "total_keys" in doc:
            out.append(Trace(kind=DIALOG_TURN, total_keys=_int_list(doc["total_keys"]),
                             block_mask=_mask(doc.get("block_mask")), query_type=doc.get("query_type", "prefix_match"),
                             input_len=doc["input_len"], output_len=doc["output_len"], **base))
        elif "query_type" in doc and "block_mask" in doc and "input_len" not in doc:
            out.append(Trace(kind=GET_LOCATION, block_mask=_mask(doc["block_mask"]), query_type=doc["query_type"],
                             **base))
        else:
            out.append(Trace(kind=WRITE_CACHE, **base))
    return out


def read_publisher_log(lines: Iterable[str], block_sizes: Dict[str, int]) -> List[Trace]:
    """block_sizes: instance_id -> block size; events of other instances are dropped, as the reference does."""
    traces: List[Trace] = []
    pending_gets: List[Trace] = []
    pending_writes: Dict[str, Trace] = {}  # write_session_id -> write trace waiting for its FinishWriteCache
    session_ops: List[tuple] = []          # what happened to that map, in order: (session id, erased?, trace)
    for doc in _json_lines(lines):
        kind = doc.get("type")
        if not isinstance(kind, str):
            continue
        source = doc.get("source") if isinstance(doc.get("source"), str) else ""
        ts = doc.get("trigger_time_us") if isinstance(doc.get("trigger_time_us"), int) else 0
        if kind == "GetCacheLocation":
            if "source" in doc and source not in block_sizes:
                continue
            t = Trace(kind=GET_LOCATION, instance_id=source, timestamp_us=ts, keys=_int_list(doc.get("keys")),
                      query_type=doc.get("query_type", "prefix_match"),
                      block_mask=_mask(doc["block_mask"]) if "block_mask" in doc else [])
            pending_gets.append(t)
            traces.append(t)
        elif kind == "StartWriteCache":
            if "source" in doc and source not in block_sizes:
                continue
            w = Trace(kind=WRITE_CACHE, instance_id=source, timestamp_us=ts, keys=_int_list(doc.get("keys")))
            session = doc.get("write_session_id")
            if isinstance(session, str) and session:
                pending_writes[session] = w
                session_ops.append((session, False, w))
            # the latest earlier GetCacheLocation of the same instance whose keys but the last open the write's keys
            # becomes a dialog turn over the written keys (publisher_log_converter.cc:226-256)
            for i in range(len(pending_gets) - 1, -1, -1):
                g = pending_gets[i]
                if g.instance_id != w.instance_id or g.timestamp_us > w.timestamp_us or not g.keys:
                    continue
                m = len(g.keys) - 1
                if len(w.keys) >= m and g.keys[:m] == w.keys[:m]:
                    bs = block_sizes.get(g.instance_id, 0)
                    traces.append(Trace(kind=DIALOG_TURN, instance_id=g.instance_id, timestamp_us=g.timestamp_us,
                                        keys=list(g.keys), total_keys=list(w.keys), block_mask=g.block_mask,
                                        query_type=g.query_type, input_len=len(g.keys) * bs,
                                        output_len=(len(w.keys) - m) * bs))
                    del pending_gets[i]
                    break
        elif kind == "FinishWriteCache":
            session = doc.get("write_session_id")
            if not isinstance(session, str) or session not in pending_writes:
                continue
            w = pending_writes[session]
            if "source" in doc and (source != w.instance_id or source not in block_sizes):
                continue
            del pending_writes[session]
            session_ops.append((session, True, None))
            if isinstance(doc.get("trigger_time_us"), int):
                w.timestamp_us = doc["trigger_time_us"]
            traces.append(w)
    # never finished: assumed to end 100 ms after it started, appended in the iteration order of the reference's
    # std::unordered_map of sessions (:207-219) - which matters because the sort that follows is not stable
    for w in _in_map_order(session_ops):
        w.timestamp_us += 100000
        traces.append(w)
    for g in pending_gets:  # never followed by a write: replayed as a dialog turn over its own keys (:258-267)
        traces.append(Trace(kind=DIALOG_TURN, instance_id=g.instance_id, timestamp_us=g.timestamp_us,
                            keys=list(g.keys), total_keys=list(g.keys), block_mask=g.block_mask,
                            query_type=g.query_type, input_len=len(g.keys) * block_sizes.get(g.instance_id, 0)))
    return traces


def load_traces(path: str, trace_type: str, block_sizes: Optional[Dict[str, int]] = None) -> List[Trace]:
    """trace_type as in the optimizer config: "qwen_bailian", "optimizer_schema" or "publisher_log"."""
    with open(path) as f:
        if trace_type == "qwen_bailian":
            traces = read_qwen_bailian(f)
        elif trace_type == "optimizer_schema":
            traces = read_optimizer_schema(f)
        elif trace_type == "publisher_log":
            traces = read_publisher_log(f, block_sizes or {})
        else:
            raise ValueError("unknown trace type %r" % trace_type)
    traces = [traces[i] for i in replay_order([t.timestamp_us for t in traces])]
    for position, t in enumerate(traces):
        t.order = position
    return traces


def replay_order(timestamps) -> List[int]:
    """The order OptimizerLoader::LoadTrace puts traces in: std::sort by timestamp
    (kv_cache_manager/optimizer/trace_converter/trace_util.cc:6-8,42-45).  That sort is not stable, and which of
    two traces of one timestamp is replayed first changes hits and evictions, so the library's host helper runs the
    same standard-library routine instead of a stable sort."""
    ts = np.ascontiguousarray(timestamps, dtype=np.int64)
    order = np.empty(len(ts), dtype=np.int64)
    if len(ts):
        _cabi.call("kvcm_b200_trace_replay_order", ts.ctypes.data, len(ts), order.ctypes.data)
    return order.tolist()


def mask_offset(mask: BlockMask, n_keys: int) -> int:
    """The leading masked keys of a block mask: the offset itself, or the run of leading `true`s of a vector
    (kv_cache_manager/manager/cache_location.cc:9-21).  What a vector masks beyond that run is in mask_bits()."""
    if mask is None:
        return 0
    if isinstance(mask, int):
        return min(mask, n_keys)
    m = list(mask)[:n_keys]
    lead = 0
    while lead < len(m) and m[lead]:
        lead += 1
    return lead


def mask_bits(traces: Sequence[Trace], key_off: np.ndarray) -> Optional[np.ndarray]:
    """uint8 per key of the CSR batch, 1 where a GetLocation trace's vector mask masks a key behind its leading
    run (a mask with holes); None when no trace has such a mask, which is the usual case."""
    bits = None
    for i, t in enumerate(traces):
        if t.kind != GET_LOCATION or t.block_mask is None or isinstance(t.block_mask, int):
            continue
        m = [bool(x) for x in list(t.block_mask)[:len(t.keys)]]
        lead = mask_offset(t.block_mask, len(t.keys))
        if any(m[lead:]):
            if bits is None:
                bits = np.zeros(int(key_off[-1]), dtype=np.uint8)
            bits[int(key_off[i]):int(key_off[i]) + len(m)] = m
    return bits


def masked_count(mask: BlockMask, n_keys: int) -> int:
    """Keys a mask covers: what HandleGetLocation records as internal_read_blocks
    (kv_cache_manager/optimizer/manager/optimizer_runner.cc:97-103)."""
    if mask is None:
        return 0
    if isinstance(mask, int):
        return min(mask, n_keys)
    return int(sum(1 for x in list(mask)[:n_keys] if x))


def _in_map_order(session_ops) -> List[Trace]:
    """The traces still in the reference's session map after session_ops, in that map's iteration order."""
    if not session_ops:
        return []
    names = [name.encode() for name, _, _ in session_ops]
    off = np.zeros(len(names) + 1, dtype=np.int64)
    np.cumsum([len(b) for b in names], out=off[1:])
    blob = b"".join(names) + b"\0"
    erase = np.array([1 if erased else 0 for _, erased, _ in session_ops], dtype=np.uint8)
    order = np.empty(len(names), dtype=np.int64)
    left = np.zeros(1, dtype=np.int64)
    import ctypes
    _cabi.call("kvcm_b200_string_map_iteration_order", ctypes.c_char_p(blob), off.ctypes.data, erase.ctypes.data,
               len(names), order.ctypes.data, left.ctypes.data)
    return [session_ops[int(i)][2] for i in order[:int(left[0])]]


def to_csr(traces: Sequence[Trace]):
    """(keys int64, key_off int64, kind uint8, mask_off int64, read_blocks int64) of traces of ONE instance."""
    keys = [np.asarray(t.replay_keys(), dtype=np.int64) for t in traces]
    off = np.zeros(len(traces) + 1, dtype=np.int64)
    np.cumsum([len(k) for k in keys], out=off[1:])
    kind = np.array([t.kind for t in traces], dtype=np.uint8)
    mask = np.array([mask_offset(t.block_mask, len(t.keys)) if t.kind == GET_LOCATION else 0 for t in traces],
                    dtype=np.int64)
    read = np.array([len(t.keys) if t.kind != WRITE_CACHE else 0 for t in traces], dtype=np.int64)
    flat = np.concatenate(keys) if keys else np.zeros(0, dtype=np.int64)
    return flat, off, kind, mask, read


def first_repeat_within_a_trace(keys: np.ndarray, key_off: np.ndarray) -> Optional[int]:
    """Index of a trace in which some key occurs twice, or None.  The eviction-aware replays keep one state per key
    and configuration and walk a trace 32 keys at a time, which is only the reference's tree
    (kv_cache_manager/optimizer/index/radix_tree_index.cc:19-60) when no key repeats inside a trace.  Chained
    hashes never do; keys taken verbatim from a trace file can."""
    n = len(keys)
    if n < 2:
        return None
    trace_of = np.repeat(np.arange(len(key_off) - 1, dtype=np.int64), np.diff(key_off))
    order = np.lexsort((trace_of, keys))  # by key, ties by trace: two occurrences in one trace end up adjacent
    k, t = keys[order], trace_of[order]
    hit = np.flatnonzero((k[1:] == k[:-1]) & (t[1:] == t[:-1]))
    return int(t[hit[0]]) if hit.size else None


def require_no_repeats(traces: Sequence[Trace], keys: np.ndarray, key_off: np.ndarray) -> None:
    """Refuses, before anything is launched, verbatim keys that repeat inside one trace: the eviction-aware sweeps
    would count such a block twice and return wrong curves without noticing."""
    if all(t.needs_prefix_hash for t in traces):
        return  # the chained hash makes every key of a trace distinct
    bad = first_repeat_within_a_trace(np.asarray(keys, dtype=np.int64), np.asarray(key_off, dtype=np.int64))
    if bad is not None:
        raise NotImplementedError("trace %d names the same block key twice; the eviction-aware replay needs keys "
                                  "that do not repeat inside a trace (chained block hashes never do)" % bad)
