"""TEST INFRASTRUCTURE ONLY.  ctypes access to the REFERENCE's own Optimizer, compiled from the reference's source
files into oracle/_ref/libkvcm_ref_optimizer.so (oracle/Makefile, target ref_optimizer; oracle/ref_optimizer_driver.cc
is the C-callable wrapper).  Used by tests/ to pin oracle/kvcm_oracle - the restatement the GPU kernels are compared
with - to the reference itself, and by tests/golden/make_optimizer_golden.py to record the reference's answers as
fixtures for boxes where the library is not present.  Nothing in the product path imports this.
"""
import ctypes
import json
import os
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_ref", "libkvcm_ref_optimizer.so")
_lib = None


def available():
    return os.path.exists(_LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(_LIB_PATH)
        L.kvcm_ref_optimizer_create.restype = ctypes.c_void_p
        L.kvcm_ref_optimizer_create.argtypes = [ctypes.c_char_p]
        L.kvcm_ref_optimizer_destroy.argtypes = [ctypes.c_void_p]
        L.kvcm_ref_optimizer_run.restype = ctypes.c_int32
        L.kvcm_ref_optimizer_main.restype = ctypes.c_int32
        L.kvcm_ref_optimizer_main.argtypes = [ctypes.c_char_p]
        _lib = L
    return _lib


def startup_config(groups, evict_batch=100, mode=1, trace_file_path="", trace_type="optimizer_schema",
                   output_result_path=""):
    """The Optimizer's startup configuration (kv_cache_manager/optimizer/optimizer_startup_config_load.json's format)
    as a dict.  groups: dicts with quota_capacity, instances = [(instance_id, policy[, sample_rate[, block_size]])]
    and optionally used_percentage, hierarchical (bool), tier_capacity (capacity of the first storage tier)."""
    out = []
    for g, group in enumerate(groups):
        instances = []
        for inst in group["instances"]:
            iid, policy = inst[0], inst[1]
            rate = inst[2] if len(inst) > 2 else 0.1
            instances.append({"instance_id": str(iid), "block_size": int(inst[3]) if len(inst) > 3 else 16,
                              "eviction_policy_type": policy, "eviction_policy_params": {"sample_rate": float(rate)}})
        out.append({"group_name": group.get("group_name", "group_%02d" % g),
                    "quota_capacity": int(group["quota_capacity"]),
                    "used_percentage": float(group.get("used_percentage", 1.0)),
                    "hierarchical_eviction_enabled": bool(group.get("hierarchical", False)),
                    "storages": [{"unique_name": "tier_0", "storage_type": "pace", "band_width_mbps": 20000,
                                  "priority": 0, "capacity": int(group.get("tier_capacity", 1 << 40))},
                                 {"unique_name": "tier_1", "storage_type": "hf3fs", "band_width_mbps": 20000,
                                  "priority": 1, "capacity": 1 << 40}],
                    "instances": instances})
    return {"trace_file_path": trace_file_path, "trace_type": trace_type, "output_result_path": output_result_path,
            "eviction_params": {"eviction_mode": int(mode), "eviction_batch_size_per_instance": int(evict_batch)},
            "instance_groups": out}


def _write_config(config):
    f = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
    json.dump(config, f)
    f.close()
    return f.name


class RefOptimizer:
    """An OptimizerManager of the reference, fed one trace at a time through its runner's handlers."""

    def __init__(self, groups, evict_batch=100, mode=1):
        config = startup_config(groups, evict_batch, mode)
        self.instance_ids = [i["instance_id"] for g in config["instance_groups"] for i in g["instances"]]
        path = _write_config(config)
        try:
            self._h = ctypes.c_void_p(lib().kvcm_ref_optimizer_create(path.encode()))
        finally:
            os.unlink(path)
        if not self._h:
            raise RuntimeError("the reference's OptimizerManager refused the configuration")

    def __del__(self):
        if getattr(self, "_h", None):
            lib().kvcm_ref_optimizer_destroy(self._h)
            self._h = None

    def run(self, keys, key_off, trace_type, trace_instance=None, mask_off=None, mask_bits=None, timestamps=None):
        """Per trace: external hits, internal hits, written blocks, usage of the trace's instance afterwards, and
        the usage of every instance afterwards ([n_traces, n_instances], instances in configuration order).
        trace_type: 0 dialog turn, 1 GetLocation (prefix match), 2 WriteCache."""
        keys = np.ascontiguousarray(keys, dtype=np.int64)
        key_off = np.ascontiguousarray(key_off, dtype=np.int64)
        n = len(key_off) - 1
        trace_type = np.ascontiguousarray(trace_type, dtype=np.uint8)
        ptr = lambda a, t: a.ctypes.data_as(ctypes.POINTER(t)) if a is not None else None
        inst = np.ascontiguousarray(trace_instance, dtype=np.int32) if trace_instance is not None else None
        mo = np.ascontiguousarray(mask_off, dtype=np.int64) if mask_off is not None else None
        mb = np.ascontiguousarray(mask_bits, dtype=np.uint8) if mask_bits is not None else None
        ts = np.ascontiguousarray(timestamps, dtype=np.int64) if timestamps is not None else None
        ext, inte, wr = (np.zeros(n, dtype=np.int32) for _ in range(3))
        cached = np.zeros(n, dtype=np.int64)
        k = len(self.instance_ids)
        every = np.zeros((max(n, 1), k), dtype=np.int64)[:n]
        ids = (ctypes.c_char_p * k)(*[i.encode() for i in self.instance_ids])
        rc = lib().kvcm_ref_optimizer_run(self._h, ids, ctypes.c_int32(k), ptr(keys, ctypes.c_int64),
                                          ptr(key_off, ctypes.c_int64), ptr(trace_type, ctypes.c_uint8),
                                          ptr(mo, ctypes.c_int64), ptr(mb, ctypes.c_uint8), ptr(ts, ctypes.c_int64),
                                          ptr(inst, ctypes.c_int32), ctypes.c_int64(n), ptr(ext, ctypes.c_int32),
                                          ptr(inte, ctypes.c_int32), ptr(wr, ctypes.c_int32),
                                          ptr(cached, ctypes.c_int64), ptr(every, ctypes.c_int64))
        if rc != 0:
            raise RuntimeError("kvcm_ref_optimizer_run failed with %d" % rc)
        return ext, inte, wr, cached, every


def load_traces(config):
    """The traces the reference's loader makes of the configuration's trace file, in its replay order: a list of
    (kind, dict) with kind 0 dialog turn, 1 GetLocation, 2 WriteCache and the trace's own JSON as a dict."""
    path = config if isinstance(config, str) else _write_config(config)
    out = tempfile.NamedTemporaryFile("w", suffix=".traces", delete=False)
    out.close()
    try:
        lib().kvcm_ref_optimizer_dump_traces.restype = ctypes.c_int64
        n = lib().kvcm_ref_optimizer_dump_traces(path.encode(), out.name.encode())
        if n < 0:
            raise RuntimeError("the reference's loader failed")
        with open(out.name) as f:
            rows = [line.split(" ", 1) for line in f.read().splitlines()]
    finally:
        os.unlink(out.name)
        if not isinstance(config, str):
            os.unlink(path)
    return [(int(kind), json.loads(doc)) for kind, doc in rows]


def optimizer_main(config):
    """What the reference's `optimizer_main <config>` does: load the trace file the configuration names, replay it,
    write `<instance>_hit_rates.csv` per instance under output_result_path.  config: a dict or a path."""
    path = config if isinstance(config, str) else _write_config(config)
    try:
        rc = lib().kvcm_ref_optimizer_main(path.encode())
    finally:
        if not isinstance(config, str):
            os.unlink(path)
    if rc != 0:
        raise RuntimeError("the reference's optimizer_main path failed with %d" % rc)
