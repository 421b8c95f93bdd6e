"""Trace replay on the GPU, no eviction.

RunTraces is the batched twin of OptimizerRunner::RunTraces
(kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215): every trace of one instance in one
call, results as the per-trace numbers the reference keeps in ReadRecord / WriteRecord
(kv_cache_manager/optimizer/analysis/result_structure.h:6-33).
"""
from typing import NamedTuple, Optional

import torch

from .. import _cabi

TRACE_DIALOG_TURN, TRACE_GET_LOCATION, TRACE_WRITE_CACHE = 0, 1, 2


class ReplayResult(NamedTuple):
    external_hit_blocks: torch.Tensor  # int32 per trace
    internal_hit_blocks: torch.Tensor  # int32 per trace (masked keys that were cached)
    write_blocks: torch.Tensor         # int32 per trace
    current_cache_blocks: torch.Tensor  # int64 per trace, after the trace


def replay_workspace_bytes(n_keys_total: int) -> int:
    n = _cabi.lib().kvcm_b200_replay_workspace_bytes(n_keys_total)
    if n < 0:
        raise ValueError("too many keys for one replay call")
    return n


def _mask_bits_ptr(mask_bits: Optional[torch.Tensor], keys: torch.Tensor):
    if mask_bits is None:
        return None
    if mask_bits.dtype != torch.uint8 or mask_bits.numel() != keys.numel() or mask_bits.device != keys.device:
        raise ValueError("mask_bits must be a uint8 tensor with one entry per key, on the keys' device")
    return mask_bits.contiguous().data_ptr()


def RunTraces(keys: torch.Tensor, key_off: torch.Tensor, trace_type: torch.Tensor,
              mask_off: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
              status: Optional[torch.Tensor] = None, mask_bits: Optional[torch.Tensor] = None) -> ReplayResult:
    """keys: int64 CUDA tensor of chained block keys, CSR by key_off (int64, n_traces + 1), traces in replay
    (timestamp) order; trace_type: uint8 per trace (TRACE_*); mask_off: int64 per trace for GetLocation traces
    (BlockMaskOffset); mask_bits: optional uint8 per key, 1 = masked (a BlockMaskVector, holes allowed).
    workspace: optional uint8 CUDA tensor of replay_workspace_bytes(keys.numel()) bytes to reuse across calls."""
    if not keys.is_cuda:
        raise ValueError("keys must be a CUDA tensor: this path has no CPU implementation")
    dev = keys.device
    keys, key_off, trace_type = keys.contiguous(), key_off.contiguous(), trace_type.contiguous()
    n_traces = key_off.numel() - 1
    need = replay_workspace_bytes(keys.numel())
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    elif workspace.numel() < need or workspace.device != dev:
        raise ValueError("workspace too small: %d < %d bytes" % (workspace.numel(), need))
    ext = torch.empty(max(n_traces, 1), dtype=torch.int32, device=dev)
    inte = torch.empty_like(ext)
    wr = torch.empty_like(ext)
    size = torch.empty(max(n_traces, 1), dtype=torch.int64, device=dev)
    _cabi.bind_device(dev.index)
    _cabi.call("kvcm_b200_replay", keys.data_ptr(), key_off.data_ptr(), trace_type.data_ptr(),
               mask_off.contiguous().data_ptr() if mask_off is not None else None, _mask_bits_ptr(mask_bits, keys),
               n_traces, keys.numel(), workspace.data_ptr(), workspace.numel(), ext.data_ptr(), inte.data_ptr(),
               wr.data_ptr(),
               size.data_ptr(), status.data_ptr() if status is not None else None,
               torch.cuda.current_stream(dev).cuda_stream)
    return ReplayResult(ext[:n_traces], inte[:n_traces], wr[:n_traces], size[:n_traces])


class LruSweepResult(NamedTuple):
    external_hit_blocks: Optional[torch.Tensor]   # int32 [n_configs, n_traces]; None with per_trace=False
    internal_hit_blocks: Optional[torch.Tensor]   # int32 [n_configs, n_traces]
    write_blocks: Optional[torch.Tensor]          # int32 [n_configs, n_traces]
    current_cache_blocks: Optional[torch.Tensor]  # int64 [n_configs, n_traces], after the trace (and its eviction)
    totals: torch.Tensor  # int64 [n_configs, 4]: external hits, internal hits, written blocks, cached blocks at the end


POLICIES = ("lru", "leaf_aware_lru", "random_lru")  # EvictionPolicyType names (kv_cache_manager/optimizer/config/types.cc)


def replay_lru_workspace_bytes(n_keys_total: int, n_configs: int, policy: str = "lru", n_traces: int = 0) -> int:
    if policy == "leaf_aware_lru":
        n = _cabi.lib().kvcm_b200_replay_leaf_lru_workspace_bytes(n_keys_total, n_traces, n_configs)
    elif policy == "lru":
        n = _cabi.lib().kvcm_b200_replay_lru_workspace_bytes(n_keys_total, n_configs)
    elif policy == "random_lru":
        n = _cabi.lib().kvcm_b200_replay_random_lru_workspace_bytes(n_keys_total, n_configs)
    else:
        raise ValueError("eviction policy %r is not built (have: %s)" % (policy, ", ".join(POLICIES)))
    if n < 0:
        raise ValueError("too many keys or configurations for one LRU replay call")
    return n


def RunTracesLru(keys: torch.Tensor, key_off: torch.Tensor, trace_type: torch.Tensor, quota_blocks,
                 mask_off: Optional[torch.Tensor] = None, evict_batch: int = 100, precise: bool = False,
                 workspace: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                 per_trace: bool = True, mask_bits: Optional[torch.Tensor] = None, policy: str = "lru",
                 timestamps: Optional[torch.Tensor] = None, sample_rate: float = 0.0) -> LruSweepResult:
    """The replay of RunTraces with the reference's "lru" (default), "leaf_aware_lru" or "random_lru" eviction
    policy (policy; timestamps = the traces' timestamp_us as an int64 CUDA tensor, read by "leaf_aware_lru" and
    "random_lru", the trace number when None; sample_rate = RandomLruParams.sample_rate of "random_lru", 0.1 when
    <= 0 as in the reference), once per entry of quota_blocks (the
    points of a tradeoff curve: quota_capacity * used_percentage in blocks), all configurations in one launch.
    evict_batch / precise: eviction_batch_size_per_instance and the eviction mode (False = the rough modes, which
    evict whole batches; True = INSTANCE_PRECISE).  per_trace=False skips the [n_configs, n_traces] records and
    returns only the totals per configuration (what a tradeoff curve reads)."""
    if not keys.is_cuda:
        raise ValueError("keys must be a CUDA tensor: this path has no CPU implementation")
    dev = keys.device
    keys, key_off, trace_type = keys.contiguous(), key_off.contiguous(), trace_type.contiguous()
    quota = torch.as_tensor(quota_blocks, dtype=torch.int64).reshape(-1).to(dev).contiguous()
    n_cfg, n_traces = quota.numel(), key_off.numel() - 1
    if n_cfg == 0:
        raise ValueError("quota_blocks is empty")
    need = replay_lru_workspace_bytes(keys.numel(), n_cfg, policy, n_traces)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    elif workspace.numel() < need or workspace.device != dev:
        raise ValueError("workspace too small: %d < %d bytes" % (workspace.numel(), need))
    totals = torch.zeros((n_cfg, 4), dtype=torch.int64, device=dev)
    ext = inte = wr = size = None
    if per_trace:
        # the C entry point lays its outputs out as [n_configs][n_traces]
        ext = torch.empty((n_cfg, n_traces), dtype=torch.int32, device=dev)
        inte, wr = torch.empty_like(ext), torch.empty_like(ext)
        size = torch.empty((n_cfg, n_traces), dtype=torch.int64, device=dev)
    ptr = (lambda t: t.data_ptr() if t is not None and t.numel() > 0 else None)
    if per_trace and n_traces == 0:
        return LruSweepResult(ext, inte, wr, size, totals)
    _cabi.bind_device(dev.index)
    if policy in ("leaf_aware_lru", "random_lru") and timestamps is not None:
        if timestamps.dtype != torch.int64 or timestamps.numel() != n_traces or timestamps.device != dev:
            raise ValueError("timestamps must be an int64 tensor with one entry per trace, on the keys' device")
        timestamps = timestamps.contiguous()
    if policy == "random_lru":
        _cabi.call("kvcm_b200_replay_random_lru", keys.data_ptr(), key_off.data_ptr(), trace_type.data_ptr(),
                   mask_off.contiguous().data_ptr() if mask_off is not None else None,
                   _mask_bits_ptr(mask_bits, keys), timestamps.data_ptr() if timestamps is not None else None,
                   n_traces, keys.numel(), quota.data_ptr(), n_cfg, int(evict_batch), 1 if precise else 0,
                   float(sample_rate), workspace.data_ptr(), workspace.numel(), ptr(ext), ptr(inte), ptr(wr),
                   ptr(size), totals.data_ptr(), status.data_ptr() if status is not None else None,
                   torch.cuda.current_stream(dev).cuda_stream)
        return LruSweepResult(ext, inte, wr, size, totals)
    if policy == "leaf_aware_lru":
        _cabi.call("kvcm_b200_replay_leaf_lru", keys.data_ptr(), key_off.data_ptr(), trace_type.data_ptr(),
                   mask_off.contiguous().data_ptr() if mask_off is not None else None,
                   _mask_bits_ptr(mask_bits, keys), timestamps.data_ptr() if timestamps is not None else None,
                   n_traces, keys.numel(), quota.data_ptr(), n_cfg, int(evict_batch), 1 if precise else 0,
                   workspace.data_ptr(), workspace.numel(), ptr(ext), ptr(inte), ptr(wr), ptr(size),
                   totals.data_ptr(), status.data_ptr() if status is not None else None,
                   torch.cuda.current_stream(dev).cuda_stream)
        return LruSweepResult(ext, inte, wr, size, totals)
    _cabi.call("kvcm_b200_replay_lru", keys.data_ptr(), key_off.data_ptr(), trace_type.data_ptr(),
               mask_off.contiguous().data_ptr() if mask_off is not None else None, _mask_bits_ptr(mask_bits, keys),
               n_traces, keys.numel(), quota.data_ptr(), n_cfg, int(evict_batch), 1 if precise else 0, workspace.data_ptr(),
               workspace.numel(), ptr(ext), ptr(inte), ptr(wr), ptr(size), totals.data_ptr(),
               status.data_ptr() if status is not None else None, torch.cuda.current_stream(dev).cuda_stream)
    return LruSweepResult(ext, inte, wr, size, totals)


EVICTION_MODE_GROUP_ROUGH, EVICTION_MODE_INSTANCE_ROUGH, EVICTION_MODE_INSTANCE_PRECISE = 1, 2, 3


class LruGroupSweepResult(NamedTuple):
    external_hit_blocks: Optional[torch.Tensor]   # int32 [n_configs, n_traces]; None with per_trace=False
    internal_hit_blocks: Optional[torch.Tensor]
    write_blocks: Optional[torch.Tensor]
    current_cache_blocks: Optional[torch.Tensor]  # int64 [n_configs, n_traces]: usage of the trace's own instance
    totals: torch.Tensor           # int64 [n_configs, 4]: hits ext / int, written blocks, usage of the group at the end
    instance_blocks: torch.Tensor  # int64 [n_configs, n_instances]: usage of every instance at the end
    # int64 [n_configs, n_traces, n_instances]: usage of every instance after each trace (with instance_records=True)
    instance_blocks_per_trace: Optional[torch.Tensor] = None


def RunTracesLruGroup(keys: torch.Tensor, key_off: torch.Tensor, trace_type: torch.Tensor,
                      trace_instance: torch.Tensor, n_instances: int, quota_blocks,
                      mask_off: Optional[torch.Tensor] = None, evict_batch: int = 100,
                      mode: int = EVICTION_MODE_GROUP_ROUGH, workspace: Optional[torch.Tensor] = None,
                      status: Optional[torch.Tensor] = None, per_trace: bool = True,
                      mask_bits: Optional[torch.Tensor] = None, instance_records: bool = False,
                      policy="lru", timestamps: Optional[torch.Tensor] = None,
                      sample_rate=0.0) -> LruGroupSweepResult:
    """The "lru" (default) or "leaf_aware_lru" sweep for an instance group whose instances share one quota
    (kv_cache_manager/optimizer/manager/eviction_manager.cc:86-266): trace_instance (int32 per trace, values in
    [0, n_instances)) names each trace's instance, the traces of all instances come in one replay order, and the
    same key in two instances is two blocks.  mode is the reference's eviction_mode: GROUP_ROUGH takes rounds of
    evict_batch blocks from every instance, the INSTANCE modes take from the writing instance only.
    instance_records=True also returns the usage of every instance after each trace (the reference's
    ReadRecord::blocks_per_instance, which fills two columns of its hit-rate CSV).  policy is the
    eviction_policy_type of every instance of the group, or a sequence with one name per instance (a group may mix
    "lru", "leaf_aware_lru" and "random_lru" as the reference's configuration may; sample_rate is one number or one
    per instance and is read for the "random_lru" instances); timestamps (int64 per trace, the traces'
    timestamp_us) is read by "leaf_aware_lru" instances, which order re-queued blocks by it, and by "random_lru"
    ones, which pick the oldest of their samples (the trace number when None)."""
    each = [policy] * int(n_instances) if isinstance(policy, str) else list(policy)
    sampling = set(each) == {"random_lru"}  # nothing but sampling instances: no tree is kept
    if len(each) != int(n_instances) or any(e not in ("lru", "leaf_aware_lru", "random_lru") for e in each):
        raise ValueError("eviction policies %r: one of \"lru\", \"leaf_aware_lru\", \"random_lru\" for the group or "
                         "one per instance" % (policy,))
    rates = [sample_rate] * len(each) if isinstance(sample_rate, (int, float)) else list(sample_rate)
    if len(rates) != len(each):
        raise ValueError("sample_rate: one number, or one per instance")
    if not keys.is_cuda:
        raise ValueError("keys must be a CUDA tensor: this path has no CPU implementation")
    dev = keys.device
    keys, key_off, trace_type = keys.contiguous(), key_off.contiguous(), trace_type.contiguous()
    quota = torch.as_tensor(quota_blocks, dtype=torch.int64).reshape(-1).to(dev).contiguous()
    n_cfg, n_traces = quota.numel(), key_off.numel() - 1
    if n_cfg == 0:
        raise ValueError("quota_blocks is empty")
    if trace_instance.dtype != torch.int32 or trace_instance.numel() != n_traces or trace_instance.device != dev:
        raise ValueError("trace_instance must be an int32 tensor with one entry per trace, on the keys' device")
    trace_instance = trace_instance.contiguous()
    # one leaf-aware instance, or a sampling instance beside others, and the group needs the kernel that keeps trees
    leaf = not sampling and any(e != "lru" for e in each)
    import ctypes
    codes = {"lru": _cabi.POLICY_LRU, "leaf_aware_lru": _cabi.POLICY_LEAF_AWARE_LRU, "random_lru": _cabi.POLICY_RANDOM_LRU}
    policy_bytes = (ctypes.c_uint8 * len(each))(*[codes[e] for e in each])
    rate_doubles = (ctypes.c_double * len(each))(*[float(r) for r in rates])
    if leaf:
        need = _cabi.lib().kvcm_b200_replay_policy_group_workspace_bytes(
            keys.numel(), n_traces, n_cfg, ctypes.cast(policy_bytes, ctypes.c_void_p), int(n_instances))
    elif sampling:
        need = _cabi.lib().kvcm_b200_replay_random_lru_group_workspace_bytes(keys.numel(), n_cfg, int(n_instances))
    else:
        need = _cabi.lib().kvcm_b200_replay_lru_group_workspace_bytes(keys.numel(), n_cfg, int(n_instances))
    if need < 0:
        raise ValueError("too many keys, configurations or instances for one group replay call")
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    elif workspace.numel() < need or workspace.device != dev:
        raise ValueError("workspace too small: %d < %d bytes" % (workspace.numel(), need))
    totals = torch.zeros((n_cfg, 4), dtype=torch.int64, device=dev)
    inst = torch.zeros((n_cfg, int(n_instances)), dtype=torch.int64, device=dev)
    ext = inte = wr = size = None
    if per_trace:
        ext = torch.empty((n_cfg, n_traces), dtype=torch.int32, device=dev)
        inte, wr = torch.empty_like(ext), torch.empty_like(ext)
        size = torch.empty((n_cfg, n_traces), dtype=torch.int64, device=dev)
    ptr = (lambda t: t.data_ptr() if t is not None and t.numel() > 0 else None)
    per_inst = None
    if instance_records:
        per_inst = torch.zeros((n_cfg, n_traces, int(n_instances)), dtype=torch.int64, device=dev)
    if n_traces == 0:
        return LruGroupSweepResult(ext, inte, wr, size, totals, inst, per_inst)
    _cabi.bind_device(dev.index)
    if (leaf or sampling) and timestamps is not None:
        if timestamps.dtype != torch.int64 or timestamps.numel() != n_traces or timestamps.device != dev:
            raise ValueError("timestamps must be an int64 tensor with one entry per trace, on the keys' device")
        timestamps = timestamps.contiguous()
    if sampling:
        _cabi.call("kvcm_b200_replay_random_lru_group", keys.data_ptr(), key_off.data_ptr(), trace_type.data_ptr(),
                   mask_off.contiguous().data_ptr() if mask_off is not None else None, _mask_bits_ptr(mask_bits, keys),
                   timestamps.data_ptr() if timestamps is not None else None, trace_instance.data_ptr(),
                   ctypes.cast(rate_doubles, ctypes.c_void_p), int(n_instances), n_traces, keys.numel(),
                   quota.data_ptr(), n_cfg, int(evict_batch), int(mode), workspace.data_ptr(), workspace.numel(),
                   ptr(ext), ptr(inte), ptr(wr), ptr(size), totals.data_ptr(), inst.data_ptr(), ptr(per_inst),
                   status.data_ptr() if status is not None else None, torch.cuda.current_stream(dev).cuda_stream)
        return LruGroupSweepResult(ext, inte, wr, size, totals, inst, per_inst)
    if leaf:
        _cabi.call("kvcm_b200_replay_policy_group", keys.data_ptr(), key_off.data_ptr(), trace_type.data_ptr(),
                   mask_off.contiguous().data_ptr() if mask_off is not None else None, _mask_bits_ptr(mask_bits, keys),
                   timestamps.data_ptr() if timestamps is not None else None, trace_instance.data_ptr(),
                   ctypes.cast(policy_bytes, ctypes.c_void_p), ctypes.cast(rate_doubles, ctypes.c_void_p),
                   int(n_instances), n_traces, keys.numel(), quota.data_ptr(), n_cfg, int(evict_batch), int(mode),
                   workspace.data_ptr(), workspace.numel(), ptr(ext), ptr(inte), ptr(wr), ptr(size), totals.data_ptr(),
                   inst.data_ptr(), ptr(per_inst), status.data_ptr() if status is not None else None,
                   torch.cuda.current_stream(dev).cuda_stream)
        return LruGroupSweepResult(ext, inte, wr, size, totals, inst, per_inst)
    _cabi.call("kvcm_b200_replay_lru_group_records", keys.data_ptr(), key_off.data_ptr(), trace_type.data_ptr(),
               mask_off.contiguous().data_ptr() if mask_off is not None else None, _mask_bits_ptr(mask_bits, keys),
               trace_instance.data_ptr(), int(n_instances), n_traces, keys.numel(), quota.data_ptr(), n_cfg,
               int(evict_batch), int(mode), workspace.data_ptr(), workspace.numel(), ptr(ext), ptr(inte), ptr(wr),
               ptr(size), totals.data_ptr(), inst.data_ptr(), ptr(per_inst),
               status.data_ptr() if status is not None else None, torch.cuda.current_stream(dev).cuda_stream)
    return LruGroupSweepResult(ext, inte, wr, size, totals, inst, per_inst)
