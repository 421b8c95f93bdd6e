"""Batched twin of the Optimizer's trace replay loop (kv_cache_manager/optimizer/manager)."""
from .replay import (EVICTION_MODE_GROUP_ROUGH, EVICTION_MODE_INSTANCE_PRECISE,  # noqa: F401
                     EVICTION_MODE_INSTANCE_ROUGH, TRACE_DIALOG_TURN, TRACE_GET_LOCATION, TRACE_WRITE_CACHE,
                     LruGroupSweepResult, LruSweepResult, ReplayResult, RunTraces, RunTracesLru, RunTracesLruGroup,
                     replay_lru_workspace_bytes, replay_workspace_bytes)
from . import trace_reader  # noqa: F401
from .runner import (export_hit_rates, parse_startup_config, replay_group, replay_instance,  # noqa: F401
                     run_startup_config, run_trace_file, sweep_hit_rates, tradeoff_curve)
