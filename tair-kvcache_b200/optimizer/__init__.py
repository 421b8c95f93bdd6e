"""Batched twin of the Optimizer's trace replay loop (kv_cache_manager/optimizer/manager)."""
from .replay import (TRACE_DIALOG_TURN, TRACE_GET_LOCATION, TRACE_WRITE_CACHE, LruSweepResult,  # noqa: F401
                     ReplayResult, RunTraces, RunTracesLru, replay_lru_workspace_bytes, replay_workspace_bytes)
from . import trace_reader  # noqa: F401
from .runner import (export_hit_rates, parse_startup_config, replay_instance, run_startup_config,  # noqa: F401
                     run_trace_file, sweep_hit_rates, tradeoff_curve)
