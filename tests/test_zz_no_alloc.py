"""kvcm_b200_replay_noalloc: the replay for embedders that may not allocate device memory.

An engine plugin that runs after the engine has taken almost all of HBM cannot count on a cudaMalloc
succeeding (and a successful one stalls the engine's streams), so this entry point keeps its scratch table
in a fixed array inside the library.  The test drives it through the C ABI only and checks, twice in a row
with different traces, that it returns exactly what kvcm_b200_replay returns with caller-provided scratch -
the second call runs over whatever the first one left in the shared array - and what the CPU oracle's
sequential prefix-tree replay returns for the same traces.  It also reads the device's free memory before and
after the second call: the entry point exists for callers that must not allocate, so the figure may not move.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _traces(seed, n_traces):
    """Dialog-turn / get / write traces over chained-looking keys with shared prefixes."""
    rng = np.random.default_rng(seed)
    seqs, off, types, mask = [], [0], [], []
    for _ in range(n_traces):
        n = int(rng.integers(0, 60))
        k = rng.integers(-(1 << 62), 1 << 62, size=n, dtype=np.int64)
        if seqs and rng.random() < 0.7:
            src = seqs[int(rng.integers(0, len(seqs)))]
            m = int(rng.integers(0, min(len(src), n) + 1))
            k[:m] = src[:m]
        seqs.append(k)
        off.append(off[-1] + n)
        ty = int(rng.integers(0, 3))
        types.append(ty)
        mask.append(int(rng.integers(0, n + 1)) if ty == 1 else 0)
    keys = np.concatenate(seqs + [np.zeros(0, np.int64)])
    return keys, np.array(off, np.int64), np.array(types, np.uint8), np.array(mask, np.int64)


def _outputs(n):
    return [torch.full((max(n, 1),), -7, dtype=torch.int32, device=DEV) for _ in range(3)] + \
           [torch.full((max(n, 1),), -7, dtype=torch.int64, device=DEV)]


def _free_bytes():
    free = ctypes.c_int64()
    _cabi.call("kvcm_b200_device_info", None, None, ctypes.byref(free), None)
    return free.value


def _run_both(seed, n_traces, check_free=False):
    keys, off, types, mask = _traces(seed, n_traces)
    d = [torch.from_numpy(a).to(DEV) for a in (keys, off, types, mask)]
    stream = torch.cuda.current_stream().cuda_stream
    _cabi.bind_device(0)
    # existing entry point, scratch owned by the caller
    ws = torch.empty(_cabi.lib().kvcm_b200_replay_workspace_bytes(len(keys)), dtype=torch.uint8, device=DEV)
    want = _outputs(n_traces)
    _cabi.call("kvcm_b200_replay", d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(), None, n_traces,
               len(keys), ws.data_ptr(), ws.numel(), want[0].data_ptr(), want[1].data_ptr(), want[2].data_ptr(),
               want[3].data_ptr(), None, stream)
    # new entry point, nothing allocated by the library
    got = _outputs(n_traces)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    free_before = _free_bytes()
    _cabi.call("kvcm_b200_replay_noalloc", d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
               n_traces, len(keys), got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(), got[3].data_ptr(),
               status.data_ptr(), stream)
    torch.cuda.synchronize()
    if check_free:  # the device's set-up happened in an earlier call: this one may not take a byte
        assert _free_bytes() == free_before
    names = ["external hits", "internal hits", "written blocks", "cache size"]
    for g, w, name in zip(got, want, names):
        assert torch.equal(g[:n_traces], w[:n_traces]), name  # integer results: exact equality
    cpu = oracle.Replay().run(keys, off, types, mask_off=mask)
    for g, c, name in zip(got, cpu, names):
        assert np.array_equal(g[:n_traces].cpu().numpy(), c), name + " (oracle)"
    assert status[0].item() == 0
    assert int(want[0].sum()) > 0 and int(want[2].sum()) > 0
    return len(keys)


def test_noalloc_replay_equals_replay_on_two_calls_in_a_row():
    n1 = _run_both(seed=1, n_traces=4000)   # ~118k keys: most of the fixed table
    n2 = _run_both(seed=2, n_traces=700, check_free=True)  # smaller table laid over the first call's leftovers
    assert n2 < n1 <= _cabi.REPLAY_NOALLOC_MAX_KEYS


def test_noalloc_replay_rejects_sizes_beyond_its_fixed_table():
    _cabi.bind_device(0)
    t = torch.zeros(8, dtype=torch.int64, device=DEV)
    rc = _cabi.lib().kvcm_b200_replay_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), None, 1,
                                              _cabi.REPLAY_NOALLOC_MAX_KEYS + 1, t.data_ptr(), t.data_ptr(),
                                              t.data_ptr(), None, None, None)
    assert rc == _cabi.KVCM_EC_OUT_OF_LIMIT
    assert "fixed limit" in _cabi.error_string(rc)
