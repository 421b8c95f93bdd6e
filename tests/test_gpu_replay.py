"""Parity of the two-pass GPU replay with the sequential prefix-tree replay of the oracle."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.optimizer import (TRACE_DIALOG_TURN, TRACE_GET_LOCATION, TRACE_WRITE_CACHE, RunTraces,
                                         replay_workspace_bytes)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gpu(keys, off, types, mask=None, **kw):
    r = RunTraces(torch.tensor(keys, dtype=torch.int64, device=DEV), torch.tensor(off, dtype=torch.int64, device=DEV),
                  torch.tensor(types, dtype=torch.uint8, device=DEV),
                  torch.tensor(mask, dtype=torch.int64, device=DEV) if mask is not None else None, **kw)
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in r]


def test_reference_known_answers():
    # kv_cache_manager/optimizer/test/optimizer_manager_py_test.py:57-84: write [1,2,3], query [1,2,4] -> hit 2;
    # write [1,2] -> write length 2
    ext, inte, wr, size = _gpu([1, 2, 3, 1, 2, 4], [0, 3, 6], [TRACE_WRITE_CACHE, TRACE_GET_LOCATION])
    assert ext.tolist() == [0, 2] and wr.tolist() == [3, 0] and size.tolist() == [3, 3] and inte.tolist() == [0, 0]
    ext, inte, wr, size = _gpu([1, 2], [0, 2], [TRACE_WRITE_CACHE])
    assert wr.tolist() == [2] and ext.tolist() == [0]


def _workload(rng, n_traces, rw_separation):
    """Chained keys of token sequences that share prefixes with earlier ones (Zipf-like reuse)."""
    bs = 16
    seqs, keys, off, types, mask = [], [], [0], [], []
    for t in range(n_traces):
        n = int(rng.integers(0, 40)) * bs + int(rng.integers(0, bs))
        toks = rng.integers(0, 50000, size=n).astype(np.int64)
        if seqs and rng.random() < 0.7:
            src = seqs[int(rng.zipf(1.5)) % len(seqs)]
            m = int(rng.integers(0, min(len(src), n) + 1))
            toks[:m] = src[:m]
        seqs.append(toks)
        k = oracle.gen_key_vector(toks, bs)
        keys.append(k)
        off.append(off[-1] + len(k))
        if rw_separation:
            ty = TRACE_GET_LOCATION if rng.random() < 0.5 else TRACE_WRITE_CACHE
        else:
            ty = TRACE_DIALOG_TURN
        types.append(ty)
        mask.append(int(rng.integers(0, len(k) + 2)) if ty == TRACE_GET_LOCATION and rng.random() < 0.5 else 0)
    return np.concatenate(keys + [np.zeros(0, np.int64)]), np.array(off), np.array(types, np.uint8), np.array(mask)


@pytest.mark.parametrize("rw_separation", [False, True])
def test_random_traces_against_sequential_oracle(rw_separation):
    rng = np.random.default_rng(5 + rw_separation)
    keys, off, types, mask = _workload(rng, 3000, rw_separation)
    want = oracle.Replay().run(keys, off, types, mask)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = _gpu(keys, off, types, mask, status=status)
    for g, w, name in zip(got, want, ["external hits", "internal hits", "written", "cache size"]):
        assert np.array_equal(g, w), name
    assert status[0].item() == 0
    assert want[0].sum() > 0 and want[2].sum() > 0
    if rw_separation:
        assert want[1].sum() > 0


def test_workspace_reuse_and_size_check():
    keys, off, types = [7, 8, 9, 7, 8], [0, 3, 5], [TRACE_DIALOG_TURN, TRACE_DIALOG_TURN]
    ws = torch.empty(replay_workspace_bytes(5), dtype=torch.uint8, device=DEV)
    for _ in range(2):  # the table is cleared by every call
        ext, _, wr, size = _gpu(keys, off, types, workspace=ws)
        assert ext.tolist() == [0, 2] and wr.tolist() == [3, 0] and size.tolist() == [3, 3]
    with pytest.raises(ValueError):
        _gpu(keys, off, types, workspace=ws[:1024])


def test_empty_traces():
    ext, inte, wr, size = _gpu([], [0, 0, 0], [TRACE_DIALOG_TURN, TRACE_GET_LOCATION])
    assert ext.tolist() == [0, 0] and wr.tolist() == [0, 0] and size.tolist() == [0, 0]


def test_vector_masks_with_holes():
    """A BlockMaskVector may mask any keys, not only a leading run (kv_cache_manager/manager/cache_location.cc:9-21):
    hits are still the leading cached keys, each counted as internal when its own bit is set."""
    rng = np.random.default_rng(31)
    keys, off, types, mask = _workload(rng, 1500, True)
    bits = (rng.random(len(keys)) < 0.3).astype(np.uint8)
    got = RunTraces(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), torch.from_numpy(types).to(DEV),
                    torch.from_numpy(mask).to(DEV), mask_bits=torch.from_numpy(bits).to(DEV))
    want = oracle.Replay().run(keys, off, types, mask, mask_bits=bits)
    for a, b in zip(want, got):
        assert np.array_equal(a, b.cpu().numpy())
    plain = oracle.Replay().run(keys, off, types, mask)
    assert not np.array_equal(plain[1], want[1]) and np.array_equal(plain[0] + plain[1], want[0] + want[1])
    # hand-made: write 1..4, then a query of 1..4 with keys 2 and 4 masked
    ext, inte, wr, size = _gpu([1, 2, 3, 4, 1, 2, 3, 4], [0, 4, 8], [TRACE_WRITE_CACHE, TRACE_GET_LOCATION], [0, 0],
                               mask_bits=torch.tensor([0, 0, 0, 0, 0, 1, 0, 1], dtype=torch.uint8, device=DEV))
    assert ext.tolist() == [0, 2] and inte.tolist() == [0, 2]
