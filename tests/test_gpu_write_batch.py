"""StartWriteCache / FinishWriteCache for a batch of requests (kvcm_b200_start_write / kvcm_b200_finish_write) against
the oracle serving the same requests ONE AFTER THE OTHER in batch order, which is what the reference does
(CacheManager::StartWriteCache = FilterWriteCache + BatchAddLocation per request, FinishWriteCache per session:
kv_cache_manager/manager/cache_manager.cc:334-501,589-635).  The oracle's filter_write, add_location and
update_status are themselves compared with the reference's own MetaSearcher in
tests/test_matchers_reference_pins.py."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi
from tair_kvcache_b200.manager import BatchMetaSearcher, BlockIndex, encode_locations
from tair_kvcache_b200.manager.block_index import avail_mask_from_weights
from test_gpu_index_write import _check_against_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
W, S = oracle.CLS_WRITING, oracle.CLS_SERVING


def _csr(reqs):
    off = np.zeros(len(reqs) + 1, dtype=np.int64)
    np.cumsum([len(r) for r in reqs], out=off[1:])
    return np.concatenate(reqs + [np.zeros(0, np.int64)]).astype(np.int64), off


def _sequential_start(ox, reqs, cls, weights):
    """The reference's order of events: request after request, filter then add."""
    out = []
    for r in reqs:
        kind, what, n_new = ox.filter_write(r, weights=weights)
        new = r[what:] if kind == "offset" else r[~what]
        ox.add_location(new, cls, W)
        out.append((kind, what, n_new, new))
    return out


def _compare_start(sessions, reqs, off, want):
    offset, mask, n_new, added = (t.cpu().numpy() for t in sessions[:4])
    new_off = sessions.new_off.cpu().numpy()
    kinds = set()
    for r, (kind, what, n, new) in enumerate(want):
        a, b = off[r], off[r + 1]
        kinds.add(kind)
        assert n_new[r] == n, r
        if kind == "offset":
            assert offset[r] == what, r
        else:
            assert offset[r] == -1 and np.array_equal(mask[a:b].astype(bool), what), r
        assert np.array_equal(reqs[r][added[a:b].astype(bool)], new), r      # the session: the new keys, in order
        assert new_off[r + 1] - new_off[r] == len(new)
    return kinds


def _requests(rng, universe, n_req, max_len):
    """Requests that share prefixes and single keys with each other and with what the index holds."""
    reqs = []
    for _ in range(n_req):
        n = int(rng.integers(0, max_len))
        r = rng.choice(universe, size=n, replace=False)
        if reqs and rng.random() < 0.7:
            src = reqs[int(rng.integers(len(reqs)))]
            m = int(rng.integers(0, min(len(src), n) + 1))
            keep = r[~np.isin(r, src[:m])]
            r = np.concatenate([src[:m], keep])[:max(n, m)]
        reqs.append(r.astype(np.int64))
    return reqs


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_batches_against_the_requests_served_in_order(seed):
    rng = np.random.default_rng(seed)
    universe = np.unique(rng.integers(-(1 << 63), (1 << 63) - 1, size=3000, dtype=np.int64))
    universe = np.concatenate([universe, np.array([-(1 << 63), -(1 << 63) + 1], dtype=np.int64)])
    weights = (1, 3, 3, 3, 5)
    ix, ox = BlockIndex(len(universe)), oracle.Index()
    ms = BatchMetaSearcher(ix, avail_mask_from_weights(weights))
    # something is there already: served chains, keys being written, and keys whose map holds nothing writable
    held = universe[rng.permutation(len(universe))[:900]]
    maps = [[(S, 4)] if j % 3 else ([(W, 2)] if j % 2 else [(oracle.CLS_NOT_FOUND, 1)]) for j in range(len(held))]
    if seed == 3:
        maps = [m if m[0][0] != oracle.CLS_NOT_FOUND else [(S, 4)] for m in maps]  # a batch without such keys
    ox.put(held, maps)
    ix.upsert(torch.from_numpy(held).to(DEV),
              torch.tensor([encode_locations(m) for m in maps], dtype=torch.int64, device=DEV))
    full = torch.zeros(4, dtype=torch.int32, device=DEV)
    seen = set()
    for round_no in range(6):
        reqs = _requests(rng, universe, 200, 40)
        keys, off = _csr(reqs)
        sessions = ms.StartWriteCache(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), 4, full)
        want = _sequential_start(ox, reqs, 4, weights)
        seen |= _compare_start(sessions, reqs, off, want)
        _check_against_oracle(ix, ox, universe)
        assert ix.stats()[1] == len(ox)
        # finish: offsets in even rounds, one byte per session key in odd ones
        n_sess = np.array([len(w[3]) for w in want])
        if round_no % 2 == 0:
            success = np.array([int(rng.integers(0, n + 1)) for n in n_sess], dtype=np.int64)
            codes = ms.FinishWriteCache(sessions, success_off=torch.from_numpy(success).to(DEV)).cpu().numpy()
            ok = [np.arange(n) < s for n, s in zip(n_sess, success)]
        else:
            bits = (rng.random(int(n_sess.sum())) < 0.7).astype(np.uint8)
            codes = ms.FinishWriteCache(sessions, success_bits=torch.from_numpy(bits).to(DEV)).cpu().numpy()
            ok = np.split(bits.astype(bool), np.cumsum(n_sess)[:-1])
        assert not codes.any()
        for (kind, what, n, new), good in zip(want, ok):
            ox.update_status(new[good], 4, -1, S)       # BatchUpdateLocationStatus: unconditional
            ox.update_status(new[~good], 4, -1, -1)     # the failed blocks' locations go
        _check_against_oracle(ix, ox, universe)
        assert ix.stats()[1] == len(ox)
    assert seen == {"offset", "vector"} and full[0].item() == 0


def test_by_hand_and_bad_arguments():
    """Three requests over an empty index: a b c / a b d e / x b.  In order: the first writes a b c; the second sees
    a b being written and writes d e (offset 2); the third sees b and writes x (vector form)."""
    ix = BlockIndex(64)
    ms = BatchMetaSearcher(ix)
    a, b, c, d, e, x = 11, 12, 13, 14, 15, 99
    keys = torch.tensor([a, b, c, a, b, d, e, x, b], dtype=torch.int64, device=DEV)
    off = torch.tensor([0, 3, 7, 9], dtype=torch.int64, device=DEV)
    s = ms.StartWriteCache(keys, off, 4)
    assert s.offset.cpu().tolist() == [0, 2, -1] and s.n_new.cpu().tolist() == [3, 2, 1]
    assert s.added.cpu().tolist() == [1, 1, 1, 0, 0, 1, 1, 1, 0] and s.new_off.cpu().tolist() == [0, 3, 5, 6]
    assert s.mask.cpu().tolist()[7:] == [0, 1]
    ko = torch.tensor([0, 9], dtype=torch.int64, device=DEV)
    assert int(ms.PrefixMatch(keys[:3], off[:2]).cpu()[0]) == 0          # nothing is served yet
    # an offset beyond a session's keys: that request is refused and left alone, the others go through
    codes = ms.FinishWriteCache(s, success_off=torch.tensor([3, 3, 0], dtype=torch.int64, device=DEV)).cpu().tolist()
    assert codes == [0, _cabi.KVCM_EC_BADARGS, 0]
    assert int(ms.PrefixMatch(keys[:3], off[:2]).cpu()[0]) == 3
    flags = ms.BatchGet(torch.tensor([d, e, x], dtype=torch.int64, device=DEV)).cpu().numpy()
    assert (flags[:2] & _cabi.FLAG_WRITABLE).all() and not (flags[:2] & _cabi.FLAG_SERVABLE).any()   # still written
    assert flags[2] == 0                                                                              # failed: gone
    with pytest.raises(_cabi.KvcmError):
        BatchMetaSearcher(ix, avail_mask_from_weights((1, 3, 3, 3, 0))).StartWriteCache(keys, off, 4)
    with pytest.raises(_cabi.KvcmError):
        ms.StartWriteCache(keys, off, 8)
    empty = ms.StartWriteCache(keys[:0], torch.zeros(1, dtype=torch.int64, device=DEV), 4)
    assert empty.n_new.numel() == 0 and empty.new_off.cpu().tolist() == [0]


def test_small_universes_drawn_by_hypothesis():
    """Eight keys, up to eight short requests per batch: nearly every key is named by several requests, and the keys
    start out absent, served, being written, holding a map with nothing writable, or on another tier."""
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    states = [None, [(S, 4)], [(W, 4)], [(oracle.CLS_NOT_FOUND, 1)], [(S, 2)], [(oracle.CLS_NOT_FOUND, 4)], []]
    universe = np.array([5, 6, 7, 8, 9, 10, -(1 << 63), -(1 << 63) + 1], dtype=np.int64)

    @settings(max_examples=200, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
    @given(st.lists(st.integers(0, len(states) - 1), min_size=8, max_size=8),
           st.lists(st.lists(st.integers(0, 7), min_size=0, max_size=6, unique=True), min_size=1, max_size=8),
           st.integers(0, 1 << 30))
    def run(initial, picks, seed):
        ix, ox = BlockIndex(64), oracle.Index()
        ms = BatchMetaSearcher(ix)
        have = [(k, states[s]) for k, s in zip(universe, initial) if states[s] is not None]
        if have:
            ox.put([k for k, _ in have], [m for _, m in have])
            ix.upsert(torch.tensor([int(k) for k, _ in have], dtype=torch.int64, device=DEV),
                      torch.tensor([encode_locations(m) for _, m in have], dtype=torch.int64, device=DEV))
        reqs = [universe[np.array(p, dtype=np.int64)] for p in picks]
        keys, off = _csr(reqs)
        sessions = ms.StartWriteCache(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV), 4)
        want = []
        for r in reqs:  # a location of class 4 that is there already cannot take a second one: the reference's map can
            kind, what, n_new = ox.filter_write(r, weights=oracle.DEFAULT_WEIGHTS)
            new = r[what:] if kind == "offset" else r[~what]
            free = np.array([all(t != 4 for _, t in (ox.get(int(k)) or [])) for k in new], dtype=bool)
            ox.add_location(new[free], 4, W)
            want.append((kind, what, n_new, new[free]))
        _compare_start(sessions, reqs, off, want)
        _check_against_oracle(ix, ox, universe)
        rng = np.random.default_rng(seed)
        n_sess = np.array([len(w[3]) for w in want])
        bits = (rng.random(int(n_sess.sum())) < 0.5).astype(np.uint8)
        codes = ms.FinishWriteCache(sessions, success_bits=torch.from_numpy(bits).to(DEV) if len(bits) else
                                    torch.zeros(1, dtype=torch.uint8, device=DEV)).cpu().numpy()
        assert not codes.any()
        for (kind, what, n, new), good in zip(want, np.split(bits.astype(bool), np.cumsum(n_sess)[:-1])):
            ox.update_status(new[good], 4, -1, S)
            ox.update_status(new[~good], 4, -1, -1)
        _check_against_oracle(ix, ox, universe)

    run()


def test_batch_of_the_window_match_configuration_by_its_properties():
    """65,536 requests of 16-8,192 keys that share prefixes of 1,000 root prompts (the shape of the sliding-window
    configuration, some 86 M keys): too large for the oracle, so checked by what must hold after StartWriteCache and a
    FinishWriteCache in which every block succeeds - every request is served in full, the index holds every distinct
    key once, and the sessions hold every new key exactly once."""
    dev = torch.device(DEV)
    rng = np.random.default_rng(7)
    n_req, n_roots = 65536, 1000
    lens = np.exp(rng.uniform(np.log(16), np.log(8192), size=n_req)).astype(np.int64)
    root_len = np.exp(rng.uniform(np.log(16), np.log(8192), size=n_roots)).astype(np.int64)
    root = (rng.zipf(1.1, size=n_req) - 1) % n_roots
    share = np.minimum((rng.random(n_req) * np.minimum(lens, root_len[root])).astype(np.int64), lens)
    off = np.zeros(n_req + 1, dtype=np.int64)
    np.cumsum(lens, out=off[1:])
    d_off, d_len = torch.from_numpy(off).to(dev), torch.from_numpy(lens).to(dev)
    req_of = torch.repeat_interleave(torch.arange(n_req, device=dev), d_len)
    within = torch.arange(int(off[-1]), device=dev) - d_off[:-1][req_of]
    keys = torch.where(within < torch.from_numpy(share).to(dev)[req_of],
                       (torch.from_numpy(root).to(dev)[req_of] << 32) | within, ((req_of + n_roots) << 32) | within)
    del req_of, within
    distinct = int(torch.unique(keys).numel())
    index = BlockIndex(distinct + 1000, dev)
    ms = BatchMetaSearcher(index)
    full = torch.zeros(4, dtype=torch.int32, device=dev)
    s = ms.StartWriteCache(keys, d_off, 4, full)
    assert int(ms.PrefixMatch(keys, d_off).sum()) == 0                     # written, not served yet
    codes = ms.FinishWriteCache(s, success_off=s.new_off[1:] - s.new_off[:-1])
    torch.cuda.synchronize()
    assert torch.equal(ms.PrefixMatch(keys, d_off).long(), d_len)
    assert index.stats()[1] == distinct == int(s.new_off[-1]) and full[0].item() == 0 and not codes.any()
    assert int((s.offset < 0).sum()) == 0 and int(s.n_new.sum()) == distinct   # new keys form suffixes here
