"""The oracle's block index, matchers and location-status transitions against the REFERENCE's own MetaSearcher.

oracle/_ref/libkvcm_ref_searcher.so is the reference's MetaSearcher over its MetaIndexer and local meta backend,
compiled from the reference's source files in place (oracle/Makefile, target ref_searcher; oracle/
ref_searcher_driver.cc wraps it).  The known-answer tables of the reference's own tests pin the oracle everywhere
(tests/golden/match_kat.json, status_kat.json); here, where that library is present (a container that holds the
reference tree), the two are also compared live on random location maps, masks, weights and task batches.  No GPU:
the GPU kernels are compared with the same oracle in tests/test_gpu_hash_match.py and tests/test_gpu_index_write.py.
"""
import numpy as np
import pytest

from oracle import kvcm_oracle as oracle
from oracle import ref_searcher as ref

pytestmark = pytest.mark.skipif(not ref.available(),
                                reason="oracle/_ref/libkvcm_ref_searcher.so not built (reference tree absent)")

STATUSES = (oracle.CLS_NEW, oracle.CLS_WRITING, oracle.CLS_SERVING, oracle.CLS_DELETING)


def _random_world(rng, n_keys, fill=0.12):
    """The same random location maps in the reference's index and in the oracle's: per key, each storage type at
    most once, in a random status."""
    universe = rng.integers(-(1 << 62), 1 << 62, size=n_keys + n_keys // 4, dtype=np.int64)
    locs = {int(k): [] for k in universe[:n_keys]}
    r, ox = ref.RefSearcher(in_memory=n_keys > 1000), oracle.Index()  # small worlds on a file, as the reference's tests
    for ty in range(5):
        for st in STATUSES:
            ks = [k for k in locs if rng.random() < fill and all(t != ty for _, t in locs[k])]
            if ks:
                r.add(ks, ty, st)
                for k in ks:
                    locs[k].append((st, ty))
    held = [k for k in locs if locs[k]]  # the reference only knows keys that got a location
    ox.put(held, [locs[k] for k in held])
    return universe, {k: locs[k] for k in held}, r, ox


def test_matchers_on_random_location_maps():
    rng = np.random.default_rng(2024)
    universe, locs, r, ox = _random_world(rng, 6000)
    serving = [k for k in locs if any(s == oracle.CLS_SERVING for s, _ in locs[k])]
    hits = windows = 0
    forms = set()
    for weights in (None, (1, 3, 0, 3, 5), (0, 0, 0, 0, 7)):
        ow = oracle.DEFAULT_WEIGHTS if weights is None else weights
        for _ in range(150):
            n = int(rng.integers(0, 40))
            q = rng.choice(universe, size=n)
            likely = rng.random(n) < 0.85
            q[likely] = rng.choice(serving, size=int(likely.sum()))
            for mask in (None, int(rng.integers(0, n + 2)), rng.random(n) < 0.3):
                want = r.prefix_match(q, mask, weights)
                got = ox.prefix_match(q, mask.tolist() if isinstance(mask, np.ndarray) else mask, ow)
                assert got == want, (mask, weights)
                hits += want > 0
            for sw in (1, 3, 8):
                if n < sw:
                    continue  # the reference asserts here; the oracle and the kernels answer -2
                base, count = r.sw_match(q, sw, weights)
                ec, got = ox.sw_match(q, sw, ow)
                assert ec == 0 and got == base and count == (sw if base >= 0 else 0), (sw, weights)
                windows += base >= 0
            servable, nonempty = r.batch_get(q, weights)
            flags = ox.batch_get(q, ow)
            assert np.array_equal(servable, flags & 1) and np.array_equal(nonempty, (flags >> 2) & 1)
            # what StartWriteCache would still have to write (FilterWriteCache over the reference's own policy object)
            want, got = r.filter_write(q, weights), ox.filter_write(q, weights=ow)
            forms.add(want[0])
            assert want[0] == got[0] and np.array_equal(want[1], got[1]) and want[2] == got[2], (weights, want, got)
    assert hits > 300 and windows > 100 and forms == {"offset", "vector"}


def test_status_transitions_on_random_task_batches():
    """BatchUpdateLocationStatus / BatchCASLocationStatus / BatchCADLocationStatus / BatchDeleteLocation
    (kv_cache_manager/manager/meta_searcher.cc:410-820): the per-task error codes, and what the matchers see after."""
    rng = np.random.default_rng(2025)
    universe, locs, r, ox = _random_world(rng, 600, fill=0.2)
    known = np.array(sorted(locs), dtype=np.int64)
    seen = set()
    for round_ in range(60):
        op = int(rng.integers(0, 4))
        n = int(rng.integers(1, 40))
        keys = rng.choice(known, size=n, replace=False)  # one task per key and call
        if rng.random() < 0.3:  # some keys the index has never held
            keys[: n // 4] = rng.integers(1 << 62, (1 << 62) + 1000, size=n // 4)
        types = rng.integers(0, 5, size=n).astype(np.int32)
        expected = rng.choice(STATUSES, size=n).astype(np.int32)
        new = rng.choice(STATUSES, size=n).astype(np.int32)
        rc, want = r.status(op, keys, types, expected, new)
        if op == ref.OP_UPDATE:
            got = ox.update_status(keys, types, -1, new)
        elif op == ref.OP_CAS:
            got = ox.update_status(keys, types, expected, new)
        elif op == ref.OP_CAD:
            got = ox.update_status(keys, types, expected, -1)
        else:
            got = ox.update_status(keys, types, -1, -2)
        assert np.array_equal(want, got), (round_, op, want.tolist(), got.tolist())
        seen.update((op, int(c)) for c in want)
        probe = rng.choice(known, size=64)
        servable, nonempty = r.batch_get(probe)
        flags = ox.batch_get(probe)
        assert np.array_equal(servable, flags & 1) and np.array_equal(nonempty, (flags >> 2) & 1), (round_, op)
    # every operation both succeeded and failed somewhere; compare-and-set / -delete also met a wrong status
    for op in range(4):
        assert (op, 0) in seen
    assert (ref.OP_CAS, 16) in seen and (ref.OP_CAD, 16) in seen and (ref.OP_UPDATE, 2) in seen


def test_hash_and_prefix_match_of_a_batch_of_requests():
    """The reference's CPU path for the prefix-match configuration end to end - the loop of GenKeyVector around its
    hashInt64Array, then PrefixMatch, on several host threads - against the oracle's hash + batched prefix match.
    Once with the local meta backend on a file, as the reference's own tests run it (it rewrites the file on every
    mutation: 13 s for 2,000 keys), once without a storage URI, the reference's switch for a backend that lives in
    memory - which is how bench.py builds the configuration's 200,000-key index in seconds and times this path."""
    rng = np.random.default_rng(2026)
    bs = 16
    prior = [rng.integers(0, 50000, size=int(rng.integers(64, 300))).astype(np.int64) for _ in range(60)]
    reqs = []
    for _ in range(200):
        t = rng.integers(0, 50000, size=int(rng.integers(0, 300))).astype(np.int64)
        if rng.random() < 0.6:
            src = prior[int(rng.integers(len(prior)))]
            m = int(rng.integers(0, min(len(t), len(src)) + 1))
            t[:m] = src[:m]
        reqs.append(t)

    def csr(seqs):
        off = np.zeros(len(seqs) + 1, dtype=np.int64)
        np.cumsum([len(x) for x in seqs], out=off[1:])
        return np.concatenate(seqs), off

    (ptoks, poff), (toks, off) = csr(prior), csr(reqs)
    pkeys = np.unique(oracle.hash_blocks(ptoks, poff, bs, threads=2)[0])
    ox = oracle.Index()
    ox.put_uniform(pkeys)
    keys, ko = oracle.hash_blocks(toks, off, bs, threads=2)
    for in_memory in (False, True):
        r = ref.RefSearcher(in_memory=in_memory)
        r.add(pkeys, 4, oracle.CLS_SERVING)
        want = r.prefix_match_batch(toks, off, bs, threads=4)
        assert np.array_equal(want, ox.prefix_match_batch(keys, ko, threads=2)) and want.sum() > 100
        # the sliding-window configuration's path: prefix and window match per request
        for sw in (1, 3):
            matched, base = r.window_match_batch(toks, off, bs, sw, threads=4)
            assert np.array_equal(matched, want)
            assert np.array_equal(base, ox.sw_match_batch(keys, ko, sw, threads=2)) and (base >= 0).any()


def test_locations_added_between_transitions():
    """BatchAddLocation on keys that hold other locations already, that lost their last location to a compare-and-
    delete, or that BatchDeleteLocation left behind with an empty map (kv_cache_manager/manager/
    meta_searcher.cc:312-408 between the transitions of :410-820): the oracle's add_location against the reference's,
    seen through what the matchers answer afterwards and through the codes of the transitions that follow."""
    rng = np.random.default_rng(2027)
    universe, locs, r, ox = _random_world(rng, 200, fill=0.15)
    known = np.array(sorted(locs), dtype=np.int64)
    fresh = universe[~np.isin(universe, known)][:30]
    pool = np.concatenate([known, fresh])
    added = 0
    for round_ in range(50):
        if round_ % 2 == 0:
            ty, st = int(rng.integers(0, 5)), int(rng.choice(STATUSES))
            # one location per storage type and key, as the device's value word holds them
            cand = pool[rng.permutation(len(pool))[:25]]
            keys = np.array([k for k in cand if all(t != ty for _, t in (ox.get(int(k)) or []))], dtype=np.int64)
            if len(keys) == 0:
                continue
            r.add(keys, ty, st)
            ox.add_location(keys, ty, st)
            added += len(keys)
        else:
            op = int(rng.integers(1, 4))
            keys = pool[rng.permutation(len(pool))[:40]]
            types = rng.integers(0, 5, size=len(keys)).astype(np.int32)
            expected = rng.choice(STATUSES, size=len(keys)).astype(np.int32)
            new = rng.choice(STATUSES, size=len(keys)).astype(np.int32)
            rc, want = r.status(op, keys, types, expected, new)
            got = ox.update_status(keys, types, expected if op != ref.OP_DELETE else -1,
                                   new if op == ref.OP_CAS else (-1 if op == ref.OP_CAD else -2))
            assert np.array_equal(want, got), (round_, op)
        servable, nonempty = r.batch_get(pool)
        flags = ox.batch_get(pool)
        assert np.array_equal(servable, flags & 1) and np.array_equal(nonempty, (flags >> 2) & 1), round_
    assert added > 200
