"""Write side of the device-resident block index through the C ABI: location-status transitions against the
oracle's location maps and the reference's own test tables, and a table that survives insert / erase churn."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi
from tair_kvcache_b200.manager import BatchMetaSearcher, BlockIndex, encode_locations, status_task

from conftest import load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# ErrorCode numbers of the reference (kv_cache_manager/common/error_code.h) -> return codes of the C ABI
EC = {0: _cabi.KVCM_OK, 2: _cabi.KVCM_EC_NOENT, 16: _cabi.KVCM_EC_MISMATCH}


def _decode(word):
    """The (status, class) pairs a value word carries in its status fields, None for an absent key."""
    word = int(np.uint64(word))
    if word == 0:
        return None
    out = []
    for c in range(8):
        f = (word >> (_cabi.VAL_STATUS_SHIFT + 3 * c)) & 7
        if f:
            out.append((f - 1, c))
    return out


def _tasks(types, expected, new):
    words = []
    for t, e, n in zip(types, expected, new):
        words.append(status_task(t, None if e < 0 else e, None if n < 0 else n, keep_key=(n == -2)))
    return torch.tensor(words, dtype=torch.int32, device=DEV)


def _check_against_oracle(ix, ox, keys):
    """Status fields, summary bits and the matchers' flag bytes of `keys` agree with the oracle's location maps."""
    dk = torch.from_numpy(np.asarray(keys, dtype=np.int64)).to(DEV)
    words = ix.lookup(dk).cpu().numpy()
    for k, w in zip(keys, words):
        have, want = _decode(w), ox.get(int(k))
        assert (have is None) == (want is None), (k, have, want)
        if want is not None:
            assert sorted(have) == sorted(want), (k, have, want)
            assert int(np.uint64(w)) & ~(1 << 63) == encode_locations(want), (k, hex(int(np.uint64(w))))
    flags = BatchMetaSearcher(ix).BatchGet(dk).cpu().numpy()
    assert np.array_equal(flags, ox.batch_get(np.asarray(keys, dtype=np.int64)))


def test_location_status_cases_of_the_reference_tests():
    """kv_cache_manager/manager/test/meta_searcher_test.cc: update (:347-418), compare-and-set (:736-842, :1005-1074),
    compare-and-delete (:844-932, :1076-1182), delete; tests/golden/status_kat.json."""
    for case in load_golden("status_kat.json")["cases"]:
        ox, ix = oracle.Index(), BlockIndex(64)
        keys0 = [int(k) for k in case["initial"]]
        maps0 = [[tuple(l) for l in case["initial"][str(k)]] for k in keys0]
        ox.put(keys0, maps0)
        ix.upsert(torch.tensor(keys0, dtype=torch.int64, device=DEV),
                  torch.tensor([encode_locations(m) for m in maps0], dtype=torch.int64, device=DEV))
        for step in case["steps"]:
            dk = torch.tensor(step["keys"], dtype=torch.int64, device=DEV)
            got = ix.update_status(dk, _tasks(step["types"], step["expected"], step["new"])).cpu().tolist()
            assert got == [EC[r] for r in step["results"]], case["name"]
            for k, want in step["after"].items():
                have = _decode(ix.lookup(torch.tensor([int(k)], dtype=torch.int64, device=DEV)).cpu().numpy()[0])
                assert (have is None) == (want is None), case["name"]
                if want is not None:
                    assert sorted(have) == sorted(tuple(l) for l in want), case["name"]
        live = [int(k) for k in case["steps"][-1]["after"] if case["steps"][-1]["after"][k] is not None]
        assert ix.stats()[1] == len(live), case["name"]


def test_compare_and_delete_drops_a_key_left_behind_empty():
    """kv_cache_manager/manager/meta_searcher.cc:689-692: compare-and-delete removes a key whose location map is
    empty whatever its tasks did; BatchDeleteLocation leaves such keys behind (:783-786)."""
    ix = BlockIndex(64)
    keys = torch.tensor([7, 8], dtype=torch.int64, device=DEV)
    ix.upsert(keys, torch.tensor([encode_locations([(3, 4)]), encode_locations([(3, 4), (2, 1)])], dtype=torch.int64,
                                 device=DEV))
    keep = _tasks([4, 4], [-1, -1], [-2, -2])
    assert ix.update_status(keys, keep).cpu().tolist() == [_cabi.KVCM_OK, _cabi.KVCM_OK]
    assert [_decode(w) for w in ix.lookup(keys).cpu().numpy()] == [[], [(2, 1)]] and ix.stats()[1] == 2
    cad = _tasks([4, 4], [3, 3], [-1, -1])
    assert ix.update_status(keys, cad).cpu().tolist() == [_cabi.KVCM_EC_NOENT, _cabi.KVCM_EC_NOENT]
    assert [_decode(w) for w in ix.lookup(keys).cpu().numpy()] == [None, [(2, 1)]] and ix.stats()[1] == 1
    assert ix.update_status(keys[:1], keep[:1]).cpu().tolist() == [_cabi.KVCM_OK]


def test_uniform_task_and_bad_tasks():
    ix = BlockIndex(64)
    keys = torch.arange(10, 20, dtype=torch.int64, device=DEV)
    ix.upsert(keys, None, encode_locations([(oracle.CLS_WRITING, 3)]))
    # FinishWriteCache for a whole batch: WRITING -> SERVING in class 3, one task word for every key
    res = ix.update_status(keys, status_task(3, oracle.CLS_WRITING, oracle.CLS_SERVING))
    assert not res.cpu().numpy().any()
    assert (BatchMetaSearcher(ix).BatchGet(keys).cpu().numpy() & _cabi.FLAG_SERVABLE).all()
    with pytest.raises(_cabi.KvcmError):
        ix.update_status(keys, status_task(9, None, 3))          # classes 8..15 have no status field
    with pytest.raises(_cabi.KvcmError):
        ix.update_status(keys, status_task(3, 7, 3))             # no such status
    bad = torch.tensor([status_task(3, None, 6)] * 10, dtype=torch.int32, device=DEV)
    assert (ix.update_status(keys, bad).cpu().numpy() == _cabi.KVCM_EC_BADARGS).all()


def test_random_transitions_against_the_oracle():
    rng = np.random.default_rng(11)
    n = 4000
    keys = np.unique(rng.integers(-(1 << 63), (1 << 63) - 1, size=n, dtype=np.int64))
    keys = np.concatenate([keys, np.array([-(1 << 63), -(1 << 63) + 1], dtype=np.int64)])  # the two reserved values
    maps = []
    for _ in keys:
        classes = rng.choice(6, size=int(rng.integers(0, 4)), replace=False)  # at most one location per class
        maps.append([(int(rng.integers(0, 5)), int(c)) for c in classes])
    ox, ix = oracle.Index(), BlockIndex(len(keys))
    ox.put(keys, maps)
    ix.upsert(torch.from_numpy(keys).to(DEV),
              torch.tensor([encode_locations(m) for m in maps], dtype=torch.int64, device=DEV))
    _check_against_oracle(ix, ox, keys)
    absent = rng.integers(1, 1 << 62, size=200, dtype=np.int64) * 2 + 1
    absent = absent[~np.isin(absent, keys)]
    for round_no in range(12):
        pick = rng.permutation(len(keys))[:1500]           # no key twice in one call: the order would matter
        batch = np.concatenate([keys[pick], absent[:50]])
        types = rng.integers(0, 6, size=len(batch))
        expected = rng.choice([-1, 0, 1, 2, 3, 4], size=len(batch))
        new = rng.choice([-2, -1, 0, 1, 2, 3, 4], size=len(batch))
        want = ox.update_status(batch, types, expected, new)
        got = ix.update_status(torch.from_numpy(batch).to(DEV), _tasks(types, expected, new)).cpu().numpy()
        assert np.array_equal(got, np.array([EC[int(r)] for r in want], dtype=np.int32)), round_no
        _check_against_oracle(ix, ox, np.concatenate([keys, absent[:50]]))
        assert ix.stats()[1] == len(ox)
    # the matchers see the transitions: prefix match over a request made of the keys in table order
    dk = torch.from_numpy(keys).to(DEV)
    ko = torch.tensor([0, len(keys)], dtype=torch.int64, device=DEV)
    assert int(BatchMetaSearcher(ix).PrefixMatch(dk, ko).cpu()[0]) == ox.prefix_match(keys)


def test_sharded_transitions_touch_only_owned_keys():
    rng = np.random.default_rng(5)
    keys = np.unique(rng.integers(-(1 << 62), 1 << 62, size=2000, dtype=np.int64))
    dk = torch.from_numpy(keys).to(DEV)
    shards = [BlockIndex(len(keys)) for _ in range(3)]
    word = encode_locations([(oracle.CLS_WRITING, 2)])
    for r, sh in enumerate(shards):
        _cabi.call("kvcm_b200_index_upsert_sharded", sh.handle, dk.data_ptr(), None, word, dk.numel(), 3, r, None,
                   sh._s())
    out = torch.full((len(keys),), -1, dtype=torch.int32, device=DEV)
    for r, sh in enumerate(shards):
        sh.update_status(dk, status_task(2, oracle.CLS_WRITING, oracle.CLS_SERVING), shard=(3, r), out=out)
    assert not out.cpu().numpy().any()                      # every key was answered by exactly its owner
    assert sum(sh.stats()[1] for sh in shards) == len(keys)
    for sh in shards:
        w = sh.lookup(dk).cpu().numpy()
        assert all(_decode(x) in (None, [(oracle.CLS_SERVING, 2)]) for x in w)


def test_table_survives_churn():
    """Ten times the table's slots in inserts, each batch erased again a few batches later, as the reclaimer
    does: no insert is refused, the slots in use stay bounded, and every lookup stays right."""
    ix = BlockIndex(2048)                                   # 4096 slots
    slots = ix.stats()[0]
    rng = np.random.default_rng(3)
    word = encode_locations([(oracle.CLS_SERVING, 4)])
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    resident, inserted, worst_used = [], 0, 0
    gone = np.zeros(0, dtype=np.int64)
    while inserted < 10 * slots:
        batch = rng.integers(-(1 << 62), 1 << 62, size=256, dtype=np.int64)
        ix.upsert(torch.from_numpy(batch).to(DEV), None, word, status)
        resident.append(batch)
        inserted += len(batch)
        if len(resident) > 6:                               # 6 x 256 = 1536 live keys, 0.375 of the slots
            gone = resident.pop(0)
            ix.erase(torch.from_numpy(gone).to(DEV))
        _, live, used = ix.usage()
        worst_used = max(worst_used, used)
        want_live = len(np.unique(np.concatenate(resident)))
        assert live == want_live and used >= live
    assert status[0].item() == 0                            # no insert was refused
    assert worst_used <= slots // 2 + slots // 8 + 256      # live keys + at most an eighth of the slots in tombstones
    here = np.concatenate(resident)
    assert (ix.lookup(torch.from_numpy(here).to(DEV)).cpu().numpy() != 0).all()
    gone = gone[~np.isin(gone, here)]
    assert not ix.lookup(torch.from_numpy(gone).to(DEV)).cpu().numpy().any()


def test_explicit_rehash_drops_tombstones_and_keeps_values():
    ix = BlockIndex(4096)
    _cabi.call("kvcm_b200_index_set_auto_rehash", ix.handle, 0)      # the caller rebuilds by itself
    rng = np.random.default_rng(9)
    keys = np.unique(rng.integers(-(1 << 63), (1 << 63) - 1, size=4000, dtype=np.int64))
    keys = np.concatenate([keys, np.array([-(1 << 63), -(1 << 63) + 1], dtype=np.int64)])
    vals = rng.integers(1, 1 << 32, size=len(keys)).astype(np.int64)
    dk, dv = torch.from_numpy(keys).to(DEV), torch.from_numpy(vals).to(DEV)
    ix.upsert(dk, dv)
    ix.erase(dk[:3000])
    _, live, used = ix.usage()
    assert live == len(keys) - 3000 and used > live        # tombstones are in the table
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    ix.rehash(status)
    _, live2, used2 = ix.usage()
    assert live2 == live and used2 == live - 2 and status[0].item() == 0   # the two reserved keys use no slot
    got = ix.lookup(dk).cpu().numpy()
    assert not got[:3000].any()
    assert np.array_equal(got[3000:].view(np.uint64), vals[3000:].view(np.uint64) | np.uint64(1 << 63))
    with pytest.raises(_cabi.KvcmError):                   # a workspace that is too small is refused, nothing runs
        small = torch.empty(1024, dtype=torch.uint8, device=DEV)
        _cabi.call("kvcm_b200_index_rehash", ix.handle, small.data_ptr(), small.numel(), None, ix._s())


def test_add_location_write_cycle_of_the_reference():
    """StartWriteCache adds a location in CLS_WRITING, FinishWriteCache turns it to CLS_SERVING
    (MetaSearcher::BatchAddLocation + BatchUpdateLocationStatus, kv_cache_manager/manager/meta_searcher.cc:312-487):
    the matchers see the keys only after the second step, and a second tier's location leaves the first alone."""
    ix, ox = BlockIndex(64), oracle.Index()
    keys = np.array([11, 12, 13, -(1 << 63), -(1 << 63) + 1], dtype=np.int64)  # with the two reserved values
    dk = torch.from_numpy(keys).to(DEV)
    assert not ix.add_location(dk, 4).cpu().numpy().any()
    ox.add_location(keys, 4)
    _check_against_oracle(ix, ox, keys)
    assert ix.stats()[1] == 5
    ko = torch.tensor([0, 5], dtype=torch.int64, device=DEV)
    assert int(BatchMetaSearcher(ix).PrefixMatch(dk, ko).cpu()[0]) == 0       # written, not served yet
    assert not ix.update_status(dk, status_task(4, oracle.CLS_WRITING, oracle.CLS_SERVING)).cpu().numpy().any()
    ox.update_status(keys, 4, oracle.CLS_WRITING, oracle.CLS_SERVING)
    assert int(BatchMetaSearcher(ix).PrefixMatch(dk, ko).cpu()[0]) == 5
    # a location on another tier for three of them: the served one stays
    classes = torch.tensor([2, 2, 0], dtype=torch.uint8, device=DEV)
    assert not ix.add_location(dk[1:4], classes).cpu().numpy().any()
    ox.add_location(keys[1:4], [2, 2, 0])
    _check_against_oracle(ix, ox, keys)
    assert int(BatchMetaSearcher(ix).PrefixMatch(dk, ko).cpu()[0]) == 5 and ix.stats()[1] == 5
    # the word keeps one status per class: a second location of a class is refused, nothing changes
    again = ix.add_location(dk, 4).cpu().numpy()
    assert (again == _cabi.KVCM_EC_EXIST).all()
    _check_against_oracle(ix, ox, keys)
    assert (ix.add_location(dk, torch.full((5,), 9, dtype=torch.uint8, device=DEV)).cpu().numpy()
            == _cabi.KVCM_EC_BADARGS).all()
    with pytest.raises(_cabi.KvcmError):
        ix.add_location(dk, 8)
    with pytest.raises(_cabi.KvcmError):
        ix.add_location(dk, 4, status=5)


def test_add_location_random_rounds_against_the_oracle():
    """Adds, transitions and deletions interleaved; several tasks of one launch may name the same key with different
    classes (they take turns on the word), and a key whose last location went away comes back through an add."""
    rng = np.random.default_rng(21)
    universe = np.unique(rng.integers(-(1 << 63), (1 << 63) - 1, size=600, dtype=np.int64))
    universe = np.concatenate([universe, np.array([-(1 << 63), -(1 << 63) + 1], dtype=np.int64)])
    ix, ox = BlockIndex(len(universe)), oracle.Index()
    full = torch.zeros(4, dtype=torch.int32, device=DEV)
    exist = 0
    for round_no in range(40):
        if round_no % 3 != 2:
            # up to three tasks per key in one launch, each on a class of its own
            pick = universe[rng.permutation(len(universe))[:150]]
            reps = rng.integers(1, 4, size=len(pick))
            batch = np.repeat(pick, reps)
            classes = np.concatenate([rng.permutation(6)[:r] for r in reps]).astype(np.uint8)
            status = int(rng.integers(0, 5))
            order = rng.permutation(len(batch))
            batch, classes = batch[order], classes[order]
            free = np.array([all(t != c for _, t in (ox.get(int(k)) or [])) for k, c in zip(batch, classes)])
            got = ix.add_location(torch.from_numpy(batch).to(DEV), torch.from_numpy(classes).to(DEV), status,
                                  table_full=full).cpu().numpy()
            assert np.array_equal(got, np.where(free, 0, _cabi.KVCM_EC_EXIST)), round_no
            exist += int((~free).sum())
            ox.add_location(batch[free], classes[free], status)
        else:
            batch = universe[rng.permutation(len(universe))[:300]]   # no key twice: the order would matter
            types = rng.integers(0, 6, size=len(batch))
            expected = rng.choice([-1, 0, 1, 2, 3, 4], size=len(batch))
            new = rng.choice([-2, -1, -1, 3], size=len(batch))
            want = ox.update_status(batch, types, expected, new)
            got = ix.update_status(torch.from_numpy(batch).to(DEV), _tasks(types, expected, new)).cpu().numpy()
            assert np.array_equal(got, np.array([EC[int(r)] for r in want], dtype=np.int32)), round_no
        _check_against_oracle(ix, ox, universe)
        assert ix.stats()[1] == len(ox), round_no
    assert full[0].item() == 0 and exist > 50


def test_add_location_full_table_and_shards():
    ix = BlockIndex(8)
    slots = ix.stats()[0]
    keys = torch.arange(1, 4 * slots + 1, dtype=torch.int64, device=DEV)
    full = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = ix.add_location(keys, 3, table_full=full).cpu().numpy()
    refused = int((got == _cabi.KVCM_EC_NOSPC).sum())
    assert refused > 0 and refused == full[0].item() and set(got.tolist()) <= {0, _cabi.KVCM_EC_NOSPC}
    assert ix.stats()[1] == len(keys) - refused
    held = ix.lookup(keys).cpu().numpy() != 0
    assert np.array_equal(held, got == 0)
    # three shards: every key is added by exactly its owner
    rng = np.random.default_rng(6)
    k = np.unique(rng.integers(-(1 << 62), 1 << 62, size=1500, dtype=np.int64))
    dk = torch.from_numpy(k).to(DEV)
    shards = [BlockIndex(len(k)) for _ in range(3)]
    out = torch.full((len(k),), -1, dtype=torch.int32, device=DEV)
    for r, sh in enumerate(shards):
        sh.add_location(dk, 1, shard=(3, r), out=out)
    assert not out.cpu().numpy().any() and sum(sh.stats()[1] for sh in shards) == len(k)
    for sh in shards:
        assert all(_decode(x) in (None, [(oracle.CLS_WRITING, 1)]) for x in sh.lookup(dk).cpu().numpy())
