"""The CPU oracle against the reference's golden vectors (no GPU)."""
import numpy as np
import pytest

from oracle import kvcm_oracle as oracle


def _index_from(table):
    ix = oracle.Index()
    keys = [int(k) for k in table]
    ix.put(keys, [[tuple(l) for l in table[str(k)]] for k in keys])
    return ix


def test_hash_steps_match_reference_header(hash_kat):
    for s in hash_kat["steps"]:
        h, v, out = int(s["h"]), int(s["v"]), int(s["out"])
        assert oracle.hash_step(h, v) == out
        assert oracle.hash_step_py(h, v) == out


def test_hash_chains_match_reference_header(hash_kat):
    for c in hash_kat["chains"]:
        want = np.array([int(k) for k in c["keys"]], dtype=np.int64)
        got = oracle.gen_key_vector(np.array(c["tokens"], dtype=np.int64), c["block_size"])
        assert np.array_equal(got, want), c["name"]
        got32 = oracle.gen_key_vector(np.array(c["tokens"], dtype=np.uint32), c["block_size"])
        assert np.array_equal(got32, want), c["name"]


def test_apply_prefix_hash(hash_kat):
    p = hash_kat["apply_prefix_hash"]
    assert oracle.apply_prefix_hash(p["ids"]).tolist() == [int(k) for k in p["keys"]]
    # ApplyPrefixHash is GenKeyVector with block_size 1
    assert np.array_equal(oracle.apply_prefix_hash(p["ids"]), oracle.gen_key_vector(np.array(p["ids"]), 1))


def test_oracle_equals_compiled_reference_header_on_random_chains():
    ref = oracle.ref_hash()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    import ctypes
    rng = np.random.default_rng(7)
    p64 = ctypes.POINTER(ctypes.c_int64)
    for bs in (1, 16, 64):
        toks = rng.integers(0, 1 << 32, size=5000).astype(np.int64)
        want = np.empty(len(toks) // bs, dtype=np.int64)
        ref.kvcm_ref_gen_key_vector(toks.ctypes.data_as(p64), ctypes.c_int64(len(toks)), ctypes.c_int64(bs),
                                    want.ctypes.data_as(p64))
        assert np.array_equal(oracle.gen_key_vector(toks, bs), want)


def test_hash_blocks_csr_is_per_request_gen_key_vector():
    rng = np.random.default_rng(3)
    lens = [0, 5, 64, 130, 63, 1000]
    toks = rng.integers(0, 151936, size=sum(lens)).astype(np.uint32)
    off = np.concatenate([[0], np.cumsum(lens)])
    for threads in (1, 4):
        keys, key_off = oracle.hash_blocks(toks, off, 64, threads=threads)
        assert key_off.tolist() == [0, 0, 0, 1, 3, 3, 18]
        for r in range(len(lens)):
            want = oracle.gen_key_vector(toks[off[r]:off[r + 1]], 64)
            assert np.array_equal(keys[key_off[r]:key_off[r + 1]], want)


def test_prefix_match_tables(match_kat):
    for group in match_kat["prefix"]:
        ix = _index_from(group["index"])
        for case in group["cases"]:
            assert ix.prefix_match(case["keys"], case["mask"]) == case["len"], (group["source"], case)


def test_sw_match_tables(match_kat):
    for group in match_kat["sw"]:
        ix = _index_from(group["index"])
        for case in group["cases"]:
            ec, base = ix.sw_match(case["keys"], case["sw"])
            assert (ec, base) == (case["ec"], case["base"]), (group["source"], case)


def test_sw_zero_is_rejected():
    ix = oracle.Index()
    ix.put_uniform([1, 2])
    assert ix.sw_match([1, 2], 0)[0] == 6


def test_batch_get_tables(match_kat):
    for group in match_kat["batch_get"]:
        ix = _index_from(group["index"])
        for case in group["cases"]:
            flags = ix.batch_get(case["keys"])
            assert [(int(f) & 1) == 1 for f in flags] == case["servable"], (group["source"], case)


def test_sw_match_is_rightmost_full_window_property():
    rng = np.random.default_rng(11)
    for _ in range(200):
        n = int(rng.integers(1, 40))
        sw = int(rng.integers(1, n + 1))
        state = rng.integers(0, 3, size=n)  # 0 absent, 1 writing, 2 serving
        ix = oracle.Index()
        keys = np.arange(100, 100 + n)
        ix.put(keys[state == 1], [[(oracle.CLS_WRITING, 4)]] * int((state == 1).sum()))
        ix.put(keys[state == 2], [[(oracle.CLS_SERVING, 4)]] * int((state == 2).sum()))
        want = -1
        for base in range(n - sw, -1, -1):
            if np.all(state[base:base + sw] == 2):
                want = base
                break
        assert ix.sw_match(keys, sw) == (0, want)


def test_policy_weights_gate_servable():
    ix = oracle.Index()
    ix.put([1, 2], [[(oracle.CLS_SERVING, 1)], [(oracle.CLS_SERVING, 4)]])
    assert ix.prefix_match([1, 2]) == 2
    assert ix.prefix_match([1, 2], weights=(1, 0, 3, 3, 5)) == 0  # HF3FS unavailable
    assert ix.prefix_match([2, 1], weights=(1, 0, 3, 3, 5)) == 1
    # storage type beyond the weight table gets the default weight 1
    ix.put([3], [[(oracle.CLS_SERVING, 5)]])
    assert ix.prefix_match([3]) == 1


def test_filter_write():
    ix = oracle.Index()
    ix.put([1, 2, 3], [[(oracle.CLS_SERVING, 4)], [(oracle.CLS_WRITING, 4)], []])
    assert ix.filter_write([1, 2, 9, 8]) == ("offset", 2, 2)
    assert ix.filter_write([9, 8]) == ("offset", 0, 2)
    kind, mask, n_new = ix.filter_write([1, 9, 2, 3])
    assert kind == "vector" and mask.tolist() == [True, False, True, False] and n_new == 2


def test_crc_known_answers(match_kat):
    for case in match_kat["crc"][0]["cases"]:
        data = case["text"].encode()
        cal = min(case["min_cal_bytes"], len(data) // 2)
        assert oracle.iov_crc(data, cal) == int(case["crc"], 16)


def _pools(rng, n_pools, pool_rows, row_bytes):
    return [rng.integers(0, 256, size=pool_rows * row_bytes, dtype=np.uint8) for _ in range(n_pools)]


def test_move_rows_matches_python_loops_and_roundtrips():
    rng = np.random.default_rng(42)
    n_pools, pool_rows, row_bytes, rpb, n_blocks, n_slots = 4, 200, 48, 8, 10, 16
    pools = _pools(rng, n_pools, pool_rows, row_bytes)
    row_idx = rng.permutation(pool_rows)[:n_blocks * rpb].astype(np.int32)
    slot_idx = rng.permutation(n_slots)[:n_blocks].astype(np.int32)
    st_c = np.zeros(n_slots * n_pools * rpb * row_bytes, dtype=np.uint8)
    st_py = st_c.copy()
    assert oracle.move_rows(pools, st_c, row_idx, slot_idx, rpb, row_bytes, 0, threads=3) == 0
    oracle.move_rows_py(pools, st_py, row_idx, slot_idx, rpb, row_bytes, 0)
    assert np.array_equal(st_c, st_py)
    # element-wise statement of the rule (batch_gather_scatter_helper.py:57-98)
    st = st_c.reshape(n_slots, n_pools, rpb, row_bytes)
    for b in range(n_blocks):
        for p in range(n_pools):
            for t in range(rpb):
                row = row_idx[b * rpb + t]
                assert np.array_equal(st[slot_idx[b], p, t], pools[p].reshape(-1, row_bytes)[row])
    fresh = [np.zeros_like(p) for p in pools]
    oracle.move_rows(fresh, st_c, row_idx, slot_idx, rpb, row_bytes, 1)
    for p in range(n_pools):
        a = fresh[p].reshape(-1, row_bytes)
        assert np.array_equal(a[row_idx], pools[p].reshape(-1, row_bytes)[row_idx])
        untouched = np.setdiff1d(np.arange(pool_rows), row_idx)
        assert not a[untouched].any()


def test_move_rows_skips_out_of_range():
    rng = np.random.default_rng(1)
    pools = _pools(rng, 2, 10, 16)
    st = np.zeros(2 * 2 * 2 * 16, dtype=np.uint8)
    skipped = oracle.move_rows(pools, st, np.array([0, 10, -1, 3], dtype=np.int32), None, 2, 16, 0)
    assert skipped == 2 * 2  # two bad rows x two pools
    assert not st.reshape(2, 2, 2, 16)[0, :, 1].any()


def test_move_legacy_skips_tokens_past_the_cache():
    rng = np.random.default_rng(5)
    total, hidden, n_layers = 32, 24, 3
    layers = [rng.integers(0, 256, size=2 * total * hidden, dtype=np.uint8) for _ in range(n_layers)]
    tok = np.array([4, 31, 32, 0], dtype=np.int32)
    st = np.zeros(n_layers * 2 * len(tok) * hidden, dtype=np.uint8)
    oracle.move_legacy(layers, total, st, tok, hidden, 0)
    v = st.reshape(n_layers, 2, len(tok), hidden)
    for l in range(n_layers):
        cache = layers[l].reshape(2, total, hidden)
        assert np.array_equal(v[l, :, 0], cache[:, 4]) and np.array_equal(v[l, :, 1], cache[:, 31])
        assert not v[l, :, 2].any()


def test_copy_iovs_ignore_advances_offset():
    a = np.arange(8, dtype=np.uint8)
    b = np.arange(100, 104, dtype=np.uint8)
    s = np.zeros(16, dtype=np.uint8)
    n = oracle.copy_iovs([(a, 8, False), (None, 4, True), (b, 4, False)], s, 0)
    assert n == 16 and s.tolist() == list(range(8)) + [0] * 4 + [100, 101, 102, 103]
    a2, b2 = np.zeros_like(a), np.zeros_like(b)
    oracle.copy_iovs([(a2, 8, False), (None, 4, True), (b2, 4, False)], s, 1)
    assert np.array_equal(a, a2) and np.array_equal(b, b2)


def test_replay_reference_known_answers():
    # kv_cache_manager/optimizer/test/optimizer_manager_py_test.py:57-84
    ext, inte, wr, size = oracle.Replay().run([1, 2, 3, 1, 2, 4], [0, 3, 6],
                                              [oracle.TRACE_WRITE_CACHE, oracle.TRACE_GET_LOCATION])
    assert ext.tolist() == [0, 2] and wr.tolist() == [3, 0] and size.tolist() == [3, 3]
    ext, inte, wr, size = oracle.Replay().run([1, 2], [0, 2], [oracle.TRACE_WRITE_CACHE])
    assert wr.tolist() == [2] and ext.tolist() == [0]
    # dialog turns read and write in one step; masked keys count as internal hits
    ext, inte, wr, size = oracle.Replay().run([1, 2, 3, 1, 2, 4, 5, 1, 2, 4], [0, 3, 7, 10],
                                              [oracle.TRACE_DIALOG_TURN, oracle.TRACE_DIALOG_TURN,
                                               oracle.TRACE_GET_LOCATION], [0, 0, 1])
    assert ext.tolist() == [0, 2, 2] and inte.tolist() == [0, 0, 1] and wr.tolist() == [3, 2, 0]
    assert size.tolist() == [3, 5, 5]


W, G, D = oracle.TRACE_WRITE_CACHE, oracle.TRACE_GET_LOCATION, oracle.TRACE_DIALOG_TURN


def test_lru_replay_follows_the_reference_policy_tests():
    # kv_cache_manager/optimizer/test/lru_eviction_policy_test.cc:44-65 (OnBlockAccessed): write 1, write 2,
    # access 1 -> the next eviction of one block takes 2.  As traces: the third write overflows a quota of 2.
    ext, inte, wr, size = oracle.LruReplay(2, evict_batch=1, precise=True).run(
        [1, 2, 1, 3, 2, 1, 3], [0, 1, 2, 3, 4, 5, 6, 7], [W, W, G, W, G, G, G])
    assert wr.tolist() == [1, 1, 0, 1, 0, 0, 0]
    assert ext.tolist() == [0, 0, 1, 0, 0, 1, 1]  # 2 is gone, 1 and 3 stayed
    assert size.tolist() == [1, 2, 2, 2, 2, 2, 2]
    # :67-96 (EvictBlocks): write 1, 2, 3, evict 2 -> 1 and 2 go, in that order
    ext, inte, wr, size = oracle.LruReplay(1, evict_batch=1, precise=True).run(
        [1, 2, 3, 1, 2, 3], [0, 1, 2, 3, 4, 5, 6], [W, W, W, G, G, G])
    assert size.tolist() == [1, 1, 1, 1, 1, 1] and ext.tolist() == [0, 0, 0, 0, 0, 1]
    # :98-115, 133-146 (evict more than there is): a batch larger than the list empties it
    ext, inte, wr, size = oracle.LruReplay(1, evict_batch=10, precise=False).run([1, 2, 1], [0, 1, 2, 3], [W, W, G])
    assert size.tolist() == [1, 0, 0] and ext.tolist() == [0, 0, 0]


def test_lru_replay_rough_mode_evicts_whole_batches():
    # kv_cache_manager/optimizer/manager/eviction_manager.cc:148-192: rounds of evict_batch until the excess is covered
    keys = list(range(1, 11))
    run = lambda precise: oracle.LruReplay(7, evict_batch=2, precise=precise).run(  # noqa: E731
        keys + [11], [0, 10, 11], [W, W])
    assert run(True)[3].tolist() == [7, 7]     # 10 -> excess 3 -> 7; 8 -> excess 1 -> 7
    assert run(False)[3].tolist() == [6, 7]    # 10 -> two batches of 2 -> 6; 7 -> no excess


def test_lru_replay_with_room_for_everything_is_the_plain_replay():
    rng = np.random.default_rng(3)
    prompts = [rng.integers(1, 1 << 60, size=int(rng.integers(1, 30))) for _ in range(8)]
    keys, off, types, mo = [], [0], [], []
    for t in range(500):
        p = prompts[int(rng.integers(0, len(prompts)))]
        k = list(p[:int(rng.integers(0, len(p) + 1))]) + [int(x) for x in rng.integers(1 << 61, 1 << 62, size=3)]
        ty = int(rng.integers(0, 3))
        keys += k
        off.append(len(keys))
        types.append(ty)
        mo.append(int(rng.integers(0, len(k))) if ty == G else 0)
    want = oracle.Replay().run(keys, off, types, mo)
    got = oracle.LruReplay(1 << 40).run(keys, off, types, mo)
    for a, b in zip(want, got):
        assert np.array_equal(a, b)
    # and a tight quota changes the answers (the test above would be vacuous otherwise)
    tight = oracle.LruReplay(20, evict_batch=4).run(keys, off, types, mo)
    assert tight[3].max() <= 20 + 40 and not np.array_equal(tight[0], want[0])


def test_lru_replay_revives_evicted_blocks_inside_a_node():
    # a chain 1-2-3-4 written as one node; a quota of 2 evicts 1 and 2 (the oldest); the dialog turn [1,2,3,4]
    # then finds no leading hit (1 is gone), rewrites 1 and 2 and leaves 3 and 4 untouched
    # (kv_cache_manager/optimizer/index/radix_tree_index.cc:246-262), so the next eviction takes 3 and 4.
    ext, inte, wr, size = oracle.LruReplay(2, evict_batch=1, precise=True).run(
        [1, 2, 3, 4, 1, 2, 3, 4, 1, 2, 3, 4], [0, 4, 8, 12], [W, D, G])
    assert wr.tolist() == [4, 2, 0] and ext.tolist() == [0, 0, 2] and size.tolist() == [2, 2, 2]


def _leaf(quota, keys, off, types, ts, batch=1, precise=True):
    return oracle.LruReplay(quota, evict_batch=batch, precise=precise, policy="leaf_aware_lru").run(
        keys, off, types, timestamps=ts)


def _flat(traces):
    keys, off = [], [0]
    for k in traces:
        keys += k
        off.append(len(keys))
    return keys, off


def test_leaf_aware_lru_keeps_shared_prefixes():
    # Worked by hand from kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:85-133 (no test of this
    # policy exists in the reference).  [1,2,3] then [1,2,9] splits the node into [1,2] -> {[3], [9]}.  Quota 3:
    # the queue's cold end holds 1 and 2, whose node now has cached children, so they leave the queue (:101-105)
    # and 3 goes.  Its emptied leaf is removed (radix_tree_index.cc:284-325).  Plain LRU would have taken 1.
    keys, off = _flat([[1, 2, 3], [1, 2, 9], [1, 2, 3], [1, 2, 9, 10], [1, 2, 9, 10]])
    ext, inte, wr, size = _leaf(3, keys, off, [W, W, G, W, G], [0, 1, 2, 3, 4])
    assert wr.tolist() == [3, 1, 0, 1, 0]
    assert size.tolist() == [3, 3, 3, 3, 3]
    # trace 3 appends 10 to the leaf [9]; the queue is then 10, 9 and 9 goes although 10 hangs below it
    assert ext.tolist() == [0, 0, 2, 0, 2]
    lru = oracle.LruReplay(3, evict_batch=1, precise=True).run(keys, off, [W, W, G, W, G])
    assert lru[0].tolist()[2] == 0  # plain LRU drops block 1 first, so the same query finds nothing


def test_leaf_aware_lru_requeues_a_parent_by_access_time():
    # Worked by hand: after [1,2,3] (t=10) and [1,2,9] (t=20) the writes of 5, 6 and 8 overflow a quota of 4 one
    # block at a time.  t=30: 1 and 2 leave the queue, 3 goes.  t=40: 9 goes, which makes [1,2] a data leaf: its
    # blocks are put back by last access time (:135-160): 1 lands behind 5, and 2, whose time ties with 1's,
    # behind 1 (insert_sorted_reverse stops at the first entry that is not younger, common_structure.h:77-89),
    # so at t=50 it is 2 that goes, not 1.
    keys, off = _flat([[1, 2, 3], [1, 2, 9], [5], [6], [8], [1, 2], [1, 2, 3], [5], [8], [1, 2, 3]])
    types = [W, W, W, W, W, G, D, G, G, G]
    ts = [10, 20, 30, 40, 50, 60, 70, 80, 90, 100]
    ext, inte, wr, size = _leaf(4, keys, off, types, ts)
    assert wr.tolist() == [3, 1, 1, 1, 1, 0, 2, 0, 0, 0]
    assert size.tolist() == [3, 4, 4, 4, 4, 4, 4, 4, 4, 4]
    # trace 6 (a dialog turn) hits 1, rewrites 2 inside the node and appends 3 to it (a leaf again); 5 and 6 go
    assert ext.tolist() == [0, 0, 0, 0, 0, 1, 1, 0, 1, 3]


def test_leaf_aware_lru_with_room_for_everything_is_the_plain_replay():
    rng = np.random.default_rng(5)
    prompts = [rng.integers(1, 1 << 60, size=int(rng.integers(1, 30))) for _ in range(8)]
    keys, off, types, mo = [], [0], [], []
    for t in range(400):
        p = prompts[int(rng.integers(0, len(prompts)))]
        k = list(p[:int(rng.integers(0, len(p) + 1))]) + [int(x) for x in rng.integers(1 << 61, 1 << 62, size=3)]
        ty = int(rng.integers(0, 3))
        keys += k
        off.append(len(keys))
        types.append(ty)
        mo.append(int(rng.integers(0, len(k))) if ty == G else 0)
    want = oracle.Replay().run(keys, off, types, mo)
    got = oracle.LruReplay(1 << 40, policy="leaf_aware_lru").run(keys, off, types, mo)
    for a, b in zip(want, got):
        assert np.array_equal(a, b)
    tight = oracle.LruReplay(20, evict_batch=4, policy="leaf_aware_lru").run(keys, off, types, mo)
    lru = oracle.LruReplay(20, evict_batch=4).run(keys, off, types, mo)
    assert not np.array_equal(tight[0], want[0]) and not np.array_equal(tight[0], lru[0])


def test_lru_group_quota_shared_by_two_instances():
    # kv_cache_manager/optimizer/manager/eviction_manager.cc:86-146,148-239 by hand (the reference tests groups of one
    # instance only, eviction_manager_test.cc): instances a and b write the same keys into separate trees, quota 4,
    # batches of 1.  a: 1 2 3, b: 1 2 -> 5 cached, one over.  GROUP_ROUGH takes a block from a AND from b in its one
    # round; the instance modes take one block from the writer b only.
    keys, off, types, inst = [1, 2, 3, 1, 2, 1, 2, 3, 1, 2], [0, 3, 5, 8, 10], [W, W, G, G], [0, 1, 0, 1]
    ext, inte, wr, size, final = oracle.LruGroupReplay(4, 2, evict_batch=1, mode=1).run(keys, off, types, inst)
    assert size.tolist() == [3, 1, 2, 1] and final.tolist() == [2, 1] and ext.tolist() == [0, 0, 0, 0]
    for mode in (2, 3):
        ext, inte, wr, size, final = oracle.LruGroupReplay(4, 2, evict_batch=1, mode=mode).run(keys, off, types, inst)
        assert size.tolist() == [3, 1, 3, 1] and final.tolist() == [3, 1] and ext.tolist() == [0, 0, 3, 0]
    # a group of one instance is the plain replay in every mode
    rng = np.random.default_rng(9)
    k = rng.integers(1, 50, size=400).tolist()
    o = list(range(0, 401, 4))
    ty = rng.integers(0, 3, size=100).tolist()
    for mode, precise in ((1, False), (2, False), (3, True)):
        a = oracle.LruReplay(30, evict_batch=3, precise=precise).run(k, o, ty)
        b = oracle.LruGroupReplay(30, 1, evict_batch=3, mode=mode).run(k, o, ty, [0] * 100)
        for x, y in zip(a, b):
            assert np.array_equal(x, y)


def test_leaf_aware_group_of_two_instances_by_hand():
    # kv_cache_manager/optimizer/manager/eviction_manager.cc:86-146 over LeafAwareLruEvictionPolicy::EvictBlocks
    # (kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:85-160), quota 5, batches of 1, group rough; no
    # test of the reference covers this.
    #   a writes 1 2 3, then 1 2 9 (a split: {1 2} over {3} and {9}); b writes 1 2: the group holds 6.
    #   The round asks a first: 1 and 2 sit in a node with cached children and only leave the queue, 3 goes;
    #   then b, whose {1 2} is a leaf: 1 goes.  a reads 1 2 3 -> 2 hits; b reads 1 2 -> none.
    #   a writes 5, b writes 7 8 (7 held).  a loses 9, which turns {1 2} into a data leaf: both are queued again,
    #   at the cold end behind 5 (their time, 3, is the oldest), 1 before 2; b loses 2.
    #   a reads 1 2 9 -> 2 hits and both move to the front, so a's next victim is 5; b's is 7.
    traces = [[1, 2, 3], [1, 2, 9], [1, 2], [1, 2, 3], [1, 2], [5], [7, 8], [1, 2, 9], [6]]
    inst = [0, 0, 1, 0, 1, 0, 1, 0, 0]
    types = [W, W, W, G, G, W, W, G, W]
    keys = [k for t in traces for k in t]
    off = np.cumsum([0] + [len(t) for t in traces])
    run = lambda mode: oracle.LruGroupReplay(5, 2, evict_batch=1, mode=mode, policy="leaf_aware_lru").run(
        keys, off, types, inst, timestamps=list(range(9)))
    ext, inte, wr, size, final = run(1)
    assert ext.tolist() == [0, 0, 0, 2, 0, 0, 0, 2, 0] and wr.tolist() == [3, 1, 2, 0, 0, 1, 2, 0, 1]
    assert size.tolist() == [3, 4, 1, 3, 1, 4, 2, 3, 3] and final.tolist() == [3, 1]
    for mode in (2, 3):  # from the writing instance only: b pays for its own writes, a keeps 3
        ext, inte, wr, size, final = run(mode)
        assert ext.tolist() == [0, 0, 0, 3, 0, 0, 0, 2, 0] and final.tolist() == [4, 1]


def test_compare_and_delete_drops_a_key_left_behind_empty():
    # kv_cache_manager/manager/meta_searcher.cc:689-692: compare-and-delete removes a key whose location map is empty
    # whatever its tasks did.  BatchDeleteLocation leaves such keys behind (:783-786).  Found by comparing with the
    # reference's own MetaSearcher compiled in place (tests/test_matchers_reference_pins.py).
    ix = oracle.Index()
    ix.put([7, 8], [[(oracle.CLS_SERVING, 4)], [(oracle.CLS_SERVING, 4), (oracle.CLS_WRITING, 1)]])
    assert ix.update_status([7, 8], 4, -1, -2).tolist() == [0, 0]      # BatchDeleteLocation: 7 stays, empty
    assert ix.get(7) == [] and ix.get(8) == [(oracle.CLS_WRITING, 1)]
    assert ix.update_status([7, 8], 4, oracle.CLS_SERVING, -1).tolist() == [2, 2]  # no such location in either
    assert ix.get(7) is None and ix.get(8) == [(oracle.CLS_WRITING, 1)]  # the empty key is gone, the other is not
    assert ix.update_status([7], 4, -1, -2).tolist() == [0]            # and a delete of an absent key is EC_OK


def test_location_status_cases_of_the_reference_tests():
    """Update / compare-and-set / compare-and-delete / delete of location statuses, replayed from the tables of
    kv_cache_manager/manager/test/meta_searcher_test.cc (tests/golden/status_kat.json)."""
    from conftest import load_golden
    for case in load_golden("status_kat.json")["cases"]:
        ix = oracle.Index()
        keys0 = [int(k) for k in case["initial"]]
        ix.put(keys0, [[tuple(l) for l in case["initial"][str(k)]] for k in keys0])
        for step in case["steps"]:
            got = ix.update_status(step["keys"], step["types"], step["expected"], step["new"])
            assert got.tolist() == step["results"], case["name"]
            for k, want in step["after"].items():
                have = ix.get(int(k))
                assert (have is None) == (want is None), case["name"]
                if want is not None:
                    assert sorted(have) == sorted(tuple(l) for l in want), case["name"]
