"""Bit-exact parity of the CUDA hash, index and matchers with the CPU oracle and with the reference's
golden vectors, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi
from tair_kvcache_b200.manager import (ApplyPrefixHashBatch, BatchMetaSearcher, BlockIndex, GenKeyVectorBatch,
                                       encode_locations, key_offsets)
from tair_kvcache_b200.manager.block_index import avail_mask_from_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _csr(lens):
    off = np.zeros(len(lens) + 1, dtype=np.int64)
    np.cumsum(lens, out=off[1:])
    return off


def _gpu_hash(tokens_np, tok_off, bs):
    ko = key_offsets(tok_off, bs)
    toks = torch.from_numpy(tokens_np.view(np.int32) if tokens_np.dtype == np.uint32 else tokens_np).to(DEV)
    keys = GenKeyVectorBatch(toks, torch.from_numpy(np.asarray(tok_off, dtype=np.int64)).to(DEV), bs,
                             torch.from_numpy(ko).to(DEV), int(ko[-1]))
    torch.cuda.synchronize()
    return keys.cpu().numpy(), ko


def test_golden_chains_from_the_reference_header(hash_kat):
    for dtype in (np.uint32, np.int64):
        lens = [len(c["tokens"]) for c in hash_kat["chains"]]
        for bs in sorted({c["block_size"] for c in hash_kat["chains"]}):
            sel = [c for c in hash_kat["chains"] if c["block_size"] == bs]
            toks = np.concatenate([np.asarray(c["tokens"], dtype=dtype) for c in sel] + [np.zeros(0, dtype)])
            off = _csr([len(c["tokens"]) for c in sel])
            keys, ko = _gpu_hash(toks, off, bs)
            for i, c in enumerate(sel):
                want = np.array([int(k) for k in c["keys"]], dtype=np.int64)
                assert np.array_equal(keys[ko[i]:ko[i + 1]], want), (c["name"], dtype)
        assert lens


def test_apply_prefix_hash_golden(hash_kat):
    p = hash_kat["apply_prefix_hash"]
    ids = torch.tensor(p["ids"] + p["ids"], dtype=torch.int64, device=DEV)
    off = torch.tensor([0, 3, 6], dtype=torch.int64, device=DEV)
    keys = ApplyPrefixHashBatch(ids, off).cpu().tolist()
    assert keys == [int(k) for k in p["keys"]] * 2


@pytest.mark.parametrize("bs", [1, 7, 16, 64, 128])
@pytest.mark.parametrize("dtype", [np.uint32, np.int64])
def test_ragged_batches_against_oracle(bs, dtype):
    rng = np.random.default_rng(bs * 31 + (dtype == np.int64))
    lens = np.concatenate([[0, 1, bs - 1, bs, bs + 1, 3 * bs, 0, 5], rng.integers(0, 3000, size=150)])
    rng.shuffle(lens)
    hi = 151936 if dtype == np.uint32 else (1 << 40)
    toks = rng.integers(0, hi, size=int(lens.sum())).astype(dtype)
    if dtype == np.uint32:
        toks[:50] = rng.integers(1 << 31, 1 << 32, size=50)  # ids above int32 must be zero-extended
    off = _csr(lens)
    got, ko = _gpu_hash(toks, off, bs)
    want, ko2 = oracle.hash_blocks(toks, off, bs, threads=4)
    assert np.array_equal(ko, ko2) and np.array_equal(got, want)


def test_long_chain_and_many_requests():
    rng = np.random.default_rng(5)
    lens = np.concatenate([[131072, 100000], rng.integers(256, 2048, size=6000)])
    toks = rng.integers(0, 151936, size=int(lens.sum())).astype(np.uint32)
    off = _csr(lens)
    got, ko = _gpu_hash(toks, off, 16)
    want, _ = oracle.hash_blocks(toks, off, 16, threads=8)
    assert np.array_equal(got, want)


def test_longest_first_order_gives_the_same_keys():
    from tair_kvcache_b200.manager import length_order
    rng = np.random.default_rng(12)
    lens = np.exp(rng.uniform(np.log(16), np.log(20000), size=700)).astype(np.int64)
    toks = rng.integers(0, 151936, size=int(lens.sum())).astype(np.uint32)
    off = _csr(lens)
    order, residency = length_order(off, with_residency=True)
    assert sorted(order.tolist()) == list(range(700)) and (np.diff(lens[order]) <= 0).all()
    assert residency == 2  # 22 warps on 148 SMs: the longest chain rules, so the smallest cap is suggested
    ko = key_offsets(off, 16)
    want, _ = oracle.hash_blocks(toks, off, 16, threads=4)
    for cap in (0, 1, 3, 4, residency):
        keys = GenKeyVectorBatch(torch.from_numpy(toks.view(np.int32)).to(DEV), torch.from_numpy(off).to(DEV), 16,
                                 torch.from_numpy(ko).to(DEV), int(ko[-1]), order=torch.from_numpy(order).to(DEV),
                                 warps_per_sm=cap)
        torch.cuda.synchronize()
        assert np.array_equal(keys.cpu().numpy(), want), cap


def test_residency_cap_with_more_warps_than_slots_gives_the_same_keys():
    """More warps than the capped residency admits at once: CTAs queue up behind the longest chains."""
    from tair_kvcache_b200.manager import length_order
    rng = np.random.default_rng(13)
    lens = np.concatenate([rng.integers(0, 300, size=30000), [40000, 35000, 7]])
    rng.shuffle(lens)
    toks = rng.integers(0, 151936, size=int(lens.sum())).astype(np.uint32)
    off = _csr(lens)
    order = length_order(off)
    ko = key_offsets(off, 16)
    want, _ = oracle.hash_blocks(toks, off, 16, threads=8)
    d = [torch.from_numpy(a).to(DEV) for a in (toks.view(np.int32), off, ko, order)]
    for use_order in (True, False):
        keys = GenKeyVectorBatch(d[0], d[1], 16, d[2], int(ko[-1]), order=d[3] if use_order else None, warps_per_sm=4)
        torch.cuda.synchronize()
        assert np.array_equal(keys.cpu().numpy(), want), use_order


def test_hash_rejects_misaligned_token_buffer():
    t = torch.zeros(64, dtype=torch.int32, device=DEV)
    off = torch.tensor([0, 16], dtype=torch.int64, device=DEV)
    out = torch.zeros(4, dtype=torch.int64, device=DEV)
    _cabi.bind_device(0)
    rc = _cabi.lib().kvcm_b200_hash_blocks_u32(t.data_ptr() + 4, 32, off.data_ptr(), 1, 4, out.data_ptr(),
                                               off.data_ptr(), None, 0, None)
    assert rc == _cabi.KVCM_ER_INVALID_ADDRESS


def _put(ix, ox, table):
    keys = [int(k) for k in table]
    locs = [[tuple(l) for l in table[str(k)]] for k in keys]
    ox.put(keys, locs)
    vals = torch.tensor([encode_locations(l) for l in locs], dtype=torch.int64, device=DEV)
    ix.upsert(torch.tensor(keys, dtype=torch.int64, device=DEV), vals)


def _mask_args(mask, n):
    if mask is None:
        return None, None
    if isinstance(mask, int):
        return torch.tensor([mask], dtype=torch.int64, device=DEV), None
    bits = np.zeros(max(n, 1), dtype=np.uint8)
    m = np.asarray(mask, dtype=np.uint8)[:n]
    bits[:len(m)] = m
    return None, torch.from_numpy(bits).to(DEV)


def test_match_known_answer_tables(match_kat):
    for group in match_kat["prefix"]:
        ix, ox = BlockIndex(64), oracle.Index()
        _put(ix, ox, group["index"])
        ms = BatchMetaSearcher(ix)
        for case in group["cases"]:
            keys = torch.tensor(case["keys"], dtype=torch.int64, device=DEV)
            off = torch.tensor([0, len(case["keys"])], dtype=torch.int64, device=DEV)
            mo, mb = _mask_args(case["mask"], len(case["keys"]))
            got = ms.PrefixMatch(keys, off, mo, mb).cpu().tolist()
            assert got == [case["len"]], (group["source"], case)
    for group in match_kat["sw"]:
        ix, ox = BlockIndex(64), oracle.Index()
        _put(ix, ox, group["index"])
        ms = BatchMetaSearcher(ix)
        for case in group["cases"]:
            keys = torch.tensor(case["keys"], dtype=torch.int64, device=DEV)
            off = torch.tensor([0, len(case["keys"])], dtype=torch.int64, device=DEV)
            if case["sw"] <= 0:
                with pytest.raises(_cabi.KvcmError) as e:
                    ms.ReverseRollSlideWindowMatch(keys, off, case["sw"])
                assert e.value.code == _cabi.KVCM_EC_BADARGS
                continue
            got = ms.ReverseRollSlideWindowMatch(keys, off, case["sw"]).cpu().tolist()
            assert got == [case["base"] if case["ec"] == 0 else -2], (group["source"], case)
    for group in match_kat["batch_get"]:
        ix, ox = BlockIndex(64), oracle.Index()
        _put(ix, ox, group["index"])
        ms = BatchMetaSearcher(ix)
        for case in group["cases"]:
            flags = ms.BatchGet(torch.tensor(case["keys"], dtype=torch.int64, device=DEV)).cpu().numpy()
            assert [(int(f) & 1) == 1 for f in flags] == case["servable"]
            assert np.array_equal(flags, ox.batch_get(case["keys"]))


def test_sw_zero_window_is_rejected():
    ix = BlockIndex(8)
    k = torch.tensor([1], dtype=torch.int64, device=DEV)
    off = torch.tensor([0, 1], dtype=torch.int64, device=DEV)
    with pytest.raises(_cabi.KvcmError):
        BatchMetaSearcher(ix).ReverseRollSlideWindowMatch(k, off, 0)


def test_index_upsert_lookup_erase_and_reserved_keys():
    ix = BlockIndex(1000)
    rng = np.random.default_rng(1)
    keys = np.unique(rng.integers(-(1 << 63), (1 << 63) - 1, size=900, dtype=np.int64))
    keys = np.concatenate([keys, np.array([-(1 << 63), -(1 << 63) + 1, 0, -1], dtype=np.int64)])
    vals = rng.integers(1, 1 << 33, size=len(keys)).astype(np.int64)
    dk, dv = torch.from_numpy(keys).to(DEV), torch.from_numpy(vals).to(DEV)
    ix.upsert(dk, dv)
    ix.upsert(dk[:10], dv[:10])  # overwrite in place: live count unchanged
    slots, live = ix.stats()
    assert live == len(keys) and slots >= 2 * 1000
    got = ix.lookup(dk).cpu().numpy()
    assert np.array_equal(got.view(np.uint64), vals.view(np.uint64) | np.uint64(1 << 63))
    absent = torch.from_numpy(rng.integers(1, 1 << 62, size=100).astype(np.int64) * 2 + 1).to(DEV)
    present = np.isin(absent.cpu().numpy(), keys)
    assert np.array_equal(ix.lookup(absent).cpu().numpy() != 0, present)
    ix.erase(dk[::2])
    got = ix.lookup(dk).cpu().numpy()
    assert not got[::2].any() and (got[1::2] != 0).all()
    assert ix.stats()[1] == len(keys) - len(keys[::2])
    ix.upsert(dk[:4:2], dv[:4:2])  # re-insert after erase
    assert (ix.lookup(dk[:4]).cpu().numpy() != 0).all()
    ix.clear()
    assert ix.stats()[1] == 0 and not ix.lookup(dk).cpu().numpy().any()


def test_index_refuses_keys_beyond_capacity_without_spinning():
    ix = BlockIndex(100)  # 1024 slots, at most 896 live keys
    keys = torch.arange(1, 2001, dtype=torch.int64, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    ix.upsert(keys, None, encode_locations([(3, 4)]), status)
    torch.cuda.synchronize()
    slots, live = ix.stats()
    assert slots == 1024 and live == 896 and status[0].item() == 2000 - 896
    assert int((ix.lookup(keys) != 0).sum()) == 896


def test_duplicate_keys_in_one_batch():
    ix = BlockIndex(64)
    keys = torch.tensor([5] * 500 + [6] * 500, dtype=torch.int64, device=DEV)
    ix.upsert(keys, None, 3)
    assert ix.stats()[1] == 2


def _random_world(rng, n_index, n_req, max_len, hit_bias):
    universe = rng.integers(-(1 << 62), 1 << 62, size=n_index * 2, dtype=np.int64)
    state = rng.choice([0, 1, 2, 3], size=len(universe), p=[0.3, 0.1, 0.1, 0.5])  # absent, empty, writing, serving
    ox, ix = oracle.Index(), BlockIndex(len(universe))
    locs_by_state = {1: [], 2: [(oracle.CLS_WRITING, 1)], 3: [(oracle.CLS_SERVING, 2), (oracle.CLS_WRITING, 4)]}
    for s, locs in locs_by_state.items():
        ks = universe[state == s]
        ox.put(ks, [locs] * len(ks))
        ix.upsert(torch.from_numpy(ks).to(DEV), None, encode_locations(locs))
    lens = rng.integers(0, max_len, size=n_req)
    lens[:3] = [0, 1, max_len]
    reqs = []
    serving = universe[state == 3]
    for n in lens:
        r = rng.choice(universe, size=n)
        run = rng.random(n) < hit_bias
        r[run] = rng.choice(serving, size=int(run.sum()))
        reqs.append(r)
    keys = np.concatenate(reqs + [np.zeros(0, np.int64)])
    return ox, ix, keys, _csr(lens)


@pytest.mark.parametrize("hit_bias", [0.5, 0.97])
def test_prefix_match_random_against_oracle(hit_bias):
    rng = np.random.default_rng(int(hit_bias * 100))
    ox, ix, keys, off = _random_world(rng, 5000, 700, 300, hit_bias)
    n_req = len(off) - 1
    dk, doff = torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV)
    for weights in [(1, 3, 3, 3, 5), (1, 3, 0, 3, 5)]:
        ms = BatchMetaSearcher(ix, avail_mask_from_weights(weights))
        got = ms.PrefixMatch(dk, doff).cpu().numpy()
        want = ox.prefix_match_batch(keys, off, weights=weights, threads=4)
        assert np.array_equal(got, want)
        mask_off = rng.integers(0, 20, size=n_req).astype(np.int64)
        got = ms.PrefixMatch(dk, doff, torch.from_numpy(mask_off).to(DEV)).cpu().numpy()
        assert np.array_equal(got, ox.prefix_match_batch(keys, off, mask_off, weights=weights))
    # arbitrary (non-prefix) bool masks
    bits = (rng.random(len(keys)) < 0.2).astype(np.uint8)
    got = BatchMetaSearcher(ix).PrefixMatch(dk, doff, None, torch.from_numpy(bits).to(DEV)).cpu().numpy()
    for r in range(0, n_req, 7):
        a, b = off[r], off[r + 1]
        assert got[r] == ox.prefix_match(keys[a:b], bits[a:b].astype(bool))


@pytest.mark.parametrize("sw", [1, 2, 5, 31, 32, 33, 100])
def test_sw_match_random_against_oracle(sw):
    rng = np.random.default_rng(sw)
    ox, ix, keys, off = _random_world(rng, 3000, 500, 400, 0.96)
    dk, doff = torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV)
    got = BatchMetaSearcher(ix).ReverseRollSlideWindowMatch(dk, doff, sw).cpu().numpy()
    want = ox.sw_match_batch(keys, off, sw, threads=4)
    assert np.array_equal(got, want)
    assert (want >= 0).any() and (sw < 100 or (want == -1).any())


def test_batch_get_random_against_oracle():
    rng = np.random.default_rng(77)
    ox, ix, keys, off = _random_world(rng, 2000, 50, 200, 0.5)
    for weights in [(1, 3, 3, 3, 5), (1, 0, 0, 3, 0)]:
        got = BatchMetaSearcher(ix, avail_mask_from_weights(weights)).BatchGet(torch.from_numpy(keys).to(DEV))
        assert np.array_equal(got.cpu().numpy(), ox.batch_get(keys, weights=weights))


def test_both_matchers_from_one_look_up_per_key():
    """BatchGet once, then prefix and window match over the flag bytes: the plan for batches that ask both questions."""
    rng = np.random.default_rng(78)
    ox, ix, keys, off = _random_world(rng, 3000, 400, 300, 0.95)
    dk, doff = torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV)
    for weights in [(1, 3, 3, 3, 5), (1, 3, 0, 3, 5)]:
        ms = BatchMetaSearcher(ix, avail_mask_from_weights(weights))
        flags = ms.BatchGet(dk, out=torch.empty(len(keys), dtype=torch.uint8, device=DEV))
        mask_off = rng.integers(0, 20, size=len(off) - 1).astype(np.int64)
        got = ms.PrefixMatchFromFlags(flags, doff, torch.from_numpy(mask_off).to(DEV)).cpu().numpy()
        assert np.array_equal(got, ox.prefix_match_batch(keys, off, mask_off, weights=weights))
        for sw in (1, 7, 40):
            got = ms.ReverseRollSlideWindowMatchFromFlags(flags, doff, sw).cpu().numpy()
            assert np.array_equal(got, ox.sw_match_batch(keys, off, sw, weights=weights, threads=4))


def test_filter_write_cache_against_oracle():
    rng = np.random.default_rng(31)
    for hit_bias in (0.3, 0.9):
        ox, ix, keys, off = _random_world(rng, 3000, 400, 150, hit_bias)
        # make some requests exact "existing prefix + missing suffix" shapes
        for weights in [(1, 3, 3, 3, 5), (1, 0, 0, 3, 0)]:
            ms = BatchMetaSearcher(ix, avail_mask_from_weights(weights))
            offset, mask, n_new = (t.cpu().numpy() for t in
                                   ms.FilterWriteCache(torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV)))
            kinds = set()
            for r in range(len(off) - 1):
                a, b = off[r], off[r + 1]
                want = ox.filter_write(keys[a:b], weights=weights)
                kinds.add(want[0])
                if want[0] == "offset":
                    assert (offset[r], n_new[r]) == (want[1], want[2]), r
                else:
                    assert offset[r] == -1 and n_new[r] == want[2], r
                    assert np.array_equal(mask[a:b].astype(bool), want[1]), r
            if weights[1] > 0:  # with every storage class available both answer shapes occur
                assert kinds == {"offset", "vector"}


def test_hash_then_match_prefix_reuse_workload():
    """Shrunk version of the CPU-runnable prefix-match configuration: uint32 tokens in [0,151936), block 64,
    half of the requests reuse a random-length prefix of an earlier one, index pre-filled with prior blocks."""
    rng = np.random.default_rng(2024)
    bs, n_req = 64, 512
    prior = [rng.integers(0, 151936, size=int(rng.integers(512, 4096))).astype(np.uint32) for _ in range(64)]
    reqs = []
    for i in range(n_req):
        n = int(rng.integers(512, 4096))
        t = rng.integers(0, 151936, size=n).astype(np.uint32)
        if rng.random() < 0.5:
            src = (prior + reqs)[int(rng.integers(0, len(prior) + len(reqs)))]
            m = int(rng.integers(1, min(n, len(src)) + 1))
            t[:m] = src[:m]
        reqs.append(t)
    pk, _ = oracle.hash_blocks(np.concatenate(prior), _csr([len(p) for p in prior]), bs)
    ox, ix = oracle.Index(), BlockIndex(len(pk))
    ox.put_uniform(pk)
    ix.upsert(torch.from_numpy(pk).to(DEV), None, encode_locations([(oracle.CLS_SERVING, 4)]))
    toks, off = np.concatenate(reqs), _csr([len(r) for r in reqs])
    keys, ko = _gpu_hash(toks, off, bs)
    want_keys, _ = oracle.hash_blocks(toks, off, bs, threads=4)
    assert np.array_equal(keys, want_keys)
    got = BatchMetaSearcher(ix).PrefixMatch(torch.from_numpy(keys).to(DEV), torch.from_numpy(ko).to(DEV)).cpu().numpy()
    want = ox.prefix_match_batch(want_keys, ko, threads=4)
    assert np.array_equal(got, want) and want.max() > 0
