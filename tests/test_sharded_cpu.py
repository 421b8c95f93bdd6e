"""The multi-rank logic of the hash-range-sharded matcher on CPU: two gloo ranks, the shard-local work done by
an oracle-backed stand-in (test only), results compared with the unsharded oracle."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.manager.sharded_searcher import ShardedMetaSearcher, shard_of_keys


class OracleShardBackend:
    """CPU stand-in for CudaShardBackend, for tests only: same four operations through the oracle."""

    def __init__(self):
        self.index = oracle.Index()
        self.device = torch.device("cpu")

    def upsert_owned(self, keys, value_word, shard_count, shard_rank):
        k = keys.numpy()
        self.index.put_uniform(k[shard_of_keys(k, shard_count) == shard_rank])

    def prefix_owned(self, keys, key_off, mask_off, shard_count, shard_rank):
        k, off = keys.numpy(), key_off.numpy()
        owner = shard_of_keys(k, shard_count)
        flags = self.index.batch_get(k) & 1
        ok = (owner != shard_rank) | (flags == 1)
        out = np.zeros(len(off) - 1, dtype=np.int32)
        for r in range(len(off) - 1):
            skip = int(mask_off[r]) if mask_off is not None else 0
            n = 0
            for i in range(off[r] + skip, off[r + 1]):
                if not ok[i]:
                    break
                n += 1
            out[r] = n
        return torch.from_numpy(out)

    def servable_flags(self, keys, shard_count=1, shard_rank=0):
        return torch.from_numpy(self.index.batch_get(keys.numpy()))

    # ---- the write side: the same contract as CudaShardBackend, served request after request ----
    def write_snapshot(self, keys, storage_class, shard_count, shard_rank):
        k = keys.numpy()
        flags = self.index.batch_get(k).astype(np.uint8)
        for i, key in enumerate(k):
            if any(t == storage_class for _, t in (self.index.get(int(key)) or [])):
                flags[i] |= 16
        flags[shard_of_keys(k, shard_count) != shard_rank] = 0
        return torch.from_numpy(flags)

    def start_write_owned(self, keys, key_off, flags, skip, storage_class, shard_count, shard_rank, table_full=None):
        k, off, f = keys.numpy(), key_off.numpy(), flags.numpy()
        n_req = len(off) - 1
        owner = shard_of_keys(k, shard_count)
        offset, n_new = np.zeros(n_req, np.int32), np.zeros(n_req, np.int32)
        mask, added = np.zeros(len(k), np.uint8), np.zeros(len(k), np.uint8)
        written = set()  # keys that got their location from a request served before
        for r in range(n_req):
            if skip is not None and skip[r]:
                continue
            a, b = off[r], off[r + 1]
            exists = np.array([bool(f[i] & 8) or int(k[i]) in written for i in range(a, b)], dtype=bool)
            nonempty = np.array([bool(f[i] & 4) or int(k[i]) in written for i in range(a, b)], dtype=bool)
            mask[a:b] = nonempty
            first = int(np.argmin(exists)) if not exists.all() else b - a
            if not exists[first:].any():
                offset[r], new = first, np.arange(first, b - a)
            else:
                offset[r], new = -1, np.flatnonzero(~nonempty)
            n_new[r] = len(new)
            for i in new + a:
                if f[i] & 16:
                    continue
                added[i] = 1
                written.add(int(k[i]))
                if owner[i] == shard_rank:
                    self.index.add_location([k[i]], storage_class, oracle.CLS_WRITING)
        new_off = np.zeros(n_req + 1, np.int64)
        np.cumsum([added[off[r]:off[r + 1]].sum() for r in range(n_req)], out=new_off[1:])
        return tuple(torch.from_numpy(x) for x in (offset, mask, n_new, added, new_off))

    def finish_write_owned(self, keys, key_off, added, new_off, success_off, storage_class, shard_count, shard_rank):
        k, off, ad = keys.numpy(), key_off.numpy(), added.numpy().astype(bool)
        owner = shard_of_keys(k, shard_count)
        for r in range(len(off) - 1):
            session = np.flatnonzero(ad[off[r]:off[r + 1]]) + off[r]
            for j, i in enumerate(session):
                if owner[i] == shard_rank:
                    self.index.update_status([k[i]], storage_class, -1,
                                             oracle.CLS_SERVING if j < int(success_off[r]) else -1)
        return torch.zeros(len(off) - 1, dtype=torch.int32)

    def prefix_from_flags(self, flags, key_off, mask_off):
        f, off = flags.numpy() & 1, key_off.numpy()
        out = np.zeros(len(off) - 1, dtype=np.int32)
        for r in range(len(off) - 1):
            skip = int(mask_off[r]) if mask_off is not None else 0
            seg = f[off[r] + skip:off[r + 1]]
            out[r] = len(seg) if seg.all() else int(np.argmin(seg))
        return torch.from_numpy(out)

    def route_count(self, keys, shard_count):
        return torch.from_numpy(np.bincount(shard_of_keys(keys.numpy(), shard_count),
                                            minlength=shard_count).astype(np.int32))

    def route_scatter(self, keys, shard_count, cursor):
        k = keys.numpy()
        order = np.argsort(shard_of_keys(k, shard_count), kind="stable")
        pos = np.empty(len(k), dtype=np.int32)
        pos[order] = np.arange(len(k), dtype=np.int32)
        return torch.from_numpy(k[order].copy()), torch.from_numpy(pos)

    def gather_bytes(self, src, pos):
        return torch.from_numpy(src.numpy()[pos.numpy()].copy())

    def sw_from_flags(self, flags, key_off, sw):
        f, off = flags.numpy() & 1, key_off.numpy()
        out = np.full(len(off) - 1, -1, dtype=np.int32)
        for r in range(len(off) - 1):
            seg = f[off[r]:off[r + 1]]
            if len(seg) < sw:
                out[r] = -2
                continue
            for base in range(len(seg) - sw, -1, -1):
                if seg[base:base + sw].all():
                    out[r] = base
                    break
        return torch.from_numpy(out)


def _world(seed):
    rng = np.random.default_rng(seed)
    universe = rng.integers(-(1 << 62), 1 << 62, size=600, dtype=np.int64)
    present = universe[rng.random(600) < 0.7]
    reqs = {}
    for rank in range(2):
        lens = rng.integers(0, 40, size=5 + 3 * rank)
        keys = [rng.choice(universe, size=n) for n in lens]
        for k in keys:  # long servable runs so windows exist
            hit = rng.random(len(k)) < 0.8
            k[hit] = rng.choice(present, size=int(hit.sum()))
        off = np.zeros(len(lens) + 1, dtype=np.int64)
        np.cumsum(lens, out=off[1:])
        mask = rng.integers(0, 4, size=len(lens)).astype(np.int64)
        reqs[rank] = (np.concatenate(keys + [np.zeros(0, np.int64)]), off, mask)
    return present, reqs


def _rank_main(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    try:
        present, reqs = _world(123)
        searcher = ShardedMetaSearcher(OracleShardBackend())
        # each rank submits half of the index content; ownership decides where a key is stored
        searcher.upsert(torch.from_numpy(present[rank::2].copy()), 0)
        keys, off, mask = reqs[rank]
        tk, to, tm = torch.from_numpy(keys), torch.from_numpy(off), torch.from_numpy(mask)
        out = {
            "stored": len(searcher.backend.index),
            "prefix": searcher.PrefixMatch(tk, to).numpy().copy(),
            "prefix_masked": searcher.PrefixMatch(tk, to, tm).numpy().copy(),
            "sw2": searcher.ReverseRollSlideWindowMatch(tk, to, 2).numpy().copy(),
            "sw5": searcher.ReverseRollSlideWindowMatch(tk, to, 5).numpy().copy(),
        }
        g = searcher.Gather(tk, to, tm)  # one exchange, two queries
        assert np.array_equal(searcher.PrefixMatch(g).numpy(), out["prefix_masked"])
        assert np.array_equal(searcher.ReverseRollSlideWindowMatch(g, sw_size=5).numpy(), out["sw5"])
        routed = ShardedMetaSearcher(searcher.backend, mode="route")
        assert np.array_equal(routed.PrefixMatch(tk, to).numpy(), out["prefix"])
        assert np.array_equal(routed.PrefixMatch(tk, to, tm).numpy(), out["prefix_masked"])
        assert np.array_equal(routed.ReverseRollSlideWindowMatch(tk, to, 2).numpy(), out["sw2"])
        r = routed.Route(tk, to, tm)  # one dispatch / combine, two queries
        assert np.array_equal(routed.PrefixMatch(r).numpy(), out["prefix_masked"])
        assert np.array_equal(routed.ReverseRollSlideWindowMatch(r, sw_size=5).numpy(), out["sw5"])
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_the_unsharded_oracle():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_rank_main, args=(port, results), nprocs=2, join=True)
        results = dict(results)
    present, reqs = _world(123)
    full = oracle.Index()
    full.put_uniform(present)
    assert results[0]["stored"] + results[1]["stored"] == len(np.unique(present))
    assert results[0]["stored"] > 0 and results[1]["stored"] > 0
    for rank in range(2):
        keys, off, mask = reqs[rank]
        assert np.array_equal(results[rank]["prefix"], full.prefix_match_batch(keys, off))
        assert np.array_equal(results[rank]["prefix_masked"], full.prefix_match_batch(keys, off, mask))
        assert np.array_equal(results[rank]["sw2"], full.sw_match_batch(keys, off, 2))
        assert np.array_equal(results[rank]["sw5"], full.sw_match_batch(keys, off, 5))
    assert (results[0]["sw2"] >= 0).any() and results[0]["prefix"].max() > 0


def test_shard_of_keys_is_a_balanced_partition():
    rng = np.random.default_rng(0)
    keys = rng.integers(-(1 << 63), (1 << 63) - 1, size=4000, dtype=np.int64)
    for count in (1, 2, 8):
        owner = shard_of_keys(keys, count)
        assert owner.min() >= 0 and owner.max() < count
        assert np.bincount(owner, minlength=count).min() > 4000 / count * 0.8
    # chained block hashes of consecutive blocks spread too
    chain = oracle.gen_key_vector(np.arange(64 * 800, dtype=np.int64), 64)
    assert np.bincount(shard_of_keys(chain, 8), minlength=8).min() > 60


def _write_rank_main(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    try:
        universe, held, reqs = _write_world()
        searcher = ShardedMetaSearcher(OracleShardBackend())
        searcher.upsert(torch.from_numpy(held[rank::2].copy()), 0)
        mine = reqs[rank]
        off = np.zeros(len(mine) + 1, dtype=np.int64)
        np.cumsum([len(q) for q in mine], out=off[1:])
        keys = np.concatenate(mine + [np.zeros(0, np.int64)])
        s = searcher.StartWriteCache(torch.from_numpy(keys), torch.from_numpy(off), 4)
        lens = s.session_lengths.numpy().copy()
        codes = searcher.FinishWriteCache(s, torch.from_numpy((lens + 1) // 2))
        prefix = searcher.PrefixMatch(torch.from_numpy(keys), torch.from_numpy(off))
        results[rank] = dict(offset=s.offset.numpy().copy(), mask=s.mask.numpy().copy(), n_new=s.n_new.numpy().copy(),
                             added=s.added.numpy().copy(), lens=lens, codes=codes.numpy().copy(),
                             prefix=prefix.numpy().copy(), stored=len(searcher.backend.index))
    finally:
        dist.destroy_process_group()


def _write_world():
    rng = np.random.default_rng(321)
    universe = np.unique(rng.integers(-(1 << 62), 1 << 62, size=300, dtype=np.int64))
    held = universe[rng.permutation(len(universe))[:80]]
    reqs = {0: [], 1: []}
    for rank in range(2):
        for _ in range(6 + 3 * rank):
            n = int(rng.integers(0, 12))
            r = rng.choice(universe, size=n, replace=False)
            everyone = reqs[0] + reqs[1]
            if everyone and rng.random() < 0.7:
                src = everyone[int(rng.integers(len(everyone)))]
                m = int(rng.integers(0, min(len(src), n) + 1))
                r = np.concatenate([src[:m], r[~np.isin(r, src[:m])]])[:max(n, m)]
            reqs[rank].append(r.astype(np.int64))
    return universe, held, reqs


def test_two_gloo_ranks_write_batch():
    """StartWriteCache / FinishWriteCache over two ranks: the gathering, the padding entries, the all-reduce of the
    owners' flags and the slicing of each rank's answers, against the unsharded oracle serving all requests in the
    order (rank, request)."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_write_rank_main, args=(port, results), nprocs=2, join=True)
        results = dict(results)
    universe, held, reqs = _write_world()
    ox = oracle.Index()
    ox.put_uniform(held)
    want = []
    for rank in range(2):
        for r in reqs[rank]:
            kind, what, n_new = ox.filter_write(r)
            new = r[what:] if kind == "offset" else r[~what]
            ox.add_location(new, 4, oracle.CLS_WRITING)
            want.append((kind, what, n_new, new))
    at, kinds = 0, set()
    for rank in range(2):
        res, k0 = results[rank], 0
        assert not res["codes"].any()
        for j, r in enumerate(reqs[rank]):
            kind, what, n, new = want[at]
            kinds.add(kind)
            assert res["n_new"][j] == n and res["lens"][j] == len(new)
            if kind == "offset":
                assert res["offset"][j] == what
            else:
                assert res["offset"][j] == -1 and np.array_equal(res["mask"][k0:k0 + len(r)].astype(bool), what)
            assert np.array_equal(r[res["added"][k0:k0 + len(r)].astype(bool)], new)
            k0 += len(r)
            at += 1
    for (kind, what, n, new) in want:
        good = np.arange(len(new)) < (len(new) + 1) // 2
        ox.update_status(new[good], 4, -1, oracle.CLS_SERVING)
        ox.update_status(new[~good], 4, -1, -1)
    for rank in range(2):
        flat = np.concatenate(reqs[rank] + [np.zeros(0, np.int64)])
        off = np.zeros(len(reqs[rank]) + 1, dtype=np.int64)
        np.cumsum([len(q) for q in reqs[rank]], out=off[1:])
        assert np.array_equal(results[rank]["prefix"], ox.prefix_match_batch(flat, off))
    assert results[0]["stored"] + results[1]["stored"] == len(ox) and kinds == {"offset", "vector"}
