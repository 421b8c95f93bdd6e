"""Hash-range-sharded matching on the GPU.

The shard-local kernels are checked on one GPU by running both shards of a two-way split one after the other and
combining them with the same min / max the collectives apply.  The full NCCL path runs as two ranks when the box
has two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi
from tair_kvcache_b200.manager import CudaShardBackend, ShardedMetaSearcher, encode_locations, shard_of_keys

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _world(seed, n_ranks=2):
    rng = np.random.default_rng(seed)
    universe = rng.integers(-(1 << 62), 1 << 62, size=6000, dtype=np.int64)
    present = universe[rng.random(len(universe)) < 0.7]
    reqs = []
    for rank in range(n_ranks):
        lens = rng.integers(0, 300, size=200 + 50 * rank)
        keys = [rng.choice(universe, size=n) for n in lens]
        for k in keys:
            hit = rng.random(len(k)) < 0.95
            k[hit] = rng.choice(present, size=int(hit.sum()))
        off = np.zeros(len(lens) + 1, dtype=np.int64)
        np.cumsum(lens, out=off[1:])
        reqs.append((np.concatenate(keys + [np.zeros(0, np.int64)]), off,
                     rng.integers(0, 6, size=len(lens)).astype(np.int64)))
    return present, reqs


def test_shard_kernels_combine_to_the_unsharded_answer_on_one_gpu():
    present, reqs = _world(7)
    keys, off, mask = reqs[0]
    full = oracle.Index()
    full.put_uniform(present)
    word = encode_locations([(3, 4)])
    dk, doff, dmask = (torch.from_numpy(a).to(DEV) for a in (keys, off, mask))
    dpresent = torch.from_numpy(present).to(DEV)
    for count in (2, 3):
        shards = [CudaShardBackend(len(present), torch.device(DEV)) for _ in range(count)]
        for r, sh in enumerate(shards):
            sh.upsert_owned(dpresent, word, count, r)
        stored = [sh.index.stats()[1] for sh in shards]
        # the device ownership rule equals the host one
        assert stored == np.bincount(shard_of_keys(np.unique(present), count), minlength=count).tolist()
        lens = torch.stack([sh.prefix_owned(dk, doff, None, count, r) for r, sh in enumerate(shards)]).min(0).values
        assert np.array_equal(lens.cpu().numpy(), full.prefix_match_batch(keys, off))
        lens = torch.stack([sh.prefix_owned(dk, doff, dmask, count, r) for r, sh in enumerate(shards)]).min(0).values
        assert np.array_equal(lens.cpu().numpy(), full.prefix_match_batch(keys, off, mask))
        flags = torch.stack([sh.servable_flags(dk, count, r) for r, sh in enumerate(shards)]).max(0).values
        assert np.array_equal(flags.cpu().numpy(), full.batch_get(keys))
        for sw in (1, 4, 40):
            base = shards[0].sw_from_flags(flags, doff, sw)
            assert np.array_equal(base.cpu().numpy(), full.sw_match_batch(keys, off, sw))


def test_locally_attached_shards_answer_like_one_index():
    """Three shards in one process, attached to each other: every handle resolves each key at its owner."""
    import ctypes
    from tair_kvcache_b200.manager import BatchMetaSearcher
    present, reqs = _world(17)
    keys, off, mask = reqs[0]
    full = oracle.Index()
    full.put_uniform(present)
    dk, doff, dmask = (torch.from_numpy(a).to(DEV) for a in (keys, off, mask))
    count = 3
    shards = [CudaShardBackend(len(present), torch.device(DEV)) for _ in range(count)]
    for r, sh in enumerate(shards):
        sh.upsert_owned(torch.from_numpy(present).to(DEV), encode_locations([(3, 4)]), count, r)
    handles = (ctypes.c_void_p * count)(*[sh.index.handle.value for sh in shards])
    for r, sh in enumerate(shards):
        _cabi.call("kvcm_b200_index_attach_local_peers", sh.index.handle, count, r, handles)
    for sh in shards:
        ms = BatchMetaSearcher(sh.index)
        assert np.array_equal(ms.PrefixMatch(dk, doff).cpu().numpy(), full.prefix_match_batch(keys, off))
        assert np.array_equal(ms.PrefixMatch(dk, doff, dmask).cpu().numpy(), full.prefix_match_batch(keys, off, mask))
        assert np.array_equal(ms.ReverseRollSlideWindowMatch(dk, doff, 4).cpu().numpy(),
                              full.sw_match_batch(keys, off, 4))
        assert np.array_equal(ms.BatchGet(dk).cpu().numpy(), full.batch_get(keys))
    # writes stay local: a key stored through shard 0 is seen by all once it lands in its owner's table
    new = torch.tensor([123456789], dtype=torch.int64, device=DEV)
    owner = int(shard_of_keys(new.cpu().numpy(), count)[0])
    shards[owner].upsert_owned(new, encode_locations([(3, 4)]), count, owner)
    torch.cuda.synchronize()
    for sh in shards:
        assert sh.index.lookup(new).item() != 0
    for sh in shards:
        _cabi.call("kvcm_b200_index_detach_peers", sh.index.handle)
    assert sum(int(sh.index.lookup(new).item() != 0) for sh in shards) == 1


def test_sw_from_flags_equals_match_sw_on_the_same_index():
    present, reqs = _world(8)
    keys, off, _ = reqs[1]
    sh = CudaShardBackend(len(present), torch.device(DEV))
    sh.upsert_owned(torch.from_numpy(present).to(DEV), encode_locations([(3, 1)]), 1, 0)
    dk, doff = torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV)
    from tair_kvcache_b200.manager import BatchMetaSearcher
    for sw in (2, 33, 64):
        a = sh.sw_from_flags(sh.servable_flags(dk), doff, sw)
        b = BatchMetaSearcher(sh.index).ReverseRollSlideWindowMatch(dk, doff, sw)
        assert torch.equal(a, b)


def test_routing_kernels_dispatch_to_owners_and_combine_in_key_order():
    """Dispatch / look-up / combine with the three shards of a split held on one GPU (the transport between ranks
    is then a slice of the bucketed array)."""
    present, reqs = _world(27)
    full = oracle.Index()
    full.put_uniform(present)
    count = 3
    shards = [CudaShardBackend(len(present), torch.device(DEV)) for _ in range(count)]
    for r, sh in enumerate(shards):
        sh.upsert_owned(torch.from_numpy(present).to(DEV), encode_locations([(3, 4)]), count, r)
    for keys, off, mask in reqs:
        dk, doff, dmask = (torch.from_numpy(a).to(DEV) for a in (keys, off, mask))
        owner = shard_of_keys(keys, count)
        counts = shards[0].route_count(dk, count)
        assert counts.cpu().tolist() == np.bincount(owner, minlength=count).tolist()
        start = torch.cumsum(counts, 0, dtype=torch.int32) - counts
        cursor = start.clone()
        bucketed, pos = shards[0].route_scatter(dk, count, cursor)
        assert torch.equal(cursor, start + counts)
        p, b = pos.cpu().numpy(), bucketed.cpu().numpy()
        assert np.array_equal(np.sort(p), np.arange(len(keys)))          # a permutation
        assert np.array_equal(b[p], keys)                                 # key i sits at pos[i]
        edges = np.concatenate([start.cpu().numpy(), [len(keys)]])
        assert all(((p >= edges[s]) & (p < edges[s + 1]))[owner == s].all() for s in range(count))
        answers = torch.cat([shards[s].servable_flags(bucketed[edges[s]:edges[s + 1]].contiguous())
                             for s in range(count)])
        flags = shards[0].gather_bytes(answers, pos)
        assert np.array_equal(flags.cpu().numpy(), full.batch_get(keys))
        assert np.array_equal(shards[0].prefix_from_flags(flags, doff, None).cpu().numpy(),
                              full.prefix_match_batch(keys, off))
        assert np.array_equal(shards[0].prefix_from_flags(flags, doff, dmask).cpu().numpy(),
                              full.prefix_match_batch(keys, off, mask))
    # an empty batch is a no-op with zero counts
    none = torch.zeros(0, dtype=torch.int64, device=DEV)
    assert shards[0].route_count(none, count).cpu().tolist() == [0] * count
    assert shards[0].route_scatter(none, count, torch.zeros(count, dtype=torch.int32, device=DEV))[1].numel() == 0


def test_peer_memory_exchange_between_areas_of_one_process():
    """Three ranks' exchange areas on one GPU, attached to each other: dispatch of every rank, then answer of every
    rank, then collect, as the ranks of a box do between their meeting points."""
    import ctypes
    present, _ = _world(37)
    rng = np.random.default_rng(5)
    full = oracle.Index()
    full.put_uniform(present)
    count = 3
    shards = [CudaShardBackend(len(present), torch.device(DEV)) for _ in range(count)]
    for r, sh in enumerate(shards):
        sh.upsert_owned(torch.from_numpy(present).to(DEV), encode_locations([(3, 4)]), count, r)
    areas = [sh.route_area_create(9000) for sh in shards]
    handles = (ctypes.c_void_p * count)(*[a.value for a in areas])
    for r, a in enumerate(areas):
        _cabi.call("kvcm_b200_route_area_attach_local", a, count, r, handles)
    for sizes in ((5000, 0, 7777), (1, 2, 3), (9000, 9000, 4096), (9216, 9216, 9216), (9216, 9216, 9100)):
        batches = []
        for n in sizes:  # ragged batches: hits, misses and repeated keys
            k = rng.choice(present, size=n)
            miss = rng.random(n) < 0.3
            k[miss] = rng.integers(-(1 << 62), 1 << 62, size=int(miss.sum()), dtype=np.int64)
            batches.append(k)
        dks = [torch.from_numpy(k).to(DEV) for k in batches]
        matrix = np.stack([sh.route_count(dk, count).cpu().numpy() for sh, dk in zip(shards, dks)]).astype(np.uint32)
        if matrix.sum(0).max() > 9216:  # an inbox would overflow: refused on every rank, nothing launched
            with pytest.raises(_cabi.KvcmError):
                shards[0].route_dispatch(areas[0], dks[0], matrix)
            continue
        pos = [sh.route_dispatch(a, dk, matrix) for sh, a, dk in zip(shards, areas, dks)]
        for sh, a in zip(shards, areas):
            sh.route_answer(a, matrix)
        for r, (sh, a) in enumerate(zip(shards, areas)):
            flags = sh.route_collect(a, pos[r])
            assert np.array_equal(flags.cpu().numpy(), full.batch_get(batches[r]))
            p = pos[r].cpu().numpy()
            assert np.array_equal(np.sort(p), np.arange(len(p)))
    torch.cuda.synchronize()
    for a in areas:
        _cabi.call("kvcm_b200_route_area_detach", a)
    for sh, a in zip(shards, areas):
        sh.route_area_destroy(a)


def _rank_main(rank, port, results, mode):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=2, device_id=dev)
    try:
        present, reqs = _world(9)
        searcher = ShardedMetaSearcher(CudaShardBackend(len(present), dev), mode=mode, route_capacity=1 << 16)
        searcher.upsert(torch.from_numpy(present[rank::2].copy()).to(dev), encode_locations([(3, 4)]))
        keys, off, mask = (torch.from_numpy(a).to(dev) for a in reqs[rank])
        out = {
            "stored": searcher.backend.index.stats()[1],
            "prefix": searcher.PrefixMatch(keys, off).cpu().numpy(),
            "prefix_masked": searcher.PrefixMatch(keys, off, mask).cpu().numpy(),
            "sw4": searcher.ReverseRollSlideWindowMatch(keys, off, sw_size=4).cpu().numpy(),
        }
        if mode in ("route", "route_peer"):  # one dispatch / combine serves both queries
            routed = searcher.Route(keys, off, mask)
            assert np.array_equal(searcher.PrefixMatch(routed).cpu().numpy(), out["prefix_masked"])
            assert np.array_equal(searcher.ReverseRollSlideWindowMatch(routed, sw_size=4).cpu().numpy(), out["sw4"])
        torch.cuda.synchronize()
        results[rank] = out
        if mode == "peer":
            searcher.detach_peers()  # nobody frees a shard while a peer still maps it
        if mode == "route_peer":
            searcher.detach_route_areas()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["exchange", "peer", "route", "route_peer"])
def test_two_nccl_ranks_match_the_unsharded_oracle(mode):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_rank_main, args=(port, results, mode), nprocs=2, join=True)
        results = dict(results)
    present, reqs = _world(9)
    full = oracle.Index()
    full.put_uniform(present)
    assert results[0]["stored"] + results[1]["stored"] == len(np.unique(present))
    for rank in range(2):
        keys, off, mask = reqs[rank]
        assert np.array_equal(results[rank]["prefix"], full.prefix_match_batch(keys, off))
        assert np.array_equal(results[rank]["prefix_masked"], full.prefix_match_batch(keys, off, mask))
        assert np.array_equal(results[rank]["sw4"], full.sw_match_batch(keys, off, 4))


def _write_world(seed, n_ranks):
    """Per rank a few requests that share keys within and across ranks, over an index that already holds served,
    half-written and nothing-writable keys."""
    rng = np.random.default_rng(seed)
    universe = np.unique(rng.integers(-(1 << 62), 1 << 62, size=2500, dtype=np.int64))
    held = universe[rng.permutation(len(universe))[:700]]
    maps = [[(oracle.CLS_SERVING, 4)] if j % 3 else ([(oracle.CLS_WRITING, 2)] if j % 2 else
                                                      [(oracle.CLS_NOT_FOUND, 1)]) for j in range(len(held))]
    reqs = []
    for rank in range(n_ranks):
        mine = []
        for _ in range(60 + 10 * rank):
            n = int(rng.integers(0, 30))
            r = rng.choice(universe, size=n, replace=False)
            everyone = [q for per_rank in reqs for q in per_rank] + mine
            if everyone and rng.random() < 0.7:
                src = everyone[int(rng.integers(len(everyone)))]
                m = int(rng.integers(0, min(len(src), n) + 1))
                r = np.concatenate([src[:m], r[~np.isin(r, src[:m])]])[:max(n, m)]
            mine.append(r.astype(np.int64))
        reqs.append(mine)
    return universe, held, maps, reqs


def _serve_in_order(ox, reqs, cls, success):
    """The reference's order of events over all ranks' requests: (rank, request), filter then add; then every session
    finishes with its success offset."""
    want = []
    for per_rank in reqs:
        for r in per_rank:
            kind, what, n_new = ox.filter_write(r)
            new = r[what:] if kind == "offset" else r[~what]
            free = np.array([all(t != cls for _, t in (ox.get(int(k)) or [])) for k in new], dtype=bool)
            ox.add_location(new[free], cls, oracle.CLS_WRITING)
            want.append((kind, what, n_new, new[free]))
    for (kind, what, n_new, new), s in zip(want, success):
        good = np.arange(len(new)) < s
        ox.update_status(new[good], cls, -1, oracle.CLS_SERVING)
        ox.update_status(new[~good], cls, -1, -1)
    return want


def test_sharded_write_batch_on_one_gpu():
    """Three shards in one process, the collectives replaced by what they compute (concatenation, bytewise maximum):
    every shard answers alike, and together the shards hold what the unsharded oracle holds after serving the same
    requests in order."""
    from test_gpu_index_write import _decode
    count = 3
    universe, held, maps, reqs = _write_world(31, count)
    ox = oracle.Index()
    ox.put(held, maps)
    shards = [CudaShardBackend(len(universe), torch.device(DEV)) for _ in range(count)]
    words = torch.tensor([encode_locations(m) for m in maps], dtype=torch.int64, device=DEV)
    for r, sh in enumerate(shards):
        _cabi.call("kvcm_b200_index_upsert_sharded", sh.index.handle, torch.from_numpy(held).to(DEV).data_ptr(),
                   words.data_ptr(), 0, len(held), count, r, None, sh.index._s())
    flat = [q for per_rank in reqs for q in per_rank]
    off = np.zeros(len(flat) + 1, dtype=np.int64)
    np.cumsum([len(q) for q in flat], out=off[1:])
    keys = np.concatenate(flat + [np.zeros(0, np.int64)])
    dk, doff = torch.from_numpy(keys).to(DEV), torch.from_numpy(off).to(DEV)
    flags = torch.stack([sh.write_snapshot(dk, 4, count, r) for r, sh in enumerate(shards)]).max(0).values
    outs = [sh.start_write_owned(dk, doff, flags, None, 4, count, r) for r, sh in enumerate(shards)]
    for o in outs[1:]:  # every shard gives the same answers
        for a, b in zip(outs[0], o):
            assert torch.equal(a, b)
    offset, mask, n_new, added, new_off = (t.cpu().numpy() for t in outs[0])
    rng = np.random.default_rng(5)
    lens = new_off[1:] - new_off[:-1]
    success = np.array([int(rng.integers(0, n + 1)) for n in lens], dtype=np.int64)
    want = _serve_in_order(ox, reqs, 4, success)
    kinds = set()
    for r, (kind, what, n, new) in enumerate(want):
        a, b = off[r], off[r + 1]
        kinds.add(kind)
        assert n_new[r] == n
        if kind == "offset":
            assert offset[r] == what
        else:
            assert offset[r] == -1 and np.array_equal(mask[a:b].astype(bool), what)
        assert np.array_equal(flat[r][added[a:b].astype(bool)], new), r
    assert kinds == {"offset", "vector"}
    codes = torch.stack([sh.finish_write_owned(dk, doff, outs[0][3], outs[0][4], torch.from_numpy(success).to(DEV), 4,
                                               count, r) for r, sh in enumerate(shards)]).max(0).values
    assert not codes.cpu().numpy().any()
    # together the shards hold the oracle's maps, each key on its owner only
    du = torch.from_numpy(universe).to(DEV)
    words = torch.stack([sh.index.lookup(du) for sh in shards]).cpu().numpy()
    owner = shard_of_keys(universe, count)
    for j, k in enumerate(universe):
        want_map = ox.get(int(k))
        for r in range(count):
            have = _decode(words[r][j])
            if r != owner[j]:
                assert have is None
            else:
                assert (have is None) == (want_map is None) and (want_map is None or sorted(have) == sorted(want_map)), k
    assert sum(sh.index.stats()[1] for sh in shards) == len(ox)


def _write_rank_main(rank, port, results):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=2, device_id=dev)
    try:
        universe, held, maps, reqs = _write_world(33, 2)
        searcher = ShardedMetaSearcher(CudaShardBackend(len(universe), dev), mode="exchange")
        words = torch.tensor([encode_locations(m) for m in maps], dtype=torch.int64, device=dev)
        _cabi.call("kvcm_b200_index_upsert_sharded", searcher.backend.index.handle,
                   torch.from_numpy(held).to(dev).data_ptr(), words.data_ptr(), 0, len(held), 2, rank, None,
                   searcher.backend.index._s())
        mine = reqs[rank]
        off = np.zeros(len(mine) + 1, dtype=np.int64)
        np.cumsum([len(q) for q in mine], out=off[1:])
        keys = np.concatenate(mine + [np.zeros(0, np.int64)])
        s = searcher.StartWriteCache(torch.from_numpy(keys).to(dev), torch.from_numpy(off).to(dev), 4)
        lens = s.session_lengths.cpu().numpy()
        success = (lens + 1) // 2
        codes = searcher.FinishWriteCache(s, torch.from_numpy(success.astype(np.int64)).to(dev))
        prefix = searcher.PrefixMatch(torch.from_numpy(keys).to(dev), torch.from_numpy(off).to(dev))
        torch.cuda.synchronize()
        results[rank] = dict(offset=s.offset.cpu().numpy(), mask=s.mask.cpu().numpy(), n_new=s.n_new.cpu().numpy(),
                             added=s.added.cpu().numpy(), lens=lens, codes=codes.cpu().numpy(),
                             prefix=prefix.cpu().numpy(), stored=searcher.backend.index.stats()[1])
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_nccl_ranks_write_batch():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_write_rank_main, args=(port, results), nprocs=2, join=True)
        results = dict(results)
    universe, held, maps, reqs = _write_world(33, 2)
    ox = oracle.Index()
    ox.put(held, maps)
    success = np.concatenate([(results[r]["lens"] + 1) // 2 for r in range(2)])
    want = _serve_in_order(ox, reqs, 4, success)
    at = 0
    for rank in range(2):
        res, k0 = results[rank], 0
        assert not res["codes"].any()
        for j, r in enumerate(reqs[rank]):
            kind, what, n, new = want[at]
            assert res["n_new"][j] == n and res["lens"][j] == len(new)
            if kind == "offset":
                assert res["offset"][j] == what
            else:
                assert res["offset"][j] == -1 and np.array_equal(res["mask"][k0:k0 + len(r)].astype(bool), what)
            assert np.array_equal(r[res["added"][k0:k0 + len(r)].astype(bool)], new)
            k0 += len(r)
            at += 1
        flat = np.concatenate(reqs[rank] + [np.zeros(0, np.int64)])
        off = np.zeros(len(reqs[rank]) + 1, dtype=np.int64)
        np.cumsum([len(q) for q in reqs[rank]], out=off[1:])
        assert np.array_equal(res["prefix"], ox.prefix_match_batch(flat, off))
    assert results[0]["stored"] + results[1]["stored"] == len(ox)
