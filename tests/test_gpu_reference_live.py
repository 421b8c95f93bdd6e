"""The CUDA path against the REFERENCE itself, with nothing in between: where the reference's MetaSearcher compiled
from its own sources has travelled with the build (oracle/_ref/libkvcm_ref_searcher.so), the same token batches go
through its GenKeyVector + PrefixMatch + ReverseRollSlideWindowMatch on the host and through the kernels, and the
same StartWriteCache / FinishWriteCache requests are served by the reference one after the other and by the kernels
as one batch.  (Everywhere else the kernels are compared with the oracle, and the oracle with the reference.)"""
import numpy as np
import pytest
import torch

from oracle import kvcm_oracle as oracle
from oracle import ref_searcher as ref

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200 import _cabi
from tair_kvcache_b200.manager import BatchMetaSearcher, BlockIndex, GenKeyVectorBatch, encode_locations, key_offsets

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref.available(),
                                                  reason="oracle/_ref/libkvcm_ref_searcher.so not built")]
DEV = "cuda:0"


def _token_batch(rng, n_prior, n_req, max_tokens):
    prior = [rng.integers(0, 151936, size=int(rng.integers(64, max_tokens))).astype(np.int64) for _ in range(n_prior)]
    reqs = []
    for _ in range(n_req):
        t = rng.integers(0, 151936, size=int(rng.integers(0, max_tokens))).astype(np.int64)
        if rng.random() < 0.7:
            src = prior[int(rng.integers(len(prior)))]
            m = int(rng.integers(0, min(len(t), len(src)) + 1))
            t[:m] = src[:m]
        reqs.append(t)

    def csr(seqs):
        off = np.zeros(len(seqs) + 1, dtype=np.int64)
        np.cumsum([len(x) for x in seqs], out=off[1:])
        return np.concatenate(seqs + [np.zeros(0, np.int64)]), off

    return csr(prior), csr(reqs)


@pytest.mark.parametrize("bs", [16, 64])
def test_hash_prefix_and_window_match_of_token_batches(bs):
    rng = np.random.default_rng(50 + bs)
    (ptoks, poff), (toks, off) = _token_batch(rng, 150, 600, 3000)
    dev = torch.device(DEV)

    def gpu_keys(t, o):
        ko = key_offsets(o, bs)
        return GenKeyVectorBatch(torch.from_numpy(t).to(dev), torch.from_numpy(o).to(dev), bs,
                                 torch.from_numpy(ko).to(dev), int(ko[-1])), torch.from_numpy(ko).to(dev)

    pkeys, _ = gpu_keys(ptoks, poff)
    pkeys = torch.unique(pkeys)
    # the index: the prior prompts' blocks, a tenth of them only being written (in the index, not servable)
    n_writing = pkeys.numel() // 10
    r = ref.RefSearcher(max_keys=4 * pkeys.numel(), in_memory=True)
    host_keys = pkeys.cpu().numpy()
    r.add(host_keys[n_writing:], 4, oracle.CLS_SERVING)
    r.add(host_keys[:n_writing], 2, oracle.CLS_WRITING)
    index = BlockIndex(pkeys.numel(), dev)
    index.upsert(pkeys[n_writing:], None, encode_locations([(oracle.CLS_SERVING, 4)]))
    index.upsert(pkeys[:n_writing], None, encode_locations([(oracle.CLS_WRITING, 2)]))
    ms = BatchMetaSearcher(index)
    keys, ko = gpu_keys(toks, off)
    got_prefix = ms.PrefixMatch(keys, ko).cpu().numpy()
    for sw in (1, 4):
        want_prefix, want_base = r.window_match_batch(toks, off, bs, sw, threads=4)
        assert np.array_equal(got_prefix, want_prefix)
        assert np.array_equal(ms.ReverseRollSlideWindowMatch(keys, ko, sw).cpu().numpy(), want_base)
        assert (want_base >= 0).any() and (want_base == -1).any() and (want_base == -2).any()
    assert got_prefix.sum() > 1000
    servable, nonempty = r.batch_get(keys.cpu().numpy())
    flags = ms.BatchGet(keys).cpu().numpy()[:keys.numel()]
    assert np.array_equal(flags & _cabi.FLAG_SERVABLE, servable)
    assert np.array_equal((flags & _cabi.FLAG_NONEMPTY) != 0, nonempty.astype(bool))


def test_write_batches_against_the_reference_serving_the_requests_in_order():
    rng = np.random.default_rng(77)
    universe = np.unique(rng.integers(-(1 << 62), 1 << 62, size=1500, dtype=np.int64))
    held = universe[rng.permutation(len(universe))[:400]]
    r = ref.RefSearcher(max_keys=4 * len(universe), in_memory=True)
    r.add(held[:300], 4, oracle.CLS_SERVING)
    r.add(held[300:], 2, oracle.CLS_WRITING)
    dev = torch.device(DEV)
    index = BlockIndex(len(universe), dev)
    index.upsert(torch.from_numpy(held[:300]).to(dev), None, encode_locations([(oracle.CLS_SERVING, 4)]))
    index.upsert(torch.from_numpy(held[300:]).to(dev), None, encode_locations([(oracle.CLS_WRITING, 2)]))
    ms = BatchMetaSearcher(index)
    forms = set()
    for round_no in range(4):
        reqs = []
        for _ in range(120):
            n = int(rng.integers(0, 25))
            q = rng.choice(universe, size=n, replace=False)
            if reqs and rng.random() < 0.7:
                src = reqs[int(rng.integers(len(reqs)))]
                m = int(rng.integers(0, min(len(src), n) + 1))
                q = np.concatenate([src[:m], q[~np.isin(q, src[:m])]])[:max(n, m)]
            reqs.append(q.astype(np.int64))
        off = np.zeros(len(reqs) + 1, dtype=np.int64)
        np.cumsum([len(q) for q in reqs], out=off[1:])
        keys = np.concatenate(reqs + [np.zeros(0, np.int64)])
        s = ms.StartWriteCache(torch.from_numpy(keys).to(dev), torch.from_numpy(off).to(dev), 4)
        offset, mask, n_new, added = (t.cpu().numpy() for t in s[:4])
        sessions = []
        for j, q in enumerate(reqs):  # the reference: FilterWriteCache, then BatchAddLocation, request after request
            kind, what, n = r.filter_write(q)
            forms.add(kind)
            new = q[what:] if kind == "offset" else q[~what]
            if len(new):
                r.add(new, 4, oracle.CLS_WRITING)
            a, b = off[j], off[j + 1]
            assert n_new[j] == n
            if kind == "offset":
                assert offset[j] == what
            else:
                assert offset[j] == -1 and np.array_equal(mask[a:b].astype(bool), what)
            assert np.array_equal(q[added[a:b].astype(bool)], new)
            sessions.append(new)
        lens = np.array([len(x) for x in sessions], dtype=np.int64)
        success = (lens + 1) // 2
        codes = ms.FinishWriteCache(s, success_off=torch.from_numpy(success).to(dev)).cpu().numpy()
        assert not codes.any()
        for new, ok in zip(sessions, success):  # FinishWriteCache: served inside the mask, removed outside it
            if ok:
                rc, res = r.status(ref.OP_UPDATE, new[:ok], np.full(ok, 4, np.int32), np.zeros(ok, np.int32),
                                   np.full(ok, oracle.CLS_SERVING, np.int32))
                assert not res.any()
            if len(new) > ok:
                m = len(new) - ok
                rc, res = r.status(ref.OP_CAD, new[ok:], np.full(m, 4, np.int32),
                                   np.full(m, oracle.CLS_WRITING, np.int32), np.zeros(m, np.int32))
                assert not res.any()
        servable, nonempty = r.batch_get(universe)
        flags = ms.BatchGet(torch.from_numpy(universe).to(dev)).cpu().numpy()[:len(universe)]
        assert np.array_equal(flags & _cabi.FLAG_SERVABLE, servable), round_no
        assert np.array_equal((flags & _cabi.FLAG_NONEMPTY) != 0, nonempty.astype(bool)), round_no
    assert forms == {"offset", "vector"}
