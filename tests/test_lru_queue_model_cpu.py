"""The per-key model behind the LRU sweep kernels, written out sequentially, against the oracle's radix trees.

The CUDA kernels of tair-kvcache_b200/csrc/replay_lru.cu keep no tree.  Per configuration they keep a stamp per key
(0 = not cached, else the sequence number of its last write or access) and an append-only queue of (key, stamp)
entries per instance; an entry is live while it still carries its key's current stamp, and the reference's recency
list (kv_cache_manager/optimizer/eviction_policy/lru.cc) is the live entries in queue order.  For a group of
instances that share a quota (kv_cache_manager/optimizer/manager/eviction_manager.cc:86-239) the kernel first works
out, from the usages alone, how many blocks every instance loses, and then pops that many live entries per instance.
This file restates that model in plain Python and compares it with the oracle, which keeps a compressed radix tree
and a real list per instance and plays the reference's eviction rounds one by one - on a box without a GPU.
"""
import numpy as np
import pytest

from oracle import kvcm_oracle as oracle

W, G, D = oracle.TRACE_WRITE_CACHE, oracle.TRACE_GET_LOCATION, oracle.TRACE_DIALOG_TURN


def queue_replay(keys, off, types, mask_off, inst, n_inst, quota, batch, mode):
    stamp = {}                                  # (instance, key) -> stamp of the last write or access
    queue = [[] for _ in range(n_inst)]         # per instance: (key, stamp), oldest first
    head = [0] * n_inst
    usage = [0] * n_inst
    counter = 0
    out = []
    for t in range(len(off) - 1):
        k = keys[off[t]:off[t + 1]]
        ty, me = types[t], inst[t]
        skip = mask_off[t] if ty == G else 0
        ext = inte = wr = 0
        alive = ty != W
        for i, key in enumerate(k):
            hit = stamp.get((me, key), 0) != 0
            if hit and alive:            # a leading cached block: counted and moved to the front
                if i < skip:
                    inte += 1
                else:
                    ext += 1
            elif hit:                    # cached, but behind the first miss: left alone
                continue
            else:
                alive = False
                if ty == G:
                    break                # a query stops at its first miss
                wr += 1
                usage[me] += 1
            counter += 1
            stamp[(me, key)] = counter
            queue[me].append((key, counter))
        if ty != G and sum(usage) > quota:
            excess = sum(usage) - quota
            take = [0] * n_inst
            if mode == 1:                # rounds over all instances, played on the counts only
                total = 0
                while total < excess:
                    any_taken = False
                    for j in range(n_inst):
                        got = min(batch, usage[j] - take[j])
                        if got > 0:
                            take[j] += got
                            total += got
                            any_taken = True
                    if not any_taken:
                        break
            else:
                need = excess if mode == 3 else -(-excess // batch) * batch
                take[me] = min(need, usage[me])
            for j in range(n_inst):      # pop that many live entries from the cold end
                while take[j] > 0:
                    key, s = queue[j][head[j]]
                    head[j] += 1
                    if stamp.get((j, key), 0) == s:
                        stamp[(j, key)] = 0
                        usage[j] -= 1
                        take[j] -= 1
        out.append((ext, inte, wr, usage[me]))
    return np.array(out, dtype=np.int64).reshape(-1, 4).T, usage


def _traces(rng, n_traces, n_inst):
    prompts = [rng.integers(1, 1 << 40, size=int(rng.integers(1, 30))).tolist() for _ in range(8)]
    for i in range(1, len(prompts)):
        if rng.random() < 0.6:
            j = int(rng.integers(0, i))
            prompts[i] = prompts[j][:int(rng.integers(0, len(prompts[j]) + 1))] + prompts[i]
    keys, off, types, mask, inst = [], [0], [], [], []
    for _ in range(n_traces):
        p = prompts[int(rng.integers(0, len(prompts)))]
        k = p[:int(rng.integers(0, len(p) + 1))] + rng.integers(1 << 41, 1 << 42, size=int(rng.integers(0, 4))).tolist()
        ty = int(rng.integers(0, 3))
        keys += k
        off.append(len(keys))
        types.append(ty)
        mask.append(int(rng.integers(0, len(k) + 1)) if ty == G else 0)
        inst.append(int(rng.integers(0, n_inst)))
    return keys, off, types, mask, inst


@pytest.mark.parametrize("mode", [1, 2, 3])
@pytest.mark.parametrize("n_inst", [1, 3])
def test_stamp_and_queue_model_equals_the_radix_trees(mode, n_inst):
    for seed in range(12):
        rng = np.random.default_rng(2000 + 100 * mode + 10 * n_inst + seed)
        keys, off, types, mask, inst = _traces(rng, int(rng.integers(30, 250)), n_inst)
        quota, batch = int(rng.integers(1, 70)), int(rng.integers(1, 9))
        want = oracle.LruGroupReplay(quota, n_inst, evict_batch=batch, mode=mode).run(keys, off, types, inst, mask)
        got, usage = queue_replay(keys, off, types, mask, inst, n_inst, quota, batch, mode)
        for name, w, g in zip(("external hits", "internal hits", "written", "cached"), want[:4], got):
            assert np.array_equal(np.asarray(w, dtype=np.int64), g), (name, seed)
        assert want[4].tolist() == usage, seed
