"""The state machine of the leaf_aware_lru replay kernel, written out sequentially, against the oracle's radix tree.

The CUDA kernel (tair-kvcache_b200/csrc/replay_leaf_lru.cu) does not keep the reference's pointer-based tree
(kv_cache_manager/optimizer/index/radix_tree_index.cc) but flat arrays: the node of every key, seven counters per
node, the queue as a linked list over key ids.  That this representation replays a trace exactly as the tree does
rests on a few claims - a key is in the tree exactly when its node still has blocks; a split can hand the new
node number to the upper part; removing an emptied leaf is zeroing its block count; accessed blocks may move to the
front in pieces; evictions may go in groups when nothing gets re-queued; a node's blocks are the ids in front of
one occurrence of its last key; blocks of one access time that are re-queued one after the other end up side by
side, so a run of them is one search and one splice.  This file restates those steps in plain
Python, one key at a time, and compares them with the oracle (which keeps real nodes and lists) on random traces
with shared prefixes and tied timestamps, so the claims are checked on a box without a GPU.  The GPU tests compare
the kernel itself with the same oracle.
"""
import numpy as np
import pytest

from oracle import kvcm_oracle as oracle

NONE = -1
GROUP = 4  # keys handled together (32 in the kernel); small, so that group edges fall everywhere


def flat_replay(keys, off, types, mask_off, stamps, quota, batch, precise):
    ids_of = {}
    ids = [ids_of.setdefault(k, len(ids_of)) for k in keys]
    nk = len(ids) + 1
    occ = [NONE] * nk  # a position of every key in ids (the last one, as it happens; any would do)
    for i, k in enumerate(ids):
        occ[k] = i
    node_of, flags, time = [NONE] * nk, [0] * nk, [0] * nk  # flags: 1 cached, 2 in the queue
    head, tail = nk, nk + 1
    before, after = [0] * (nk + 2), [0] * (nk + 2)  # towards the head / towards the tail
    after[head], before[tail] = tail, head
    parent, children, blocks, last, cached, child_cached, unlisted = [NONE], [0], [0], [NONE], [0], [0], [0]

    def new_node(above):
        for column, value in ((parent, above), (children, 0), (blocks, 0), (last, NONE), (cached, 0),
                              (child_cached, 0), (unlisted, 0)):
            column.append(value)
        return len(parent) - 1

    def push_front(i):
        f = after[head]
        after[i], before[i], before[f], after[head] = f, head, i, i

    def insertion_point(bt):  # leaf_aware_lru.cc:53-83 over common_structure.h:62-89: (goes in front of, from the head?)
        h = after[head]
        from_head = True
        if h == tail:
            spot = tail
        else:
            tl = before[tail]
            ht, tt = time[h], time[tl]
            from_head = True if bt >= ht else (False if bt <= tt else (ht - bt) < (bt - tt))
            if from_head:
                cur = h
                while cur != tail and bt < time[cur]:
                    cur = after[cur]
                spot = cur
            else:
                cur = tl
                while cur != head and time[cur] < bt:
                    cur = before[cur]
                spot = after[cur]
        return spot, from_head

    def splice_run(run):  # blocks of one access time, in key order
        spot, from_head = insertion_point(time[run[0]])
        # searched from the head each one lands in front of the one before it, from the tail behind it
        seq = list(reversed(run)) if from_head else list(run)
        a = before[spot]
        for x in seq:
            after[a], before[x] = x, a
            a = x
        after[a], before[spot] = spot, a

    resident, out = 0, []
    for t in range(len(off) - 1):
        beg, n, ty, now = off[t], off[t + 1] - off[t], types[t], stamps[t]
        skip = mask_off[t] if ty == 1 else 0
        ext = inte = wr = 0
        leaves, first_gone = n, -1  # where the trace leaves the tree; its first block that is not cached
        for i in range(n):
            k = ids[beg + i]
            if node_of[k] == NONE or blocks[node_of[k]] == 0:
                leaves = i
                break
            if not flags[k] & 1 and first_gone < 0:
                first_gone = i
                if ty == 1:
                    break
        hit = 0 if ty == 2 else (first_gone if first_gone >= 0 else leaves)
        if ty != 2:
            inte = min(hit, skip)
            ext = hit - inte
            for base in range(0, hit, GROUP):  # pieces that already sit in the queue in order move as one
                piece = [ids[beg + i] for i in range(base, min(hit, base + GROUP))]
                for k in piece:
                    time[k] = now
                listed = [bool(flags[k] & 2) for k in piece]
                joins = [listed[j] and j > 0 and listed[j - 1] and after[piece[j]] == piece[j - 1]
                         for j in range(len(piece))]
                j = 0
                while j < len(piece):
                    if not listed[j]:
                        j += 1
                        continue
                    e = j
                    while e + 1 < len(piece) and joins[e + 1]:
                        e += 1
                    deepest, front = piece[j], piece[e]
                    a = before[front]
                    if a != head:
                        b, f = after[deepest], after[head]
                        after[a], before[b], after[deepest], before[f] = b, a, f, deepest
                        after[head], before[front] = front, head
                    j = e + 1
        if ty != 1:
            for i in range(hit, leaves):  # evicted blocks on the walked path get their location back
                k = ids[beg + i]
                if flags[k] & 1:
                    continue
                nd = node_of[k]
                time[k] = now
                cached[nd] += 1
                child_cached[parent[nd]] += 1
                resident += 1
                wr += 1
                if children[nd] == 0:
                    flags[k] = 3
                    push_front(k)
                else:
                    flags[k] = 1
                    unlisted[nd] += 1
            if leaves < n:
                at_key = ids[beg + leaves - 1] if leaves > 0 else NONE
                at = node_of[at_key] if leaves > 0 else 0
                if leaves == 0 or last[at] == at_key:
                    if at != 0 and children[at] == 0:
                        target = at
                    else:
                        target = new_node(at)
                        children[at] += 1
                else:  # split: the new number goes to the upper part, whose keys were just walked
                    lower, upper = at, new_node(parent[at])
                    target = new_node(upper)
                    moved = out_of_queue = 0
                    j = leaves - 1
                    while j >= 0 and node_of[ids[beg + j]] == lower:
                        k = ids[beg + j]
                        node_of[k] = upper
                        out_of_queue += flags[k] & 3 == 1
                        moved += 1
                        j -= 1
                    above = parent[lower]
                    children[upper], blocks[upper], last[upper] = 2, moved, at_key
                    cached[upper], unlisted[upper] = moved, out_of_queue
                    blocks[lower] -= moved
                    cached[lower] -= moved
                    unlisted[lower] -= out_of_queue
                    parent[lower] = upper
                    child_cached[upper] = cached[lower]
                    child_cached[above] -= cached[lower]
                for i in range(leaves, n):
                    k = ids[beg + i]
                    node_of[k], flags[k], time[k] = target, 3, now
                    push_front(k)
                count = n - leaves
                blocks[target] += count
                cached[target] += count
                last[target] = ids[beg + n - 1]
                child_cached[parent[target]] += count
                resident += count
                wr += count
            if resident > quota:
                excess, total, gone = resident - quota, 0, []
                while total < excess:
                    want_round = min(batch, excess - total) if precise else batch
                    got = 0
                    while got < want_round:
                        want = min(GROUP, want_round - got)
                        group, b = [], before[tail]
                        while len(group) < want and b != head:
                            group.append(b)
                            b = before[b]
                        if not group:
                            break
                        nodes = [node_of[c] for c in group]
                        ups = [parent[x] for x in nodes]
                        if all(child_cached[x] == 0 and (u == 0 or unlisted[u] == 0 or child_cached[u] > ups.count(u))
                               for x, u in zip(nodes, ups)):  # nothing gets re-queued: the group goes at once
                            for c, x, u in zip(group, nodes, ups):
                                flags[c] = 0
                                gone.append(x)
                                cached[x] -= 1
                                child_cached[u] -= 1
                            after[b], before[tail] = tail, b
                            resident -= len(group)
                            got += len(group)
                            continue
                        g = 0
                        while g < want:  # one by one (leaf_aware_lru.cc:85-133)
                            b = before[tail]
                            if b == head:
                                break
                            a = before[b]
                            after[a], before[tail] = tail, a
                            x = node_of[b]
                            if child_cached[x] != 0:
                                flags[b] = 1
                                unlisted[x] += 1
                                continue
                            flags[b] = 0
                            cached[x] -= 1
                            u = parent[x]
                            child_cached[u] -= 1
                            resident -= 1
                            gone.append(x)
                            g += 1
                            if u != 0 and child_cached[u] == 0 and unlisted[u] != 0:
                                first = occ[last[u]] - blocks[u] + 1
                                chain = ids[first:first + blocks[u]]
                                assert first >= 0 and all(node_of[k] == u for k in chain)
                                for g0 in range(0, len(chain), GROUP):  # a run ends with the keys handled together
                                    run = []
                                    for k in chain[g0:g0 + GROUP]:
                                        if flags[k] & 3 != 1:
                                            continue
                                        if run and time[run[0]] != time[k]:
                                            splice_run(run)
                                            run = []
                                        run.append(k)
                                        flags[k] = 3
                                    if run:
                                        splice_run(run)
                                unlisted[u] = 0
                        got += g
                        if g < want:
                            break
                    if got == 0:
                        break
                    total += got
                again = bool(gone)
                while again:  # emptied leaves go; their keys leave the tree with the block count
                    again = False
                    for x in gone:
                        if x != 0 and cached[x] == 0 and children[x] == 0 and blocks[x] != 0:
                            children[parent[x]] -= 1
                            blocks[x] = 0
                            again = True
        out.append((ext, inte, wr, resident))
    return np.array(out, dtype=np.int64).reshape(-1, 4).T


def _traces(rng, n_traces, n_prompts, max_len, max_tail):
    prompts = [rng.integers(1, 1 << 40, size=int(rng.integers(1, max_len))).tolist() for _ in range(n_prompts)]
    for i in range(1, n_prompts):  # prompts that start with a piece of another prompt
        if rng.random() < 0.6:
            j = int(rng.integers(0, i))
            prompts[i] = prompts[j][:int(rng.integers(0, len(prompts[j]) + 1))] + prompts[i]
    keys, off, types, mask, stamps, now = [], [0], [], [], [], 0
    for _ in range(n_traces):
        p = prompts[int(rng.integers(0, len(prompts)))]
        k = p[:int(rng.integers(0, len(p) + 1))]
        if rng.random() < 0.5:
            k = k + rng.integers(1 << 41, 1 << 42, size=int(rng.integers(0, max_tail))).tolist()
        if rng.random() < 0.3 and k:
            prompts.append(k)  # later traces may extend this one
        ty = int(rng.integers(0, 3))
        keys += k
        off.append(len(keys))
        types.append(ty)
        mask.append(int(rng.integers(0, len(k) + 1)) if ty == 1 else 0)
        now += int(rng.integers(0, 3))  # equal timestamps on purpose
        stamps.append(now)
    return keys, off, types, mask, stamps


@pytest.mark.parametrize("seed", range(40))
def test_flat_state_machine_equals_the_radix_tree(seed):
    rng = np.random.default_rng(1000 + seed)
    keys, off, types, mask, stamps = _traces(rng, int(rng.integers(20, 300)), int(rng.integers(2, 12)),
                                             int(rng.integers(2, 40)), int(rng.integers(1, 8)))
    quota, batch, precise = int(rng.integers(1, 80)), int(rng.integers(1, 12)), bool(rng.integers(0, 2))
    want = oracle.LruReplay(quota, evict_batch=batch, precise=precise, policy="leaf_aware_lru").run(
        keys, off, types, mask, timestamps=stamps)
    got = flat_replay(keys, off, types, mask, stamps, quota, batch, precise)
    for name, w, g in zip(("external hits", "internal hits", "written", "cached"), want, got):
        assert np.array_equal(np.asarray(w, dtype=np.int64), g), name


def test_the_traces_above_do_evict_and_differ_from_plain_lru():
    differs = evicts = 0
    for seed in range(40):
        rng = np.random.default_rng(1000 + seed)
        keys, off, types, mask, stamps = _traces(rng, int(rng.integers(20, 300)), int(rng.integers(2, 12)),
                                                 int(rng.integers(2, 40)), int(rng.integers(1, 8)))
        quota, batch, precise = int(rng.integers(1, 80)), int(rng.integers(1, 12)), bool(rng.integers(0, 2))
        leaf = oracle.LruReplay(quota, evict_batch=batch, precise=precise, policy="leaf_aware_lru").run(
            keys, off, types, mask, timestamps=stamps)
        lru = oracle.LruReplay(quota, evict_batch=batch, precise=precise).run(keys, off, types, mask)
        free = oracle.Replay().run(keys, off, types, mask)
        differs += not np.array_equal(leaf[0], lru[0])
        evicts += not np.array_equal(leaf[0], free[0])
    assert evicts >= 30 and differs >= 20
