"""Hypothesis strategies shared by the property tests: small trace replays of the Optimizer, shaped so that a failing
example shrinks to a handful of short traces over a two- or three-letter alphabet.

Keys are prefix-unique as the chained block hash makes them: the key of a block is a function of the whole path of
symbols up to and including that block, so two traces share keys exactly on their common prefix."""
import numpy as np
from hypothesis import strategies as st

POLICIES = ("lru", "leaf_aware_lru", "random_lru")
W, G, D = 2, 1, 0  # WriteCache, GetLocation, DialogTurn


def path_key(path):
    """A 63-bit key for a path of symbols (FNV-1a over the symbols; the sign bit stays clear)."""
    h = 0xcbf29ce484222325
    for s in path:
        h = ((h ^ (s + 1)) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return h >> 1


@st.composite
def replay_cases(draw, max_traces=22, max_blocks=7, max_instances=3, policies=POLICIES):
    """(dict) keys / key_off / types / instance / mask_off / mask_bits / timestamps as numpy arrays, policies and
    sample rates per instance, quota, evict_batch, mode."""
    k = draw(st.integers(1, max_instances))
    each = [draw(st.sampled_from(policies)) for _ in range(k)]
    rates = [draw(st.sampled_from([0.1, 0.25, 0.5, 1.0])) for _ in range(k)]
    rw = draw(st.booleans())
    alphabet = draw(st.integers(1, 3))
    n = draw(st.integers(0, max_traces))
    use_bits = rw and draw(st.booleans())
    keys, off, types, inst, mask, bits, ts = [], [0], [], [], [], [], []
    now = 1000
    for _ in range(n):
        path = draw(st.lists(st.integers(0, alphabet - 1), min_size=0, max_size=max_blocks))
        keys += [path_key(path[:i + 1]) for i in range(len(path))]
        off.append(len(keys))
        ty = draw(st.sampled_from([W, G])) if rw else D
        types.append(ty)
        inst.append(draw(st.integers(0, k - 1)))
        if use_bits:
            bits += [draw(st.integers(0, 1)) if ty == G else 0 for _ in path]
            mask.append(0)
        else:
            mask.append(draw(st.integers(0, len(path) + 1)) if ty == G else 0)
        now += draw(st.integers(0, 2))
        ts.append(now)
    return dict(keys=np.array(keys, dtype=np.int64), key_off=np.array(off, dtype=np.int64),
                types=np.array(types, dtype=np.uint8), instance=np.array(inst, dtype=np.int32),
                mask_off=None if use_bits else np.array(mask, dtype=np.int64),
                mask_bits=np.array(bits, dtype=np.uint8) if use_bits else None,
                timestamps=np.array(ts, dtype=np.int64), policies=each, sample_rates=rates,
                quota=draw(st.integers(1, 30)), evict_batch=draw(st.integers(1, 5)), mode=draw(st.integers(1, 3)))
