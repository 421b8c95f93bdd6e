"""Generates tests/golden/hash_kat.json from the reference's OWN hash header.

Run in a container that holds the reference tree: `make -C oracle` compiles
kv_cache_manager/manager/hash_util.h in place into oracle/_ref/libkvcm_ref_hash.so, and this
script calls that library on seeded inputs.  The committed JSON is what travels; the tests
replay it against the oracle restatement and against the CUDA kernels.

    python tests/golden/make_hash_golden.py
"""
import ctypes
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import kvcm_oracle  # noqa: E402


def main():
    kvcm_oracle.build(force=True)
    ref = kvcm_oracle.ref_hash()
    if ref is None:
        raise SystemExit("oracle/_ref/libkvcm_ref_hash.so not built: the reference tree is needed")
    p64 = ctypes.POINTER(ctypes.c_int64)

    def gen(tokens, bs):
        t = np.ascontiguousarray(tokens, dtype=np.int64)
        keys = np.empty(len(t) // bs, dtype=np.int64)
        ref.kvcm_ref_gen_key_vector(t.ctypes.data_as(p64), ctypes.c_int64(len(t)), ctypes.c_int64(bs),
                                    keys.ctypes.data_as(p64))
        return keys

    steps = []
    rng = np.random.default_rng(0xB2000001)
    step_inputs = [(0, 0), (-1, 7), (1, 1), (-(1 << 63), 0), ((1 << 63) - 1, (1 << 31) - 1), (0, 151935),
                   (-7046029254386353131, 42), (0x123456789ABCDEF, 0xFFFFFFFF)]
    for _ in range(24):
        step_inputs.append((int(rng.integers(-(1 << 63), (1 << 63) - 1)), int(rng.integers(0, 1 << 32))))
    for h, v in step_inputs:
        steps.append({"h": str(h), "v": str(v), "out": str(int(ref.kvcm_ref_hash_step(h, v)))})

    chains = []
    named = [
        ("tokens_1_2_3_4_bs2", [1, 2, 3, 4], 2),
        ("tokens_0_to_129_bs64", list(range(130)), 64),
        ("tokens_desc_from_151935_bs16", [151935 - i for i in range(48)], 16),
        ("empty_bs16", [], 16),
        ("shorter_than_block_bs64", list(range(63)), 64),
        ("exact_one_block_bs1", [7], 1),
    ]
    for name, toks, bs in named:
        chains.append({"name": name, "tokens": toks, "block_size": bs, "keys": [str(int(k)) for k in gen(toks, bs)]})
    # seeded uint32-range token streams with the vocabulary of the prefix-match config
    for i, (n, bs) in enumerate([(512, 64), (1000, 16), (8192, 64), (257, 1), (4096, 128)]):
        toks = rng.integers(0, 151936, size=n).astype(np.int64)
        keys = gen(toks, bs)
        chains.append({"name": "seeded_%d" % i, "seed_stream": "default_rng(0xB2000001) after step draws",
                       "tokens": toks.tolist(), "block_size": bs, "keys": [str(int(k)) for k in keys]})

    ids = [100, 200, 300]
    out = np.empty(3, dtype=np.int64)
    a = np.asarray(ids, dtype=np.int64)
    ref.kvcm_ref_apply_prefix_hash(a.ctypes.data_as(p64), ctypes.c_int64(3), out.ctypes.data_as(p64))
    prefix = {"ids": ids, "keys": [str(int(k)) for k in out]}

    doc = {
        "source": "kv_cache_manager/manager/hash_util.h:8-24 compiled in place (g++ -O2, libstdc++); "
                  "GenKeyVector loop kv_cache_manager/manager/cache_manager.cc:76-87; "
                  "ApplyPrefixHash loop kv_cache_manager/optimizer/trace_converter/trace_util.cc:47-56",
        "steps": steps, "chains": chains, "apply_prefix_hash": prefix,
    }
    path = os.path.join(ROOT, "tests", "golden", "hash_kat.json")
    with open(path, "w") as f:
        json.dump(doc, f, indent=0, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
