"""ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

The oracle restates the reference's hot-path algorithms on the CPU (see kvcm_oracle.cc for the
reference file:line of every function).  Only tests, the smoke check and the bench's CPU-baseline
leg import this module; the product package never does.

`ref_hash()` additionally loads oracle/_ref/libkvcm_ref_hash.so - the reference's own
kv_cache_manager/manager/hash_util.h compiled in place by oracle/Makefile - when it has been built.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkvcm_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libkvcm_ref_hash.so")

# kv_cache_manager/manager/select_location_policy.h:42-57: weights indexed by DataStorageType
# (UNKNOWN, HF3FS, MOONCAKE, TAIR_MEMPOOL, NFS).
DEFAULT_WEIGHTS = (1, 3, 3, 3, 5)

# kv_cache_manager/manager/cache_location.h:44-50
CLS_NOT_FOUND, CLS_NEW, CLS_WRITING, CLS_SERVING, CLS_DELETING = range(5)

_c_i64p = ctypes.POINTER(ctypes.c_int64)
_c_i32p = ctypes.POINTER(ctypes.c_int32)
_c_u32p = ctypes.POINTER(ctypes.c_uint32)
_c_u8p = ctypes.POINTER(ctypes.c_uint8)


def build(force=False):
    """Compile the oracle (and the reference header wrapper when the reference tree is present)."""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
            os.path.join(_HERE, "kvcm_oracle.cc")):
        subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.kvcm_oracle_hash_step.restype = ctypes.c_int64
        L.kvcm_oracle_hash_step.argtypes = [ctypes.c_int64, ctypes.c_int64]
        for name in ("kvcm_oracle_gen_key_vector_i64", "kvcm_oracle_gen_key_vector_u32"):
            getattr(L, name).restype = ctypes.c_int64
        L.kvcm_oracle_index_create.restype = ctypes.c_void_p
        L.kvcm_oracle_index_size.restype = ctypes.c_int64
        L.kvcm_oracle_index_get.restype = ctypes.c_int64
        L.kvcm_oracle_prefix_match.restype = ctypes.c_int64
        L.kvcm_oracle_sw_match.restype = ctypes.c_int32
        L.kvcm_oracle_filter_write.restype = ctypes.c_int32
        L.kvcm_oracle_move_rows.restype = ctypes.c_int64
        L.kvcm_oracle_copy_iovs.restype = ctypes.c_int64
        L.kvcm_oracle_iov_crc.restype = ctypes.c_uint32
        _lib = L
    return _lib


def ref_hash():
    """The reference's own hash header behind a C wrapper, or None when it was not built."""
    global _ref
    if _ref is None and os.path.exists(_REF_PATH):
        R = ctypes.CDLL(_REF_PATH)
        R.kvcm_ref_hash_step.restype = ctypes.c_int64
        R.kvcm_ref_hash_step.argtypes = [ctypes.c_int64, ctypes.c_int64]
        R.kvcm_ref_hash_array.restype = ctypes.c_int64
        R.kvcm_ref_gen_key_vector.restype = ctypes.c_int64
        _ref = R
    return _ref


def _ptr(a, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype))


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _weights(weights):
    w = np.ascontiguousarray(weights, dtype=np.uint32)
    return w, _ptr(w, ctypes.c_uint32), ctypes.c_int(len(w))


# ------------------------------------------------------------------------------------------
# hash
# ------------------------------------------------------------------------------------------

def hash_step(h, v):
    return int(lib().kvcm_oracle_hash_step(h, v))


def hash_step_py(h, v):
    """Pure-Python closed form of one step (kv_cache_manager/manager/hash_util.h:8-12), for tiny cases."""
    m = (1 << 64) - 1
    hu = h & m
    sra = (h >> 32) & m  # Python's >> on a negative int is arithmetic
    out = hu ^ (((v & m) + 0x9E3779B97F4A7C15 + ((hu << 12) & m) + sra) & m)
    return out - (1 << 64) if out >> 63 else out


def gen_key_vector(tokens, block_size):
    """GenKeyVector of one request (kv_cache_manager/manager/cache_manager.cc:76-87)."""
    tokens = np.asarray(tokens)
    n = len(tokens) // block_size if block_size > 0 else 0
    keys = np.empty(n, dtype=np.int64)
    if tokens.dtype == np.uint32:
        t = np.ascontiguousarray(tokens)
        lib().kvcm_oracle_gen_key_vector_u32(_ptr(t, ctypes.c_uint32), ctypes.c_int64(len(t)),
                                             ctypes.c_int64(block_size), _ptr(keys, ctypes.c_int64))
    else:
        t = _i64(tokens)
        lib().kvcm_oracle_gen_key_vector_i64(_ptr(t, ctypes.c_int64), ctypes.c_int64(len(t)),
                                             ctypes.c_int64(block_size), _ptr(keys, ctypes.c_int64))
    return keys


def apply_prefix_hash(ids):
    ids = _i64(ids)
    keys = np.empty(len(ids), dtype=np.int64)
    lib().kvcm_oracle_apply_prefix_hash(_ptr(ids, ctypes.c_int64), ctypes.c_int64(len(ids)),
                                        _ptr(keys, ctypes.c_int64))
    return keys


def key_offsets(tok_off, block_size):
    """Exclusive prefix sum of floor(len / block_size) per request."""
    tok_off = _i64(tok_off)
    counts = (tok_off[1:] - tok_off[:-1]) // block_size
    out = np.zeros(len(tok_off), dtype=np.int64)
    np.cumsum(counts, out=out[1:])
    return out


def hash_blocks(tokens, tok_off, block_size, threads=1):
    """Keys of a CSR batch of requests; returns (keys, key_off)."""
    tokens = np.ascontiguousarray(tokens)
    tok_off = _i64(tok_off)
    key_off = key_offsets(tok_off, block_size)
    keys = np.empty(int(key_off[-1]), dtype=np.int64)
    n_req = len(tok_off) - 1
    if tokens.dtype == np.uint32:
        fn, ct = lib().kvcm_oracle_hash_blocks_u32, ctypes.c_uint32
    else:
        tokens = _i64(tokens)
        fn, ct = lib().kvcm_oracle_hash_blocks_i64, ctypes.c_int64
    fn(_ptr(tokens, ct), _ptr(tok_off, ctypes.c_int64), ctypes.c_int64(n_req), ctypes.c_int64(block_size),
       _ptr(keys, ctypes.c_int64), _ptr(key_off, ctypes.c_int64), ctypes.c_int(threads))
    return keys, key_off


# ------------------------------------------------------------------------------------------
# index + matchers
# ------------------------------------------------------------------------------------------

class Index:
    """Block index as the matchers see it: int64 key -> list of (status, storage type)."""

    def __init__(self):
        self._h = ctypes.c_void_p(lib().kvcm_oracle_index_create())

    def __del__(self):
        if getattr(self, "_h", None):
            lib().kvcm_oracle_index_destroy(self._h)
            self._h = None

    def __len__(self):
        return int(lib().kvcm_oracle_index_size(self._h))

    def put(self, keys, locations):
        """locations[i] = list of (status, type) for keys[i]; an empty list is an empty location map."""
        keys = _i64(keys)
        loc_off = np.zeros(len(keys) + 1, dtype=np.int64)
        st, ty = [], []
        for i, locs in enumerate(locations):
            for s, t in locs:
                st.append(s)
                ty.append(t)
            loc_off[i + 1] = len(st)
        st = np.asarray(st, dtype=np.int32)
        ty = np.asarray(ty, dtype=np.int32)
        lib().kvcm_oracle_index_put(self._h, _ptr(keys, ctypes.c_int64), ctypes.c_int64(len(keys)),
                                    _ptr(loc_off, ctypes.c_int64), _ptr(st, ctypes.c_int32), _ptr(ty, ctypes.c_int32))

    def put_uniform(self, keys, status=CLS_SERVING, storage_type=4):
        keys = _i64(keys)
        lib().kvcm_oracle_index_reserve(self._h, ctypes.c_int64(len(self) + len(keys)))
        lib().kvcm_oracle_index_put_uniform(self._h, _ptr(keys, ctypes.c_int64), ctypes.c_int64(len(keys)),
                                            ctypes.c_int32(status), ctypes.c_int32(storage_type))

    def erase(self, keys):
        keys = _i64(keys)
        lib().kvcm_oracle_index_erase(self._h, _ptr(keys, ctypes.c_int64), ctypes.c_int64(len(keys)))

    def update_status(self, keys, types, expected, new_status):
        """One task per key on the location of storage type types[i]: expected[i] < 0 = no comparison;
        new_status[i] = -1 deletes the location as BatchCADLocationStatus does (an emptied key goes), -2 as
        BatchDeleteLocation does (an emptied key stays, a missing key is EC_OK).  Returns the reference's
        ErrorCode per key (0, 2 EC_NOENT, 16 EC_MISMATCH).  kv_cache_manager/manager/meta_searcher.cc:410-820."""
        keys = _i64(keys)
        n = len(keys)
        ty = np.ascontiguousarray(np.broadcast_to(np.asarray(types, dtype=np.int32), (n,)))
        ex = np.ascontiguousarray(np.broadcast_to(np.asarray(expected, dtype=np.int32), (n,)))
        nw = np.ascontiguousarray(np.broadcast_to(np.asarray(new_status, dtype=np.int32), (n,)))
        res = np.zeros(n, dtype=np.int32)
        lib().kvcm_oracle_index_update_status(self._h, _ptr(keys, ctypes.c_int64), ctypes.c_int64(n),
                                              _ptr(ty, ctypes.c_int32), _ptr(ex, ctypes.c_int32),
                                              _ptr(nw, ctypes.c_int32), _ptr(res, ctypes.c_int32))
        return res

    def add_location(self, keys, types, status=CLS_WRITING):
        """MetaSearcher::BatchAddLocation (kv_cache_manager/manager/meta_searcher.cc:312-408): key i gets one more
        location of storage type types[i] (the reference adds it in CLS_WRITING); an absent key is created, a present
        one keeps its other locations.  A plain loop over get / put: small cases only."""
        keys = _i64(keys)
        types = np.broadcast_to(np.asarray(types, dtype=np.int32), (len(keys),))
        for k, t in zip(keys.tolist(), types.tolist()):
            self.put([k], [(self.get(k) or []) + [(int(status), int(t))]])

    def get(self, key):
        """The (status, storage type) list of one key, or None when the key is absent."""
        st = np.zeros(64, dtype=np.int32)
        ty = np.zeros(64, dtype=np.int32)
        n = int(lib().kvcm_oracle_index_get(self._h, ctypes.c_int64(int(key)), _ptr(st, ctypes.c_int32),
                                            _ptr(ty, ctypes.c_int32), ctypes.c_int64(64)))
        return None if n < 0 else [(int(st[j]), int(ty[j])) for j in range(min(n, 64))]

    def prefix_match(self, keys, mask=None, weights=DEFAULT_WEIGHTS):
        """mask: None, an int offset, or a sequence of bools (kv_cache_manager/manager/cache_location.h:52-57)."""
        keys = _i64(keys)
        w, wp, nw = _weights(weights)
        kind, vec, vec_len, off = 1, None, 0, 0
        if mask is None:
            kind = 0
            vec = np.zeros(0, dtype=np.uint8)
        elif isinstance(mask, (int, np.integer)):
            off = int(mask)
        else:
            kind = 0
            vec = np.ascontiguousarray(np.asarray(mask, dtype=bool).astype(np.uint8))
            vec_len = len(vec)
        vp = _ptr(vec, ctypes.c_uint8) if vec is not None else None
        return int(lib().kvcm_oracle_prefix_match(self._h, _ptr(keys, ctypes.c_int64), ctypes.c_int64(len(keys)),
                                                  ctypes.c_int(kind), vp, ctypes.c_int64(vec_len), ctypes.c_int64(off),
                                                  wp, nw))

    def sw_match(self, keys, sw, weights=DEFAULT_WEIGHTS):
        """Returns (error_code, base): base = start of the matched window or -1."""
        keys = _i64(keys)
        w, wp, nw = _weights(weights)
        base = ctypes.c_int64(-1)
        ec = lib().kvcm_oracle_sw_match(self._h, _ptr(keys, ctypes.c_int64), ctypes.c_int64(len(keys)),
                                        ctypes.c_int64(sw), wp, nw, ctypes.byref(base))
        return int(ec), int(base.value)

    def batch_get(self, keys, weights=DEFAULT_WEIGHTS):
        """flags per key: bit0 servable, bit1 exists, bit2 location map non-empty, bit3 exists-for-write."""
        keys = _i64(keys)
        w, wp, nw = _weights(weights)
        flags = np.zeros(len(keys), dtype=np.uint8)
        lib().kvcm_oracle_batch_get(self._h, _ptr(keys, ctypes.c_int64), ctypes.c_int64(len(keys)), wp, nw,
                                    _ptr(flags, ctypes.c_uint8))
        return flags

    def filter_write(self, keys, weights=DEFAULT_WEIGHTS):
        """Returns ("offset", first_missing, n_new) or ("vector", bool mask, n_new)."""
        keys = _i64(keys)
        w, wp, nw = _weights(weights)
        off = ctypes.c_int64(0)
        n_new = ctypes.c_int64(0)
        mask = np.zeros(max(len(keys), 1), dtype=np.uint8)
        is_off = lib().kvcm_oracle_filter_write(self._h, _ptr(keys, ctypes.c_int64), ctypes.c_int64(len(keys)), wp, nw,
                                                ctypes.byref(off), _ptr(mask, ctypes.c_uint8), ctypes.byref(n_new))
        if is_off:
            return "offset", int(off.value), int(n_new.value)
        return "vector", mask[:len(keys)].astype(bool), int(n_new.value)

    def prefix_match_batch(self, keys, key_off, mask_off=None, weights=DEFAULT_WEIGHTS, threads=1):
        keys = _i64(keys)
        key_off = _i64(key_off)
        w, wp, nw = _weights(weights)
        n_req = len(key_off) - 1
        out = np.zeros(n_req, dtype=np.int32)
        mp = None
        if mask_off is not None:
            mask_off = _i64(mask_off)
            mp = _ptr(mask_off, ctypes.c_int64)
        lib().kvcm_oracle_prefix_match_batch(self._h, _ptr(keys, ctypes.c_int64), _ptr(key_off, ctypes.c_int64),
                                             ctypes.c_int64(n_req), mp, wp, nw, _ptr(out, ctypes.c_int32),
                                             ctypes.c_int(threads))
        return out

    def sw_match_batch(self, keys, key_off, sw, weights=DEFAULT_WEIGHTS, threads=1):
        keys = _i64(keys)
        key_off = _i64(key_off)
        w, wp, nw = _weights(weights)
        n_req = len(key_off) - 1
        out = np.zeros(n_req, dtype=np.int32)
        lib().kvcm_oracle_sw_match_batch(self._h, _ptr(keys, ctypes.c_int64), _ptr(key_off, ctypes.c_int64),
                                         ctypes.c_int64(n_req), ctypes.c_int64(sw), wp, nw,
                                         _ptr(out, ctypes.c_int32), ctypes.c_int(threads))
        return out


# ------------------------------------------------------------------------------------------
# gather / scatter
# ------------------------------------------------------------------------------------------

def _ptr_table(arrays):
    tab = (ctypes.c_void_p * len(arrays))()
    for i, a in enumerate(arrays):
        tab[i] = a.ctypes.data if a is not None else None
    return tab


def move_rows(pools, staging, row_idx, slot_idx, rows_per_block, row_bytes, direction, threads=1):
    """Gather (direction 0) or scatter (1) between numpy uint8 pools [pool_rows*row_bytes] and staging.

    Layout rule: kv_cache_manager/py_connector/kernel/batch_gather_scatter_helper.py:46-98,152-205.
    Returns the number of rows skipped for being out of range.
    """
    row_idx = np.ascontiguousarray(row_idx, dtype=np.int32)
    n_blocks = len(row_idx) // rows_per_block
    sp = None
    if slot_idx is not None:
        slot_idx = np.ascontiguousarray(slot_idx, dtype=np.int32)
        sp = _ptr(slot_idx, ctypes.c_int32)
    n_pools = len(pools)
    slot_bytes = n_pools * rows_per_block * row_bytes
    n_slots = staging.nbytes // slot_bytes if slot_bytes else 0
    pool_rows = pools[0].nbytes // row_bytes
    tab = _ptr_table(pools)
    return int(lib().kvcm_oracle_move_rows(tab, ctypes.c_int32(n_pools), ctypes.c_void_p(staging.ctypes.data),
                                           ctypes.c_int64(n_slots), _ptr(row_idx, ctypes.c_int32), sp,
                                           ctypes.c_int64(n_blocks), ctypes.c_int64(rows_per_block),
                                           ctypes.c_int64(row_bytes), ctypes.c_int64(pool_rows),
                                           ctypes.c_int(direction), ctypes.c_int(threads)))


def move_rows_py(pools, staging, row_idx, slot_idx, rows_per_block, row_bytes, direction):
    """The same rule as plain Python loops over numpy views (small cases only)."""
    n_pools = len(pools)
    n_blocks = len(row_idx) // rows_per_block
    st = staging.reshape(-1, n_pools, rows_per_block, row_bytes)
    for b in range(n_blocks):
        slot = slot_idx[b] if slot_idx is not None else b
        for p in range(n_pools):
            pool = pools[p].reshape(-1, row_bytes)
            for t in range(rows_per_block):
                row = row_idx[b * rows_per_block + t]
                if row < 0 or row >= pool.shape[0]:
                    continue
                if direction == 0:
                    st[slot, p, t] = pool[row]
                else:
                    pool[row] = st[slot, p, t]


def move_legacy(layers, total_tokens, staging, token_idx, hidden_bytes, direction):
    """Legacy single-block form (kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:10-107)."""
    token_idx = np.ascontiguousarray(token_idx, dtype=np.int32)
    tab = _ptr_table(layers)
    lib().kvcm_oracle_move_legacy(tab, ctypes.c_int32(len(layers)), ctypes.c_int64(total_tokens),
                                  ctypes.c_void_p(staging.ctypes.data), _ptr(token_idx, ctypes.c_int32),
                                  ctypes.c_int64(len(token_idx)), ctypes.c_int64(hidden_bytes),
                                  ctypes.c_int(direction))


def copy_iovs(iovs, block_string, direction):
    """iovs: list of (numpy uint8 array or None, size, ignore).  direction 0: iovs -> string, 1: string -> iovs."""
    n = len(iovs)
    tab = (ctypes.c_void_p * n)()
    sizes = np.zeros(n, dtype=np.int64)
    ign = np.zeros(n, dtype=np.uint8)
    for i, (arr, size, ignore) in enumerate(iovs):
        tab[i] = arr.ctypes.data if arr is not None else None
        sizes[i] = size
        ign[i] = 1 if ignore else 0
    return int(lib().kvcm_oracle_copy_iovs(tab, _ptr(sizes, ctypes.c_int64), _ptr(ign, ctypes.c_uint8),
                                           ctypes.c_int64(n), ctypes.c_void_p(block_string.ctypes.data),
                                           ctypes.c_int(direction)))


def iov_crc(buf, cal_bytes):
    buf = np.ascontiguousarray(np.frombuffer(buf, dtype=np.uint8) if isinstance(buf, (bytes, bytearray)) else buf)
    return int(lib().kvcm_oracle_iov_crc(ctypes.c_void_p(buf.ctypes.data), ctypes.c_int64(buf.nbytes),
                                         ctypes.c_int64(cal_bytes)))


# ------------------------------------------------------------------------------------------
# optimizer trace replay
# ------------------------------------------------------------------------------------------

TRACE_DIALOG_TURN, TRACE_GET_LOCATION, TRACE_WRITE_CACHE = 0, 1, 2


def partial_sort_by_time(indices, k, times):
    """std::partial_sort(indices, indices + k, end) with the comparator times[a] < times[b], as the reference's
    random_lru policy calls it (eviction_policy/random_lru.cc:72-74).  Returns the reordered index array."""
    idx = np.ascontiguousarray(indices, dtype=np.uint64).copy()
    times = _i64(times)
    lib().kvcm_oracle_partial_sort_by_time(_ptr(idx, ctypes.c_uint64), ctypes.c_int64(len(idx)), ctypes.c_int64(int(k)),
                                           _ptr(times, ctypes.c_int64))
    return idx


class Replay:
    """Sequential replay over the prefix tree, no eviction
    (kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215)."""

    def __init__(self):
        lib().kvcm_oracle_replay_create.restype = ctypes.c_void_p
        self._h = ctypes.c_void_p(lib().kvcm_oracle_replay_create())

    def __del__(self):
        if getattr(self, "_h", None):
            lib().kvcm_oracle_replay_destroy(self._h)
            self._h = None

    def run(self, keys, key_off, trace_type, mask_off=None, mask_bits=None):
        """Returns (external hits, internal hits, written blocks, cached blocks after) per trace.  mask_off: leading
        masked keys per GetLocation trace; mask_bits: optional uint8 per key (a BlockMaskVector, holes allowed)."""
        keys, key_off = _i64(keys), _i64(key_off)
        n = len(key_off) - 1
        trace_type = np.ascontiguousarray(trace_type, dtype=np.uint8)
        mp = None
        if mask_off is not None:
            mask_off = _i64(mask_off)
            mp = _ptr(mask_off, ctypes.c_int64)
        ext = np.zeros(n, dtype=np.int32)
        inte = np.zeros(n, dtype=np.int32)
        wr = np.zeros(n, dtype=np.int32)
        cached = np.zeros(n, dtype=np.int64)
        bp = None
        if mask_bits is not None:
            mask_bits = np.ascontiguousarray(mask_bits, dtype=np.uint8)
            bp = _ptr(mask_bits, ctypes.c_uint8)
        lib().kvcm_oracle_replay_run(self._h, _ptr(keys, ctypes.c_int64), _ptr(key_off, ctypes.c_int64),
                                     _ptr(trace_type, ctypes.c_uint8), mp, bp, ctypes.c_int64(n),
                                     _ptr(ext, ctypes.c_int32), _ptr(inte, ctypes.c_int32), _ptr(wr, ctypes.c_int32),
                                     _ptr(cached, ctypes.c_int64))
        return ext, inte, wr, cached


class LruReplay(Replay):
    """Sequential replay over the compressed prefix tree with the "lru" or "leaf_aware_lru" eviction policy and a
    block quota (kv_cache_manager/optimizer/index/radix_tree_index.cc, eviction_policy/lru.cc, leaf_aware_lru.cc,
    manager/eviction_manager.cc:148-266).  precise=False evicts whole batches of evict_batch blocks until the
    excess is covered (EVICTION_MODE_GROUP_ROUGH / INSTANCE_ROUGH with one instance per group), precise=True
    evicts exactly the excess (INSTANCE_PRECISE)."""

    POLICIES = {"lru": 0, "leaf_aware_lru": 1}

    def __init__(self, quota_blocks, evict_batch=100, precise=False, policy="lru", sample_rate=0.0):
        """policy "random_lru" (eviction_policy/random_lru.cc) takes `sample_rate` (RandomLruParams; <= 0 means 0.1)."""
        if policy == "random_lru":
            lib().kvcm_oracle_random_lru_replay_create.restype = ctypes.c_void_p
            self._h = ctypes.c_void_p(lib().kvcm_oracle_random_lru_replay_create(
                ctypes.c_int64(int(quota_blocks)), ctypes.c_int32(int(evict_batch)),
                ctypes.c_int32(1 if precise else 0), ctypes.c_double(float(sample_rate))))
            return
        lib().kvcm_oracle_lru_replay_create_policy.restype = ctypes.c_void_p
        self._h = ctypes.c_void_p(lib().kvcm_oracle_lru_replay_create_policy(
            ctypes.c_int64(int(quota_blocks)), ctypes.c_int32(int(evict_batch)), ctypes.c_int32(1 if precise else 0),
            ctypes.c_int32(self.POLICIES[policy])))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().kvcm_oracle_lru_replay_destroy(self._h)
            self._h = None

    def run(self, keys, key_off, trace_type, mask_off=None, mask_bits=None, timestamps=None):
        """timestamps: the traces' timestamp_us (int64 per trace; the trace number when None).  Only the
        "leaf_aware_lru" policy reads them."""
        keys, key_off = _i64(keys), _i64(key_off)
        n = len(key_off) - 1
        trace_type = np.ascontiguousarray(trace_type, dtype=np.uint8)
        mp = None
        if mask_off is not None:
            mask_off = _i64(mask_off)
            mp = _ptr(mask_off, ctypes.c_int64)
        ext = np.zeros(n, dtype=np.int32)
        inte = np.zeros(n, dtype=np.int32)
        wr = np.zeros(n, dtype=np.int32)
        cached = np.zeros(n, dtype=np.int64)
        bp = None
        if mask_bits is not None:
            mask_bits = np.ascontiguousarray(mask_bits, dtype=np.uint8)
            bp = _ptr(mask_bits, ctypes.c_uint8)
        tp = None
        if timestamps is not None:
            timestamps = _i64(timestamps)
            tp = _ptr(timestamps, ctypes.c_int64)
        lib().kvcm_oracle_lru_replay_run_ts(self._h, _ptr(keys, ctypes.c_int64), _ptr(key_off, ctypes.c_int64),
                                            _ptr(trace_type, ctypes.c_uint8), mp, bp, tp, ctypes.c_int64(n),
                                            _ptr(ext, ctypes.c_int32), _ptr(inte, ctypes.c_int32),
                                            _ptr(wr, ctypes.c_int32), _ptr(cached, ctypes.c_int64))
        return ext, inte, wr, cached


class LruGroupReplay:
    """Several instances that share one group quota (kv_cache_manager/optimizer/manager/eviction_manager.cc:86-266):
    every instance has its own radix tree and eviction policy, the quota is checked against the sum of their usage
    after every write.  mode: 1 = EVICTION_MODE_GROUP_ROUGH (rounds of evict_batch blocks from every instance),
    2 = INSTANCE_ROUGH and 3 = INSTANCE_PRECISE (from the writing instance only)."""

    def __init__(self, quota_blocks, n_instances, evict_batch=100, mode=1, policy="lru", sample_rate=0.0):
        """policy: one name for every instance, or a sequence with one name per instance ("lru", "leaf_aware_lru",
        "random_lru"); sample_rate: that of the "random_lru" instances, one number or one per instance."""
        lib().kvcm_oracle_lru_group_create.restype = ctypes.c_void_p
        self.n_instances = int(n_instances)
        each = [policy] * self.n_instances if isinstance(policy, str) else list(policy)
        rates = [sample_rate] * self.n_instances if np.isscalar(sample_rate) else list(sample_rate)
        assert len(each) == self.n_instances == len(rates)
        assert all(e in ("lru", "leaf_aware_lru", "random_lru") for e in each)
        self._h = ctypes.c_void_p(lib().kvcm_oracle_lru_group_create(
            ctypes.c_int64(int(quota_blocks)), ctypes.c_int32(int(evict_batch)), ctypes.c_int32(int(mode)),
            ctypes.c_int32(self.n_instances), ctypes.c_int32(0)))
        for j, e in enumerate(each):
            if e == "random_lru":
                lib().kvcm_oracle_lru_group_set_random(self._h, ctypes.c_int32(j), ctypes.c_double(float(rates[j])))
            else:
                lib().kvcm_oracle_lru_group_set_policy(self._h, ctypes.c_int32(j),
                                                       ctypes.c_int32(LruReplay.POLICIES[e]))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().kvcm_oracle_lru_group_destroy(self._h)
            self._h = None

    def run(self, keys, key_off, trace_type, trace_instance, mask_off=None, mask_bits=None, timestamps=None,
            instance_records=False):
        """Returns (external hits, internal hits, written, usage of the trace's instance) per trace and the usage
        of every instance at the end; with instance_records=True also the usage of every instance after each trace
        ([n_traces, n_instances]; ReadRecord::blocks_per_instance, optimizer_runner.cc:116-124)."""
        keys, key_off = _i64(keys), _i64(key_off)
        n = len(key_off) - 1
        trace_type = np.ascontiguousarray(trace_type, dtype=np.uint8)
        trace_instance = np.ascontiguousarray(trace_instance, dtype=np.int32)
        assert len(trace_instance) == n and (n == 0 or 0 <= trace_instance.min() <= trace_instance.max() < self.n_instances)
        mp = bp = tp = None
        if mask_off is not None:
            mask_off = _i64(mask_off)
            mp = _ptr(mask_off, ctypes.c_int64)
        if mask_bits is not None:
            mask_bits = np.ascontiguousarray(mask_bits, dtype=np.uint8)
            bp = _ptr(mask_bits, ctypes.c_uint8)
        if timestamps is not None:
            timestamps = _i64(timestamps)
            tp = _ptr(timestamps, ctypes.c_int64)
        ext, inte, wr = (np.zeros(n, dtype=np.int32) for _ in range(3))
        cached = np.zeros(n, dtype=np.int64)
        final = np.zeros(self.n_instances, dtype=np.int64)
        every = np.zeros((max(n, 1), self.n_instances), dtype=np.int64)[:n]
        lib().kvcm_oracle_lru_group_run(self._h, _ptr(keys, ctypes.c_int64), _ptr(key_off, ctypes.c_int64),
                                        _ptr(trace_type, ctypes.c_uint8), mp, bp, tp,
                                        _ptr(trace_instance, ctypes.c_int32), ctypes.c_int64(n),
                                        _ptr(ext, ctypes.c_int32), _ptr(inte, ctypes.c_int32),
                                        _ptr(wr, ctypes.c_int32), _ptr(cached, ctypes.c_int64),
                                        _ptr(final, ctypes.c_int64),
                                        _ptr(every, ctypes.c_int64) if instance_records else None)
        return (ext, inte, wr, cached, final, every) if instance_records else (ext, inte, wr, cached, final)
