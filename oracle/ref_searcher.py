"""TEST INFRASTRUCTURE ONLY.  ctypes access to the REFERENCE's own MetaSearcher (over its MetaIndexer and local meta
backend), compiled from the reference's source files into oracle/_ref/libkvcm_ref_searcher.so (oracle/Makefile,
target ref_searcher; oracle/ref_searcher_driver.cc is the C-callable wrapper).  Used by tests/ to compare
oracle/kvcm_oracle's index, matchers and status transitions with the reference itself on random inputs.  Nothing in
the product path imports this.
"""
import ctypes
import os
import shutil
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_ref", "libkvcm_ref_searcher.so")
_lib = None

OP_UPDATE, OP_CAS, OP_CAD, OP_DELETE = 0, 1, 2, 3


def available():
    return os.path.exists(_LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(_LIB_PATH)
        L.kvcm_ref_searcher_create.restype = ctypes.c_void_p
        L.kvcm_ref_searcher_create.argtypes = [ctypes.c_char_p, ctypes.c_int64]
        L.kvcm_ref_searcher_destroy.argtypes = [ctypes.c_void_p]
        L.kvcm_ref_searcher_prefix.restype = ctypes.c_int64
        L.kvcm_ref_searcher_sw.restype = ctypes.c_int64
        _lib = L
    return _lib


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t)) if a is not None else None


# kv_cache_manager/manager/select_location_policy.h:42-57, indexed by DataStorageType.  Always passed explicitly: the
# reference's DynamicWeightSLPoliy assigns its weights THROUGH the reference member that aliases the static default
# table (select_location_policy.h:59-69), so after the first policy with other weights the "default" policy of the
# process no longer has the default weights.
DEFAULT_WEIGHTS = (1, 3, 3, 3, 5)


def _w(weights):
    return np.ascontiguousarray(DEFAULT_WEIGHTS if weights is None else weights, dtype=np.uint32)


class RefSearcher:
    def __init__(self, max_keys=100000, in_memory=False):
        """in_memory: the local backend without a storage URI - the reference's own switch
        (meta/meta_local_backend.cc:27-34) - so that it keeps no file; with one it rewrites the file on every
        mutation and a large index takes time quadratic in its keys to build."""
        self._dir = tempfile.mkdtemp(prefix="kvcm_ref_searcher_")
        path = "" if in_memory else os.path.join(self._dir, "meta_local_backend_file")
        self._h = ctypes.c_void_p(lib().kvcm_ref_searcher_create(path.encode(), ctypes.c_int64(max_keys)))
        if not self._h:
            raise RuntimeError("the reference's MetaIndexer did not initialise")

    def __del__(self):
        if getattr(self, "_h", None):
            lib().kvcm_ref_searcher_destroy(self._h)
            self._h = None
            shutil.rmtree(self._dir, ignore_errors=True)

    def add(self, keys, storage_type, status):
        """One more location of `storage_type` (DataStorageType's number) in `status` for every key."""
        k = np.ascontiguousarray(keys, dtype=np.int64)
        rc = lib().kvcm_ref_searcher_add(self._h, _p(k, ctypes.c_int64), ctypes.c_int64(len(k)),
                                         ctypes.c_int32(storage_type), ctypes.c_int32(status))
        if rc != 0:
            raise RuntimeError("BatchAddLocation / BatchUpdateLocationStatus returned %d" % rc)

    def prefix_match(self, keys, mask=None, weights=None):
        k = np.ascontiguousarray(keys, dtype=np.int64)
        kind, off, vec = 0, 0, None
        if isinstance(mask, (int, np.integer)):
            kind, off = 1, int(mask)
        elif mask is not None:
            kind, vec = 2, np.ascontiguousarray(mask, dtype=np.uint8)
        w = _w(weights)
        return int(lib().kvcm_ref_searcher_prefix(self._h, _p(k, ctypes.c_int64), ctypes.c_int64(len(k)),
                                                  ctypes.c_int32(kind), ctypes.c_int64(off), _p(vec, ctypes.c_uint8),
                                                  _p(w, ctypes.c_uint32)))

    def prefix_match_batch(self, tokens, tok_off, block_size, threads=1, weights=None):
        """GenKeyVector + PrefixMatch per request on `threads` host threads: matched blocks per request."""
        t = np.ascontiguousarray(tokens, dtype=np.int64)
        off = np.ascontiguousarray(tok_off, dtype=np.int64)
        out = np.zeros(len(off) - 1, dtype=np.int32)
        w = _w(weights)
        rc = lib().kvcm_ref_searcher_prefix_batch(self._h, _p(t, ctypes.c_int64), _p(off, ctypes.c_int64),
                                                  ctypes.c_int64(len(off) - 1), ctypes.c_int32(block_size),
                                                  _p(w, ctypes.c_uint32), ctypes.c_int32(threads),
                                                  _p(out, ctypes.c_int32))
        if rc != 0:
            raise RuntimeError("kvcm_ref_searcher_prefix_batch returned %d" % rc)
        return out

    def window_match_batch(self, tokens, tok_off, block_size, sw, threads=1, weights=None):
        """GenKeyVector + PrefixMatch + ReverseRollSlideWindowMatch per request on `threads` host threads:
        (matched blocks, start of the window or -1 / -2) per request."""
        t = np.ascontiguousarray(tokens, dtype=np.int64)
        off = np.ascontiguousarray(tok_off, dtype=np.int64)
        matched = np.zeros(len(off) - 1, dtype=np.int32)
        base = np.zeros(len(off) - 1, dtype=np.int32)
        w = _w(weights)
        rc = lib().kvcm_ref_searcher_window_batch(self._h, _p(t, ctypes.c_int64), _p(off, ctypes.c_int64),
                                                  ctypes.c_int64(len(off) - 1), ctypes.c_int32(block_size),
                                                  ctypes.c_int32(sw), _p(w, ctypes.c_uint32), ctypes.c_int32(threads),
                                                  _p(matched, ctypes.c_int32), _p(base, ctypes.c_int32))
        if rc != 0:
            raise RuntimeError("kvcm_ref_searcher_window_batch failed with %d" % rc)
        return matched, base

    def sw_match(self, keys, sw, weights=None):
        """(start of the matched window or -1, number of locations returned); needs len(keys) >= sw > 0, which the
        reference asserts."""
        k = np.ascontiguousarray(keys, dtype=np.int64)
        if sw <= 0 or len(k) < sw:
            raise ValueError("the reference asserts len(keys) >= sw_size > 0")
        count = ctypes.c_int64(0)
        w = _w(weights)
        base = int(lib().kvcm_ref_searcher_sw(self._h, _p(k, ctypes.c_int64), ctypes.c_int64(len(k)),
                                              ctypes.c_int32(sw), _p(w, ctypes.c_uint32), ctypes.byref(count)))
        return base, int(count.value)

    def batch_get(self, keys, weights=None):
        """(servable, non-empty location map) per key."""
        k = np.ascontiguousarray(keys, dtype=np.int64)
        servable, nonempty = np.zeros(len(k), dtype=np.uint8), np.zeros(len(k), dtype=np.uint8)
        w = _w(weights)
        rc = lib().kvcm_ref_searcher_batch_get(self._h, _p(k, ctypes.c_int64), ctypes.c_int64(len(k)),
                                               _p(w, ctypes.c_uint32), _p(servable, ctypes.c_uint8),
                                               _p(nonempty, ctypes.c_uint8))
        if rc != 0:
            raise RuntimeError("BatchGetBestLocation / BatchGetLocation returned %d" % rc)
        return servable, nonempty

    def filter_write(self, keys, weights=None):
        """CacheManager::FilterWriteCache (kv_cache_manager/manager/cache_manager.cc:589-635) put together from what
        the reference's own BatchGetLocation and policy object say per key: ("offset", first missing, new keys) when
        the keys that exist for a write form a prefix, else ("vector", non-empty flags, keys with an empty map)."""
        k = np.ascontiguousarray(keys, dtype=np.int64)
        exists, nonempty = np.zeros(len(k), dtype=np.uint8), np.zeros(len(k), dtype=np.uint8)
        w = _w(weights)
        rc = lib().kvcm_ref_searcher_write_view(self._h, _p(k, ctypes.c_int64), ctypes.c_int64(len(k)),
                                                _p(w, ctypes.c_uint32), _p(exists, ctypes.c_uint8),
                                                _p(nonempty, ctypes.c_uint8))
        if rc != 0:
            raise RuntimeError("BatchGetLocation returned %d" % rc)
        exists, nonempty = exists.astype(bool), nonempty.astype(bool)
        first = int(np.argmin(exists)) if not exists.all() else len(k)
        if not exists[first:].any():
            return "offset", first, len(k) - first
        return "vector", nonempty, int((~nonempty).sum())

    def status(self, op, keys, types, expected=0, new_status=0):
        """One task per key (OP_UPDATE / OP_CAS / OP_CAD / OP_DELETE) on the key's location of storage type types[i]:
        (the call's ErrorCode, the ErrorCode of every task)."""
        k = np.ascontiguousarray(keys, dtype=np.int64)
        n = len(k)
        ty = np.ascontiguousarray(np.broadcast_to(np.asarray(types, dtype=np.int32), (n,)))
        ex = np.ascontiguousarray(np.broadcast_to(np.asarray(expected, dtype=np.int32), (n,)))
        nw = np.ascontiguousarray(np.broadcast_to(np.asarray(new_status, dtype=np.int32), (n,)))
        res = np.zeros(n, dtype=np.int32)
        rc = lib().kvcm_ref_searcher_status(self._h, ctypes.c_int32(op), _p(k, ctypes.c_int64), ctypes.c_int64(n),
                                            _p(ty, ctypes.c_int32), _p(ex, ctypes.c_int32), _p(nw, ctypes.c_int32),
                                            _p(res, ctypes.c_int32))
        return int(rc), res
