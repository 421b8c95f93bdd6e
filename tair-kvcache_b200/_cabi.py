"""ctypes binding of libkvcm_b200.so - the only way this package reaches the GPU.

There is no CPU path: if the library has not been built or cannot be loaded, importing this
module's `lib()` raises, and every wrapper raises KvcmError on a non-zero return code.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkvcm_b200.so")

KVCM_OK = 0
KVCM_ER_INVALID_PARAMS = 3
KVCM_ER_INVALID_ADDRESS = 107
KVCM_ER_UNSUPPORTED_MEMORY_TYPE = 109
KVCM_ER_CUDAMEMCPY_ERROR = 112
KVCM_ER_CUDA_STREAM_SYNCHRONIZE_ERROR = 115
KVCM_ER_NO_DEVICE = 900
KVCM_EC_BASE = 1000
KVCM_EC_ERROR = KVCM_EC_BASE + 1
KVCM_EC_NOENT = KVCM_EC_BASE + 2
KVCM_EC_BADARGS = KVCM_EC_BASE + 6
KVCM_EC_EXIST = KVCM_EC_BASE + 4
KVCM_EC_NOSPC = KVCM_EC_BASE + 9
KVCM_EC_OUT_OF_LIMIT = KVCM_EC_BASE + 14
KVCM_EC_MISMATCH = KVCM_EC_BASE + 16
STATUS_ANY = STATUS_DELETE = 0xFF
STATUS_DELETE_KEEP_KEY = 0xFE
VAL_STATUS_SHIFT = 33
REPLAY_NOALLOC_MAX_KEYS = 262144
POLICY_LEAF_AWARE_LRU, POLICY_LRU, POLICY_RANDOM_LRU = 0, 1, 2  # kvcm_b200_replay_policy_group's per-instance policy bytes

VAL_NONEMPTY = 1 << 32
VAL_PRESENT = 1 << 63
AVAIL_ALL = 0xFFFF
FLAG_SERVABLE, FLAG_EXISTS, FLAG_NONEMPTY, FLAG_WRITABLE, FLAG_HAS_CLASS = 1, 2, 4, 8, 16

_vp = ctypes.c_void_p
_i32 = ctypes.c_int32
_i64 = ctypes.c_int64
_u32 = ctypes.c_uint32
_u64 = ctypes.c_uint64


class Seg(ctypes.Structure):
    _fields_ = [("dst", _vp), ("src", _vp), ("bytes", _u64)]


class IndexExport(ctypes.Structure):
    _fields_ = [("ipc_handle", ctypes.c_uint8 * 64), ("n_slots", _u64), ("device", _i32), ("reserved_", _i32)]


class RouteExport(ctypes.Structure):
    _fields_ = [("ipc_handle", ctypes.c_uint8 * 64), ("capacity_keys", _u64), ("device", _i32), ("reserved_", _i32)]


class Iov(ctypes.Structure):
    _fields_ = [("type", ctypes.c_uint8), ("ignore", ctypes.c_uint8), ("pad_", ctypes.c_uint8 * 6), ("base", _vp),
                ("size", _u64)]


# name -> argtypes, in the order of include/kvcm_b200.h; every function returns int32 unless noted.
_MOVE = [_vp, _i32, _vp, _i64, _vp, _vp, _i32, _i32, _i64, _i64, _vp, _i32, _vp]
_LEGACY = [_vp, _i32, _i64, _vp, _vp, _i32, _i64, _vp]
_HASH = [_vp, _i64, _vp, _i32, _i32, _vp, _vp, _vp, _i32, _vp]
SIGNATURES = {
    "kvcm_b200_abi_version": [],
    "kvcm_b200_set_device": [_i32],
    "kvcm_b200_error_string": [_i32],
    "kvcm_b200_device_info": [_vp, _vp, _vp, _vp],
    "kvcm_b200_selftest_bounded_wait": [_u32, _vp, _vp],
    "kvcm_b200_gather_tokens": _MOVE,
    "kvcm_b200_scatter_tokens": _MOVE,
    "kvcm_b200_gather_pages": _MOVE,
    "kvcm_b200_scatter_pages": _MOVE,
    "kvcm_b200_save_rows_to_host": [_vp, _i32, _vp, _i64, _vp, _vp, _i32, _i32, _i64, _i64, _vp, _i64, _vp, _vp],
    "kvcm_b200_load_rows_from_host": [_vp, _i32, _vp, _i64, _vp, _vp, _i32, _i32, _i64, _i64, _vp, _i64, _vp, _vp],
    "kvcm_b200_set_mover": [_i32, _i32],
    "kvcm_b200_set_bulk_geometry": [_i32, _i32, _i32],
    "kvcm_b200_set_bulk_min_row_bytes": [_i32],
    "kvcm_b200_gather_legacy": _LEGACY,
    "kvcm_b200_scatter_legacy": _LEGACY,
    "kvcm_b200_copy_segments": [_vp, _i32, _vp],
    "kvcm_b200_copy_segments_sized": [_vp, _i32, _u64, _vp],
    "kvcm_b200_copy_wait_timeouts": [_vp],
    "kvcm_b200_iovs_to_segments": [_vp, _i32, _vp, _i32, _vp, _vp, _vp],
    "kvcm_b200_iov_crc": [_vp, _i32, _u64, _vp, _vp],
    "kvcm_b200_hash_blocks_u32": _HASH,
    "kvcm_b200_hash_blocks_i64": _HASH,
    "kvcm_b200_hash_wait_timeouts": [_vp],
    "kvcm_b200_key_offsets": [_vp, _i32, _i32, _vp],
    "kvcm_b200_length_order": [_vp, _i32, _vp, _vp],
    "kvcm_b200_index_create": [_i64, _vp],
    "kvcm_b200_index_destroy": [_vp],
    "kvcm_b200_index_clear": [_vp, _vp],
    "kvcm_b200_index_stats": [_vp, _vp, _vp, _vp],
    "kvcm_b200_index_usage": [_vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_index_rehash_workspace_bytes": [_vp],
    "kvcm_b200_index_rehash": [_vp, _vp, _i64, _vp, _vp],
    "kvcm_b200_index_set_auto_rehash": [_vp, _i64],
    "kvcm_b200_index_update_status": [_vp, _vp, _vp, _u32, _i64, _vp, _vp],
    "kvcm_b200_index_update_status_sharded": [_vp, _vp, _vp, _u32, _i64, _i32, _i32, _vp, _vp],
    "kvcm_b200_start_write_workspace_bytes": [_i64, _i32],
    "kvcm_b200_start_write": [_vp, _vp, _vp, _i32, _i64, _u32, _i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_write_snapshot_sharded": [_vp, _vp, _i64, _u32, _i32, _i32, _i32, _vp, _vp],
    "kvcm_b200_start_write_sharded": [_vp, _vp, _vp, _i32, _i64, _u32, _i32, _vp, _vp, _i32, _i32, _vp, _i64, _vp, _vp,
                                      _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_finish_write_sharded": [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp],
    "kvcm_b200_finish_write": [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp],
    "kvcm_b200_index_add_location": [_vp, _vp, _vp, _i32, _i32, _i64, _vp, _vp, _vp],
    "kvcm_b200_index_add_location_sharded": [_vp, _vp, _vp, _i32, _i32, _i64, _i32, _i32, _vp, _vp, _vp],
    "kvcm_b200_index_upsert": [_vp, _vp, _vp, _u64, _i64, _vp, _vp],
    "kvcm_b200_index_erase": [_vp, _vp, _i64, _vp],
    "kvcm_b200_index_lookup": [_vp, _vp, _i64, _vp, _vp],
    "kvcm_b200_match_prefix": [_vp, _vp, _vp, _i32, _vp, _vp, _u32, _vp, _vp],
    "kvcm_b200_match_sw": [_vp, _vp, _vp, _i32, _i32, _u32, _vp, _vp],
    "kvcm_b200_batch_get": [_vp, _vp, _i64, _u32, _vp, _vp],
    "kvcm_b200_filter_write": [_vp, _vp, _vp, _i32, _u32, _vp, _vp, _vp, _vp],
    "kvcm_b200_index_upsert_sharded": [_vp, _vp, _vp, _u64, _i64, _i32, _i32, _vp, _vp],
    "kvcm_b200_match_prefix_sharded": [_vp, _vp, _vp, _i32, _vp, _vp, _u32, _i32, _i32, _vp, _vp],
    "kvcm_b200_batch_get_sharded": [_vp, _vp, _i64, _u32, _i32, _i32, _vp, _vp],
    "kvcm_b200_match_sw_from_flags": [_vp, _vp, _i32, _i32, _vp, _vp],
    "kvcm_b200_route_count": [_vp, _i64, _i32, _vp, _vp],
    "kvcm_b200_route_scatter": [_vp, _i64, _i32, _vp, _vp, _vp, _vp],
    "kvcm_b200_gather_bytes": [_vp, _vp, _i64, _vp, _vp],
    "kvcm_b200_match_prefix_from_flags": [_vp, _vp, _i32, _vp, _vp, _vp, _vp],
    "kvcm_b200_route_area_create": [_i64, _vp],
    "kvcm_b200_route_area_destroy": [_vp],
    "kvcm_b200_route_area_export": [_vp, _vp],
    "kvcm_b200_route_area_attach": [_vp, _i32, _i32, _vp],
    "kvcm_b200_route_area_attach_local": [_vp, _i32, _i32, _vp],
    "kvcm_b200_route_area_detach": [_vp],
    "kvcm_b200_route_dispatch": [_vp, _vp, _i64, _vp, _vp, _vp, _vp],
    "kvcm_b200_route_answer": [_vp, _vp, _vp, _u32, _vp],
    "kvcm_b200_route_collect": [_vp, _vp, _i64, _vp, _vp],
    "kvcm_b200_index_export": [_vp, _vp],
    "kvcm_b200_index_attach_peers": [_vp, _i32, _i32, _vp],
    "kvcm_b200_index_attach_local_peers": [_vp, _i32, _i32, _vp],
    "kvcm_b200_index_detach_peers": [_vp],
    "kvcm_b200_replay_workspace_bytes": [_i64],
    "kvcm_b200_replay": [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_replay_lru_workspace_bytes": [_i64, _i32],
    "kvcm_b200_replay_lru": [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _vp, _i32, _i32, _i32, _vp, _i64, _vp, _vp, _vp, _vp,
                             _vp, _vp, _vp],
    "kvcm_b200_replay_lru_group_workspace_bytes": [_i64, _i32, _i32],
    "kvcm_b200_replay_lru_group_records": [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _vp, _i32, _i32, _i32, _vp,
                                           _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_replay_lru_group": [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _vp, _i32, _i32, _i32, _vp, _i64,
                                   _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_replay_leaf_lru_workspace_bytes": [_i64, _i32, _i32],
    "kvcm_b200_replay_leaf_lru": [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _vp, _i32, _i32, _i32, _vp, _i64, _vp, _vp,
                                  _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_replay_leaf_lru_group_workspace_bytes": [_i64, _i32, _i32, _i32],
    "kvcm_b200_replay_leaf_lru_group": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _vp, _i32, _i32, _i32, _vp,
                                        _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_replay_tree_group": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _vp, _i32, _i32, _i32, _vp,
                                    _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_replay_policy_group_workspace_bytes": [_i64, _i32, _i32, _vp, _i32],
    "kvcm_b200_replay_policy_group": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _vp, _i32, _i32,
                                      _i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_replay_random_lru_workspace_bytes": [_i64, _i32],
    "kvcm_b200_replay_random_lru_group_workspace_bytes": [_i64, _i32, _i32],
    "kvcm_b200_replay_random_lru_group": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _vp, _i32, _i32, _i32,
                                          _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_selftest_partial_sort": [_vp, _vp, _u32, _u32],
    "kvcm_b200_replay_random_lru": [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _vp, _i32, _i32, _i32, ctypes.c_double,
                                    _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "kvcm_b200_trace_replay_order": [_vp, _i64, _vp],
    "kvcm_b200_string_map_iteration_order": [_vp, _vp, _vp, _i64, _vp, _vp],
    "kvcm_b200_replay_noalloc": [_vp, _vp, _vp, _vp, _i32, _i64, _vp, _vp, _vp, _vp, _vp, _vp],
}


class KvcmError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__("%s failed with code %d (%s)" % (what, code, error_string(code)))


_lib = None


def lib():
    """The loaded library.  Raises if it is missing: this package has no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with __graft_entry__.build() "
                              "(nvcc, sm_100a); there is no CPU fallback" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = (ctypes.c_char_p if name == "kvcm_b200_error_string" else
                          _i64 if name.endswith("_workspace_bytes") else _i32)
        _lib = L
    return _lib


def error_string(code):
    return lib().kvcm_b200_error_string(code).decode()


def check(code, what):
    if code != KVCM_OK:
        raise KvcmError(code, what)


def call(name, *args):
    check(getattr(lib(), name)(*args), name)


_tls = threading.local()


def bind_device(index):
    """Make CUDA device `index` current for this thread inside the library's own CUDA runtime
    (it is linked statically, so torch.cuda.set_device does not reach it)."""
    index = 0 if index is None else int(index)
    if getattr(_tls, "device", None) != index:
        call("kvcm_b200_set_device", index)
        _tls.device = index


_shim = None
_shim_tried = False


def shim():
    """The pybind11 module over the same C ABI (built next to the library), or None when it is not there.
    The gather / scatter operators of py_connector go through it; ctypes is the equivalent route without it."""
    global _shim, _shim_tried
    if not _shim_tried:
        _shim_tried = True
        if os.environ.get("KVCM_B200_NO_PYBIND", "") == "":
            try:
                from . import kvcm_b200_py as mod
                if mod.abi_version() == lib().kvcm_b200_abi_version():
                    _shim = mod
            except ImportError:
                _shim = None
    return _shim


def call_move(name, *args):
    """A gather / scatter entry point by its C name with integer addresses (None = NULL): through the pybind
    shim when it is built, else through ctypes.  Raises KvcmError on a non-zero code either way."""
    mod = shim()
    if mod is not None:
        fn = getattr(mod, name[len("kvcm_b200_"):], None)
        if fn is not None:
            check(fn(*[0 if a is None else int(a) for a in args]), name)
            return
    call(name, *args)
