"""ctypes binding of ``libugache_b200.so`` (the C ABI declared in include/ugache_b200.h).

Loading fails loudly when the shared library is missing: there is no CPU fallback.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libugache_b200.so")

UGC_MAX_DEVICE = 8
UGC_OK = 0
POLICY_INTUITIVE, POLICY_REP, POLICY_CLIQUE_PART, POLICY_SPLIT_SEARCH = 9, 12, 14, 100
TABLE_AUTO, TABLE_FLAT, TABLE_HASHED = 0, 1, 2
EXTRACT_AUTO, EXTRACT_GROUPED, EXTRACT_DIRECT = 0, 1, 2

ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_size_t, C.c_void_p)
FREE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)


class Config(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("num_device", C.c_int32),
        ("num_total_item", C.c_uint64),
        ("row_bytes", C.c_uint32),
        ("cache_percentage", C.c_double),
        ("empty_feat", C.c_int32),
        ("table_kind", C.c_int32),
        ("max_batch", C.c_uint32),
        ("register_host", C.c_int32),
        ("bw_local_gbs", C.c_double),
        ("bw_remote_gbs", C.c_double),
        ("bw_host_gbs", C.c_double),
        ("gather_ctas_per_sm", C.c_int32),
        ("host_ctas", C.c_int32),
        ("remote_ctas", C.c_int32),
        ("gather_vec_bytes", C.c_int32),
        ("alloc", ALLOC_FN),
        ("free", FREE_FN),
        ("alloc_user", C.c_void_p),
    ]


class PeerHandle(C.Structure):
    _fields_ = [
        ("replica_id", C.c_int32),
        ("device_id", C.c_int32),
        ("pid", C.c_int64),
        ("slice_ptr", C.c_uint64),
        ("table_ptr", C.c_uint64),
        ("table_lines", C.c_uint64),
        ("table_kind", C.c_int32),
        ("has_ipc", C.c_int32),
        ("slice_ipc", C.c_ubyte * 64),
        ("table_ipc", C.c_ubyte * 64),
    ]


class Stats(C.Structure):
    _fields_ = [
        ("num_local_rows", C.c_uint64),
        ("num_remote_keys", C.c_uint64),
        ("num_host_keys", C.c_uint64),
        ("capacity_rows", C.c_uint64),
        ("free_rows", C.c_uint64),
        ("table_kind", C.c_int32),
        ("table_bytes", C.c_uint64),
        ("slice_bytes", C.c_uint64),
        ("last_keys", C.c_uint64),
        ("last_local", C.c_uint64),
        ("last_remote", C.c_uint64),
        ("last_host", C.c_uint64),
        ("err_key_range", C.c_uint64),
        ("err_table", C.c_uint64),
        ("lookups", C.c_uint64),
        ("last_local_ns", C.c_uint64),
        ("last_remote_ns", C.c_uint64),
        ("last_host_ns", C.c_uint64),
        ("last_index_ns", C.c_uint64),
        ("device_bytes_from_allocator", C.c_uint64),
        ("device_bytes_own", C.c_uint64),
        ("lookups_host_ordered", C.c_uint64),
        ("lookups_direct", C.c_uint64),
        ("kernel_launches", C.c_uint64),
        ("lookups_pooled", C.c_uint64),
        ("pool_rows", C.c_uint64 * 3),
    ]


class Tuning(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("gather_ctas_per_sm", C.c_int32),
        ("gather_block_threads", C.c_int32),
        ("gather_vec_bytes", C.c_int32),
        ("host_ctas", C.c_int32),
        ("remote_ctas", C.c_int32),
        ("bulk_mask", C.c_int32),
        ("lookup_keys_per_thread", C.c_int32),
        ("programmatic_launch", C.c_int32),
        ("extract_mode", C.c_int32),
        ("direct_ctas_per_sm", C.c_int32),
        ("direct_max_host_rows", C.c_int32),
        ("direct_block_threads", C.c_int32),
        ("direct_tile_keys", C.c_int32),
        ("direct_deep", C.c_int32),
        ("direct_early_host", C.c_int32),
        ("host_order_min_rows", C.c_int32),
        ("refresh_fill_ctas", C.c_int32),
        ("refresh_fill_batch_rows", C.c_int32),
        ("refresh_fill_pause_us", C.c_int32),
        ("refresh_early_repoint", C.c_int32),
        ("pool_vec_bytes", C.c_int32),
        ("gather_dynamic", C.c_int32),
        ("split_fixed", C.c_int32),
        ("host_zero_copy", C.c_int32),
    ]


class LinkDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("num_device", C.c_int32),
        ("bw_local_gbs", C.c_double), ("bw_remote_gbs", C.c_double), ("bw_host_gbs", C.c_double),
        ("lat_local_us", C.c_double), ("lat_remote_us", C.c_double), ("lat_host_us", C.c_double),
        ("host_rows_per_s", C.c_double),
        ("host_total_gbs", C.c_double),
        ("t_local", C.c_double), ("t_remote", C.c_double), ("t_cpu", C.c_double),
        ("host_ctas", C.c_int32), ("remote_ctas", C.c_int32), ("per_peer_ctas", C.c_int32),
    ]


class UgcError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("ugache_b200 status %d: %s" % (status, message))
        self.status = status


_lib = None

# name -> (restype, argtypes); every symbol include/ugache_b200.h declares
_P, _I, _U64, _SZ, _D = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t, C.c_double
SIGNATURES = {
    "ugc_abi_sizes": (_I, [C.POINTER(C.c_uint32 * 5)]),
    "ugc_version": (C.c_char_p, []),
    "ugc_last_error": (C.c_char_p, []),
    "ugc_status_string": (C.c_char_p, [_I]),
    "ugc_config_default": (_I, [C.POINTER(Config)]),
    "ugc_create": (_I, [C.POINTER(Config), C.POINTER(_P)]),
    "ugc_destroy": (_I, [_P]),
    "ugc_solve_placement": (_I, [_I, _I, _U64, _P, _P, _D, _D, _D, _D, _P, _P, _P, _P,
                                 C.POINTER(_I)]),
    "ugc_link_model": (_I, [_I, C.POINTER(_D), C.POINTER(_D), C.POINTER(_D)]),
    "ugc_link_desc": (_I, [_I, C.c_uint32, C.POINTER(LinkDesc)]),
    "ugc_placement_cost": (_I, [_I, _U64, _P, _P, _P, _P, _I, _D, _D, _D, _P]),
    "ugc_set_placement": (_I, [_P, _P, _P, _P, _P, _I]),
    "ugc_classify_keys": (_I, [_P, _I, _P, _P]),
    "ugc_build": (_I, [_P, _I, _I, _P, _P]),
    "ugc_export": (_I, [_P, _I, C.POINTER(PeerHandle)]),
    "ugc_import_peer": (_I, [_P, _I, C.POINTER(PeerHandle)]),
    "ugc_connect_local": (_I, [_P]),
    "ugc_attach_peers": (_I, [_P, _I, _P]),
    "ugc_lookup_u32": (_I, [_P, _I, _P, _SZ, _P, _P]),
    "ugc_lookup_i64": (_I, [_P, _I, _P, _SZ, _P, _P]),
    "ugc_lookup_i64_static": (_I, [_P, _I, _P, _SZ, _P, _P]),
    "ugc_lookup_unique": (_I, [_P, _I, _P, _I, _SZ, _P, _P, _P, _P, _P]),
    "ugc_lookup_pool": (_I, [_P, _I, _P, _I, _SZ, _P, _SZ, _SZ, _I, _I, _P, _P]),
    "ugc_reserve_batch": (_I, [_P, _I, C.c_uint32]),
    "ugc_lookup_host": (_I, [_P, _I, _P, _I, _SZ, _P, _P]),
    "ugc_refresh_set_placement": (_I, [_P, _P, _P, _P, _P, _I]),
    "ugc_refresh_evict": (_I, [_P, _I, _P]),
    "ugc_refresh_fill": (_I, [_P, _I, _P]),
    "ugc_refresh_attach": (_I, [_P, _I, _P]),
    "ugc_refresh_commit": (_I, [_P]),
    "ugc_record": (_I, [_P, _I, _P, _I, _SZ, _P]),
    "ugc_hotness_read": (_I, [_P, _I, _P, _I, _P]),
    "ugc_stats": (_I, [_P, _I, C.POINTER(Stats)]),
    "ugc_get_tuning": (_I, [_P, _I, C.POINTER(Tuning)]),
    "ugc_set_tuning": (_I, [_P, _I, C.POINTER(Tuning)]),
    "ugc_profile_begin": (_I, [_P, _I, _I]),
    "ugc_profile_end": (_I, [_P, _I, C.POINTER(_D), C.POINTER(_D), C.POINTER(_U64)]),
    "ugc_table_words": (_I, [_P, _I, _P, _SZ, _P, _P]),
    "ugc_host_register": (_I, [_P, _SZ, C.POINTER(_P)]),
    "ugc_host_unregister": (_I, [_P]),
    "ugc_host_unregister_sized": (_I, [_P, _SZ]),
    "ugc_host_alloc": (_I, [_SZ, C.POINTER(_P), C.POINTER(_P)]),
    "ugc_host_free": (_I, [_P]),
    "ugc_host_is_large_page": (_I, [_P]),
    "ugc_gen_table": (_I, [_P, _U64, _U64, _U64, _U64, _I, _P]),
}


def lib():
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "libugache_b200.so is missing (%s): build it with "
                "`python -m ugache_b200.build`; there is no CPU fallback" % LIB_PATH)
        _lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
        sizes = (C.c_uint32 * 5)()
        _lib.ugc_abi_sizes(C.byref(sizes))
        mine = [C.sizeof(t) for t in (Config, PeerHandle, Stats, Tuning, LinkDesc)]
        if list(sizes) != mine:
            _lib = None
            raise ImportError("libugache_b200.so does not match this binding (struct sizes %s, "
                              "expected %s): rebuild with `python -m ugache_b200.build`"
                              % (list(sizes), mine))
    return _lib


def check(status):
    if status != UGC_OK:
        raise UgcError(status, lib().ugc_last_error().decode())
