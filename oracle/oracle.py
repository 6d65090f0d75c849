"""ctypes face of the C oracle (``ugache_oracle.c``).  Test infrastructure only.

Every wrapper keeps the C function's name; see the C file for the reference file:line
each one follows.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libugache_oracle.so")


def build(force=False):
    """Compile the oracle with gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "ugache_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libugache_oracle.so"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.orc_murmur3_32.restype = C.c_uint32
        _lib.orc_murmur3_32.argtypes = [C.c_uint32, C.c_uint32]
        _lib.orc_pack_loc_off.restype = C.c_uint32
        _lib.orc_pack_loc_off.argtypes = [C.c_uint32, C.c_uint32]
        _lib.orc_word_loc.restype = C.c_uint32
        _lib.orc_word_loc.argtypes = [C.c_uint32]
        _lib.orc_word_off.restype = C.c_uint32
        _lib.orc_word_off.argtypes = [C.c_uint32]
        _lib.orc_table_size.restype = C.c_uint64
        _lib.orc_table_size.argtypes = [C.c_uint64, C.c_uint64]
        _lib.orc_use_flat_table.restype = C.c_int
        _lib.orc_use_flat_table.argtypes = [C.c_uint64, C.c_uint64]
        _lib.orc_cache_capacity.restype = C.c_uint64
        _lib.orc_cache_capacity.argtypes = [C.c_uint64, C.c_double]
        _lib.orc_simple_insert.restype = C.c_uint32
        _lib.orc_simple_search.restype = C.c_uint32
        _lib.orc_max_threads.restype = C.c_int
        for name in ("orc_solve_intuitive", "orc_solve_rep", "orc_solve_clique_part",
                     "orc_model_build", "orc_model_refresh_slots"):
            getattr(_lib, name).restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


RECORD = np.dtype([("dst", np.uint32), ("loc", np.uint32), ("off", np.uint64)])
BUCKET = np.dtype([("state_key", np.uint32), ("val", np.uint32)])


def murmur3_32(key, seed=0):
    return lib().orc_murmur3_32(key, seed)


def pack_loc_off(loc, off):
    return lib().orc_pack_loc_off(loc, off)


def table_size(num, scale=2):
    return lib().orc_table_size(num, scale)


def use_flat_table(cached_plus_remote, num_total):
    return bool(lib().orc_use_flat_table(cached_plus_remote, num_total))


def cache_capacity(num_total, cache_percentage):
    return lib().orc_cache_capacity(num_total, C.c_double(cache_percentage))


class SimpleTable:
    """The reference's probing table on the CPU."""

    def __init__(self, num_entries):
        self.size = table_size(max(int(num_entries), 2))
        self.buckets = np.empty(self.size, dtype=BUCKET)
        lib().orc_simple_init(_p(self.buckets), C.c_uint64(self.size))

    def insert(self, key, val):
        return lib().orc_simple_insert(_p(self.buckets), C.c_uint64(self.size), C.c_uint32(key),
                                       C.c_uint32(val))

    def search(self, key):
        return lib().orc_simple_search(_p(self.buckets), C.c_uint64(self.size), C.c_uint32(key))

    def evict(self, key):
        lib().orc_simple_evict(_p(self.buckets), C.c_uint64(self.size), C.c_uint32(key))

    def lookup(self, keys, fallback_loc, empty_feat=0):
        keys = np.ascontiguousarray(keys, dtype=np.int64)
        rec = np.empty(len(keys), dtype=RECORD)
        lib().orc_lookup_simple(_p(self.buckets), C.c_uint64(self.size), _p(keys),
                                C.c_uint64(len(keys)), C.c_int(fallback_loc), C.c_int(empty_feat),
                                _p(rec))
        return rec


def lookup_flat(words, keys, fallback_loc, empty_feat=0):
    words = np.ascontiguousarray(words, dtype=np.uint32)
    keys = np.ascontiguousarray(keys, dtype=np.int64)
    rec = np.empty(len(keys), dtype=RECORD)
    lib().orc_lookup_flat(_p(words), _p(keys), C.c_uint64(len(keys)), C.c_int(fallback_loc),
                          C.c_int(empty_feat), _p(rec))
    return rec


def extract_records(rec, sources, row_bytes, n_out=None):
    """sources: list of contiguous uint8-viewable arrays, indexed by location."""
    n_out = len(rec) if n_out is None else n_out
    out = np.zeros((n_out, row_bytes), dtype=np.uint8)
    ptrs = (C.c_void_p * len(sources))(*[s.ctypes.data if s is not None else 0 for s in sources])
    lib().orc_extract_records(_p(rec), C.c_uint64(len(rec)), ptrs, C.c_uint64(row_bytes), _p(out))
    return out


def gather(table, keys, empty_feat=0, num_threads=0, out=None):
    """out[i] = table[keys[i]] (rows as raw bytes)."""
    table = np.ascontiguousarray(table)
    keys = np.ascontiguousarray(keys, dtype=np.int64)
    row_bytes = table.strides[0]
    if out is None:
        out = np.empty((len(keys),) + table.shape[1:], dtype=table.dtype)
    lib().orc_gather(_p(table), _p(keys), C.c_uint64(len(keys)), C.c_uint64(row_bytes),
                     C.c_int(empty_feat), _p(out), C.c_int(num_threads))
    return out


def pool(table, keys, offsets=None, bag_size=0, mean=False, empty_feat=0, num_keys=None):
    """Embedding-bag restatement: ``out[b] = sum over the keys of bag b of table[key]`` as fp32,
    added in key order starting from +0 (one IEEE addition per row and element; fp16 elements
    are widened first); ``mean`` divides once by the bag's length; ids outside the table add
    nothing; an empty bag gives zeros.  No reference counterpart: the reference's applications
    pool in the model (example/dlr/main.py).  numpy, position by position over all bags at once,
    which keeps every bag's own order."""
    table = np.ascontiguousarray(table)
    keys = np.ascontiguousarray(keys, dtype=np.int64)
    n = len(keys)
    if offsets is None:
        n_bags = n // bag_size
        offsets = np.arange(n_bags + 1, dtype=np.int64) * bag_size
    offsets = np.clip(np.asarray(offsets, dtype=np.int64), 0, n)
    begin, end = offsets[:-1], np.maximum(offsets[1:], offsets[:-1])
    length = end - begin
    out = np.zeros((len(begin), table.shape[1]), dtype=np.float32)
    mask_rows = (1 << empty_feat) - 1 if empty_feat else None
    limit = table.shape[0] if num_keys is None else num_keys   # ids of the key space
    for j in range(int(length.max()) if len(length) else 0):
        bags = np.nonzero(length > j)[0]
        k = keys[begin[bags] + j]
        ok = (k >= 0) & (k < limit)
        bags, k = bags[ok], k[ok]
        if mask_rows is not None:
            k = k & mask_rows
        out[bags] = out[bags] + table[k].astype(np.float32)
    if mean:
        nz = length > 0
        out[nz] = out[nz] / length[nz].astype(np.float32)[:, None]
    return out


def max_threads():
    return lib().orc_max_threads()


def fill(host_table, keys, slots, slice_rows, empty_feat=0):
    host_table = np.ascontiguousarray(host_table)
    keys = np.ascontiguousarray(keys, dtype=np.uint32)
    sl = None if slots is None else np.ascontiguousarray(slots, dtype=np.uint32)
    out = np.zeros((slice_rows,) + host_table.shape[1:], dtype=host_table.dtype)
    lib().orc_fill(_p(host_table), _p(keys), _p(sl) if sl is not None else None,
                   C.c_uint64(len(keys)), C.c_uint64(host_table.strides[0]), C.c_int(empty_feat),
                   _p(out))
    return out


class Placement:
    def __init__(self, nid_to_block, block_placement, block_access_from, block_density):
        self.nid_to_block = nid_to_block
        self.block_placement = block_placement
        self.block_access_from = block_access_from  # [G, B]
        self.block_density = block_density

    @property
    def num_block(self):
        return len(self.block_placement)

    @property
    def num_device(self):
        return self.block_access_from.shape[0]


def _alloc_placement(G, N, B):
    return (np.zeros(N, dtype=np.uint32), np.zeros(B, dtype=np.uint8),
            np.zeros((G, B), dtype=np.uint8), np.zeros(B, dtype=np.float64))


def solve_intuitive(G, rank_ids, rank_freqs, cache_percent, T_local, T_remote, T_cpu,
                    min_freq=0.0):
    rank_ids = np.ascontiguousarray(rank_ids, dtype=np.uint32)
    rank_freqs = np.ascontiguousarray(rank_freqs, dtype=np.uint32)
    N = len(rank_ids)
    n2b, bp, ba, bd = _alloc_placement(G, N, G + 2)
    nb = lib().orc_solve_intuitive(C.c_int(G), C.c_uint32(N), _p(rank_ids), _p(rank_freqs),
                                   C.c_double(cache_percent), C.c_double(T_local),
                                   C.c_double(T_remote), C.c_double(T_cpu), C.c_double(min_freq),
                                   _p(n2b), _p(bp), _p(ba), _p(bd))
    assert nb == G + 2
    return Placement(n2b, bp, ba, bd)


def solve_rep(G, rank_ids, cache_percent):
    rank_ids = np.ascontiguousarray(rank_ids, dtype=np.uint32)
    N = len(rank_ids)
    n2b, bp, ba, bd = _alloc_placement(G, N, 2)
    lib().orc_solve_rep(C.c_int(G), C.c_uint32(N), _p(rank_ids), C.c_double(cache_percent),
                        _p(n2b), _p(bp), _p(ba), _p(bd))
    return Placement(n2b, bp, ba, bd)


def solve_clique_part(G, rank_ids, cache_percent, clique_size=None):
    clique_size = G if clique_size is None else clique_size
    rank_ids = np.ascontiguousarray(rank_ids, dtype=np.uint32)
    N = len(rank_ids)
    n2b, bp, ba, bd = _alloc_placement(G, N, clique_size + 1)
    lib().orc_solve_clique_part(C.c_int(G), C.c_int(clique_size), C.c_uint32(N), _p(rank_ids),
                                C.c_double(cache_percent), _p(n2b), _p(bp), _p(ba), _p(bd))
    return Placement(n2b, bp, ba, bd)


def model_build(placement, rank, capacity):
    """(words[N], per_src_count[G+1], slot_of[G, N]) for reader `rank`."""
    G, N, B = placement.num_device, len(placement.nid_to_block), placement.num_block
    slot_of = np.empty((G, N), dtype=np.uint32)
    words = np.empty(N, dtype=np.uint32)
    cnt = np.zeros(G + 1, dtype=np.uint64)
    ba = np.ascontiguousarray(placement.block_access_from)
    rc = lib().orc_model_build(C.c_int(G), C.c_uint32(N), _p(placement.nid_to_block), _p(ba),
                               C.c_int(B), C.c_int(rank), C.c_uint64(capacity), _p(slot_of),
                               _p(words), _p(cnt))
    if rc != 0:
        raise ValueError("a GPU's key list exceeds the cache capacity")
    return words, cnt, slot_of


def model_refresh_slots(gpu, old, new, slots, free_list):
    """Updates slots (u32[N]) in place; returns (new_free_list, n_evicted, n_inserted)."""
    N = len(slots)
    cap = len(free_list) + N
    fl = np.empty(cap, dtype=np.uint32)
    fl[:len(free_list)] = free_list
    nf = C.c_uint64(len(free_list))
    ev, ins = C.c_uint64(0), C.c_uint64(0)
    rc = lib().orc_model_refresh_slots(C.c_uint32(N), C.c_int(gpu), _p(old.nid_to_block),
                                       _p(old.block_placement), _p(new.nid_to_block),
                                       _p(new.block_placement), _p(slots), _p(fl), C.byref(nf),
                                       C.c_uint64(cap), C.byref(ev), C.byref(ins))
    if rc != 0:
        raise ValueError("free list exhausted")
    return fl[:nf.value].copy(), ev.value, ins.value


def gen_rows(seed, row_begin, n_rows, dim, dtype=np.float32):
    if np.dtype(dtype) == np.float32:
        out = np.empty((n_rows, dim), dtype=np.float32)
        lib().orc_gen_rows_f32(C.c_uint64(seed), C.c_uint64(row_begin), C.c_uint64(n_rows),
                               C.c_uint64(dim), _p(out))
        return out
    out = np.empty((n_rows, dim), dtype=np.uint16)
    lib().orc_gen_rows_f16(C.c_uint64(seed), C.c_uint64(row_begin), C.c_uint64(n_rows),
                           C.c_uint64(dim), _p(out))
    return out.view(np.float16)


def gen_rows_for_keys(seed, keys, dim, dtype=np.float32):
    keys = np.ascontiguousarray(keys, dtype=np.int64)
    if np.dtype(dtype) == np.float32:
        out = np.empty((len(keys), dim), dtype=np.float32)
        lib().orc_gen_rows_for_keys_f32(C.c_uint64(seed), _p(keys), C.c_uint64(len(keys)),
                                        C.c_uint64(dim), _p(out))
        return out
    out = np.empty((len(keys), dim), dtype=np.uint16)
    lib().orc_gen_rows_for_keys_f16(C.c_uint64(seed), _p(keys), C.c_uint64(len(keys)),
                                    C.c_uint64(dim), _p(out))
    return out.view(np.float16)


def zipf_ranks(u, N, alpha):
    u = np.ascontiguousarray(u, dtype=np.float64)
    out = np.empty(len(u), dtype=np.int64)
    lib().orc_zipf_ranks(_p(u), C.c_uint64(len(u)), C.c_uint64(N), C.c_double(alpha), _p(out))
    return out


def rank_to_id(rank0, N, A, B):
    rank0 = np.ascontiguousarray(rank0, dtype=np.int64)
    out = np.empty(len(rank0), dtype=np.int64)
    lib().orc_rank_to_id(_p(rank0), C.c_uint64(len(rank0)), C.c_uint64(N), C.c_uint64(A),
                         C.c_uint64(B), _p(out))
    return out
