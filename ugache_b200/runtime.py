"""Python face of the C ABI: a thin object wrapper that moves pointers, nothing else.

PyTorch appears here only to own device memory and streams; every operation is a call
into ``libugache_b200.so``.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import (POLICY_CLIQUE_PART, POLICY_INTUITIVE, POLICY_REP, POLICY_SPLIT_SEARCH, TABLE_AUTO, TABLE_FLAT,
                   TABLE_HASHED, UgcError, check)

POLICIES = {"intuitive": POLICY_INTUITIVE, "coll_intuitive": POLICY_INTUITIVE,
            "rep": POLICY_REP, "clique_part": POLICY_CLIQUE_PART,
            "split_search": POLICY_SPLIT_SEARCH}


class PlacementArrays:
    """The four placement arrays (numpy, host)."""

    def __init__(self, nid_to_block, block_placement, block_access_from, block_density):
        self.nid_to_block = np.ascontiguousarray(nid_to_block, dtype=np.uint32)
        self.block_placement = np.ascontiguousarray(block_placement, dtype=np.uint8)
        self.block_access_from = np.ascontiguousarray(block_access_from, dtype=np.uint8)
        self.block_density = np.ascontiguousarray(block_density, dtype=np.float64)

    @property
    def num_block(self):
        return len(self.block_placement)

    @property
    def num_device(self):
        return self.block_access_from.shape[0]


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def link_desc(num_device, row_bytes=0):
    """The library's B200 link description as a dict (bandwidths, latencies, the scattered
    host-row rate, time-per-byte ratios, CTA budgets of the far links)."""
    d = _lib.LinkDesc()
    d.struct_size = C.sizeof(_lib.LinkDesc)
    check(_lib.lib().ugc_link_desc(num_device, row_bytes or 0, C.byref(d)))
    return {name: getattr(d, name) for name, _ in d._fields_ if name != "struct_size"}


def link_model(num_device, row_bytes=None):
    """(t_local, t_remote, t_cpu) time-per-byte ratios of the library's B200 link model.  With
    ``row_bytes`` the host term is what scattered row reads really cost (the row rate and the
    host side shared by ``num_device`` GPUs) when that is slower than the link bandwidth."""
    if row_bytes:
        d = link_desc(num_device, row_bytes)
        return d["t_local"], d["t_remote"] if num_device > 1 else 8000.0 / 900.0, d["t_cpu"]
    tl, tr, tc = C.c_double(), C.c_double(), C.c_double()
    check(_lib.lib().ugc_link_model(num_device, C.byref(tl), C.byref(tr), C.byref(tc)))
    return tl.value, tr.value, tc.value


def solve_placement(policy, num_device, rank_ids, rank_freqs, cache_percent, t_local=None,
                    t_remote=None, t_cpu=None):
    """The reference's non-MILP placement heuristics; cache_percent in percent (0..100)."""
    pol = POLICIES[policy] if isinstance(policy, str) else int(policy)
    rank_ids = np.ascontiguousarray(rank_ids, dtype=np.uint32)
    N = len(rank_ids)
    freqs = None if rank_freqs is None else np.ascontiguousarray(rank_freqs, dtype=np.uint32)
    dl, dr, dc = link_model(num_device)
    t_local = dl if t_local is None else t_local
    t_remote = dr if t_remote is None else t_remote
    t_cpu = dc if t_cpu is None else t_cpu
    B = num_device + 2
    n2b = np.zeros(N, dtype=np.uint32)
    bp = np.zeros(B, dtype=np.uint8)
    ba = np.zeros(num_device * B, dtype=np.uint8)
    bd = np.zeros(B, dtype=np.float64)
    nb = C.c_int(0)
    check(_lib.lib().ugc_solve_placement(pol, num_device, N, _ptr(rank_ids),
                                         _ptr(freqs) if freqs is not None else None,
                                         cache_percent, t_local, t_remote, t_cpu, _ptr(n2b),
                                         _ptr(bp), _ptr(ba), _ptr(bd), C.byref(nb)))
    b = nb.value
    return PlacementArrays(n2b, bp[:b].copy(), ba[:num_device * b].reshape(num_device, b).copy(),
                           bd[:b].copy())


def placement_cost(placement, rank_ids, rank_freqs, t_local=None, t_remote=None, t_cpu=None):
    """Modelled cost per reader (concurrent sources: the slowest of HBM, peer links and host
    link, in units of t_local per looked-up byte) of a placement against a hotness record."""
    G = placement.num_device
    rank_ids = np.ascontiguousarray(rank_ids, dtype=np.uint32)
    freqs = np.ascontiguousarray(rank_freqs, dtype=np.uint32)
    dl, dr, dc = link_model(G)
    cost = np.zeros(G, dtype=np.float64)
    ba = np.ascontiguousarray(placement.block_access_from, dtype=np.uint8)
    check(_lib.lib().ugc_placement_cost(
        G, len(rank_ids), _ptr(rank_ids), _ptr(freqs), _ptr(placement.nid_to_block), _ptr(ba),
        placement.num_block, dl if t_local is None else t_local,
        dr if t_remote is None else t_remote, dc if t_cpu is None else t_cpu, _ptr(cost)))
    return cost


class Cache:
    """One process' view of the multi-GPU embedding cache (a ``ugc_ctx``)."""

    def __init__(self, num_device, num_total_item, row_bytes, cache_percentage, max_batch=1 << 20,
                 empty_feat=0, table_kind=TABLE_AUTO, gather_ctas_per_sm=0, host_ctas=0,
                 remote_ctas=0, register_host=True, gather_vec_bytes=16):
        L = _lib.lib()
        cfg = _lib.Config()
        check(L.ugc_config_default(C.byref(cfg)))
        cfg.num_device = num_device
        cfg.num_total_item = num_total_item
        cfg.row_bytes = row_bytes
        cfg.cache_percentage = cache_percentage
        cfg.max_batch = max_batch
        cfg.empty_feat = empty_feat
        cfg.table_kind = table_kind
        cfg.gather_ctas_per_sm = gather_ctas_per_sm
        cfg.host_ctas = host_ctas
        cfg.remote_ctas = remote_ctas
        cfg.gather_vec_bytes = gather_vec_bytes
        cfg.register_host = 1 if register_host else 0
        self.cfg = cfg
        self._h = C.c_void_p()
        check(L.ugc_create(C.byref(cfg), C.byref(self._h)))
        self._keep = []  # host arrays the library reads in place

    # -- lifetime -----------------------------------------------------------------
    def close(self):
        if self._h:
            _lib.lib().ugc_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- placement ----------------------------------------------------------------
    def set_placement(self, p):
        check(_lib.lib().ugc_set_placement(self._h, _ptr(p.nid_to_block), _ptr(p.block_placement),
                                           _ptr(p.block_access_from), _ptr(p.block_density),
                                           p.num_block))

    def classify_keys(self, replica_id, want_keys=False):
        G = self.cfg.num_device
        counts = np.zeros(G + 1, dtype=np.uint64)
        keys = np.zeros(self.cfg.num_total_item, dtype=np.uint32) if want_keys else None
        check(_lib.lib().ugc_classify_keys(self._h, replica_id, _ptr(counts),
                                           _ptr(keys) if want_keys else None))
        if not want_keys:
            return counts
        out, pos = [], 0
        for s in range(G):
            out.append(keys[pos:pos + int(counts[s])].copy())
            pos += int(counts[s])
        return counts, out

    # -- build ----------------------------------------------------------------------
    def build(self, replica_id, device_id, host_table_ptr, stream=0):
        """host_table_ptr: integer address of the host table (kept alive by the caller)."""
        check(_lib.lib().ugc_build(self._h, replica_id, device_id, C.c_void_p(host_table_ptr),
                                   C.c_void_p(stream)))

    def export(self, replica_id):
        h = _lib.PeerHandle()
        check(_lib.lib().ugc_export(self._h, replica_id, C.byref(h)))
        return h

    def import_peer(self, replica_id, handle):
        check(_lib.lib().ugc_import_peer(self._h, replica_id, C.byref(handle)))

    def connect_local(self):
        check(_lib.lib().ugc_connect_local(self._h))

    def attach_peers(self, replica_id, stream=0):
        check(_lib.lib().ugc_attach_peers(self._h, replica_id, C.c_void_p(stream)))

    # -- lookup ---------------------------------------------------------------------
    def lookup_ptr(self, replica_id, keys_ptr, key_bytes, n, out_ptr, stream=0):
        fn = _lib.lib().ugc_lookup_i64 if key_bytes == 8 else _lib.lib().ugc_lookup_u32
        check(fn(self._h, replica_id, C.c_void_p(keys_ptr), n, C.c_void_p(out_ptr),
                 C.c_void_p(stream)))

    def lookup(self, replica_id, keys, out=None, stream=None):
        """keys: CUDA tensor (int64 / int32 / uint32); returns a uint8 [n, row_bytes] tensor
        unless ``out`` (any dtype, n*row_bytes bytes) is given."""
        import torch
        n = keys.numel()
        if keys.dtype == torch.int64:
            kb = 8
        elif keys.dtype in (torch.int32, torch.uint32):
            kb = 4
        else:
            raise TypeError("keys must be int64, int32 or uint32")
        if out is None:
            out = torch.empty((n, self.cfg.row_bytes), dtype=torch.uint8, device=keys.device)
        s = torch.cuda.current_stream(keys.device).cuda_stream if stream is None else stream
        self.lookup_ptr(replica_id, keys.data_ptr(), kb, n, out.data_ptr(), s)
        return out

    def lookup_unique(self, replica_id, keys, stream=None):
        """Deduplicated lookup on the GPU.  keys: CUDA tensor (int64 / int32).  Returns
        ``(rows, unique_keys, inverse, n_unique)``: uint8 ``rows[n, row_bytes]`` of which the
        first ``n_unique`` are filled, ``unique_keys[n]`` likewise, int32 ``inverse[n]`` and a
        one-element int32 tensor ``n_unique`` -- all on the device, nothing synchronises."""
        import torch
        keys = keys.reshape(-1)
        n = keys.numel()
        kb = 8 if keys.dtype == torch.int64 else 4
        dev = keys.device
        rows = torch.empty((n, self.cfg.row_bytes), dtype=torch.uint8, device=dev)
        uniq = torch.empty_like(keys)
        inverse = torch.empty(n, dtype=torch.int32, device=dev)
        n_unique = torch.zeros(1, dtype=torch.int32, device=dev)
        s = torch.cuda.current_stream(dev).cuda_stream if stream is None else stream
        check(_lib.lib().ugc_lookup_unique(self._h, replica_id, C.c_void_p(keys.data_ptr()), kb, n,
                                           C.c_void_p(rows.data_ptr()), C.c_void_p(uniq.data_ptr()),
                                           C.c_void_p(inverse.data_ptr()), C.c_void_p(n_unique.data_ptr()),
                                           C.c_void_p(s)))
        return rows, uniq, inverse, n_unique

    def lookup_pool(self, replica_id, keys, offsets=None, bag_size=0, elem="f32", mode="sum", out=None,
                    stream=None):
        """Pooled lookup (embedding bag): ``out[b] = sum / mean of the rows of bag b`` as fp32,
        added in key order.  keys: CUDA tensor (int64 / int32); offsets: CUDA int64 tensor of
        ``n_bags + 1`` positions, or None with ``bag_size`` keys per bag.  Returns the
        ``[n_bags, dim]`` fp32 tensor."""
        import torch
        keys = keys.reshape(-1)
        n = keys.numel()
        kb = 8 if keys.dtype == torch.int64 else 4
        dev = keys.device
        if offsets is not None:
            if offsets.dtype != torch.int64 or not offsets.is_cuda:
                raise ValueError("offsets must be a CUDA int64 tensor")
            offsets = offsets.contiguous()
            n_bags = offsets.numel() - 1
        else:
            if bag_size <= 0:
                raise ValueError("give offsets or a bag size")
            n_bags = n // bag_size
        elem_type = {"f32": 0, "f16": 1}[elem]
        dim = self.cfg.row_bytes // (2 if elem_type else 4)
        if out is None:
            out = torch.empty((max(n_bags, 0), dim), dtype=torch.float32, device=dev)
        s = torch.cuda.current_stream(dev).cuda_stream if stream is None else stream
        check(_lib.lib().ugc_lookup_pool(self._h, replica_id, C.c_void_p(keys.data_ptr()), kb, n,
                                         C.c_void_p(offsets.data_ptr() if offsets is not None else None),
                                         max(n_bags, 0), bag_size, elem_type, {"sum": 0, "mean": 1}[mode],
                                         C.c_void_p(out.data_ptr()), C.c_void_p(s)))
        return out

    def lookup_pool_ptr(self, replica_id, keys_ptr, key_bytes, n_keys, offsets_ptr, n_bags, bag_size,
                        elem_type, mode, out_ptr, stream=0):
        """ugc_lookup_pool on raw device pointers (elem_type 0 = fp32, 1 = fp16; mode 0 = sum, 1 = mean)."""
        check(_lib.lib().ugc_lookup_pool(self._h, replica_id, C.c_void_p(keys_ptr), key_bytes, n_keys,
                                         C.c_void_p(offsets_ptr), n_bags, bag_size, elem_type, mode,
                                         C.c_void_p(out_ptr), C.c_void_p(stream)))

    def reserve_batch(self, replica_id, max_batch):
        check(_lib.lib().ugc_reserve_batch(self._h, replica_id, max_batch))

    def lookup_host(self, replica_id, keys_np, out_np, stream=0):
        keys_np = np.ascontiguousarray(keys_np)
        kb = keys_np.dtype.itemsize
        check(_lib.lib().ugc_lookup_host(self._h, replica_id, _ptr(keys_np), kb, len(keys_np),
                                         _ptr(out_np), C.c_void_p(stream)))
        return out_np

    def lookup_host_ptr(self, replica_id, keys_ptr, key_bytes, n, out_ptr, stream=0):
        check(_lib.lib().ugc_lookup_host(self._h, replica_id, C.c_void_p(keys_ptr), key_bytes, n,
                                         C.c_void_p(out_ptr), C.c_void_p(stream)))

    # -- refresh ----------------------------------------------------------------------
    def refresh_set_placement(self, p):
        check(_lib.lib().ugc_refresh_set_placement(self._h, _ptr(p.nid_to_block),
                                                   _ptr(p.block_placement),
                                                   _ptr(p.block_access_from),
                                                   _ptr(p.block_density), p.num_block))

    def refresh_evict(self, replica_id, stream=0):
        check(_lib.lib().ugc_refresh_evict(self._h, replica_id, C.c_void_p(stream)))

    def refresh_fill(self, replica_id, stream=0):
        check(_lib.lib().ugc_refresh_fill(self._h, replica_id, C.c_void_p(stream)))

    def refresh_attach(self, replica_id, stream=0):
        check(_lib.lib().ugc_refresh_attach(self._h, replica_id, C.c_void_p(stream)))

    def refresh_commit(self):
        check(_lib.lib().ugc_refresh_commit(self._h))

    def refresh_all_local(self, p, replicas, stream=0):
        """Whole refresh for replicas that all live in this process (no barriers needed:
        the phases run replica after replica)."""
        self.refresh_set_placement(p)
        for r in replicas:
            self.refresh_evict(r, stream)
        for r in replicas:
            self.refresh_fill(r, stream)
        for r in replicas:
            self.refresh_attach(r, stream)
        self.refresh_commit()

    # -- hotness ---------------------------------------------------------------------------
    def record(self, replica_id, keys, stream=None):
        """Count the accesses of a CUDA key tensor (int64 / int32) on the device."""
        import torch
        kb = 8 if keys.dtype == torch.int64 else 4
        s = torch.cuda.current_stream(keys.device).cuda_stream if stream is None else stream
        check(_lib.lib().ugc_record(self._h, replica_id, C.c_void_p(keys.data_ptr()), kb,
                                    keys.numel(), C.c_void_p(s)))

    def hotness_read(self, replica_id, reset=False, stream=0):
        counts = np.empty(self.cfg.num_total_item, dtype=np.uint32)
        check(_lib.lib().ugc_hotness_read(self._h, replica_id, _ptr(counts), 1 if reset else 0,
                                          C.c_void_p(stream)))
        return counts

    @staticmethod
    def rank_hotness(counts):
        """(rank_ids, rank_freqs) for the placement solvers: ids by descending count, ties by id."""
        order = np.argsort(-counts.astype(np.int64), kind="stable").astype(np.uint32)
        return order, counts[order]

    # -- introspection ------------------------------------------------------------------
    def stats(self, replica_id):
        s = _lib.Stats()
        check(_lib.lib().ugc_stats(self._h, replica_id, C.byref(s)))
        out = {name: getattr(s, name) for name, _ in s._fields_}
        out["pool_rows"] = [int(x) for x in s.pool_rows]
        return out

    def launches(self, replica_id):
        """Kernels launched by this replica's lookups so far."""
        return int(self.stats(replica_id)["kernel_launches"])

    def get_tuning(self, replica_id):
        t = _lib.Tuning()
        check(_lib.lib().ugc_get_tuning(self._h, replica_id, C.byref(t)))
        return {name: getattr(t, name) for name, _ in t._fields_ if name != "struct_size"}

    def tune(self, replica_id, **kw):
        """Change launch-shape fields of ``ugc_tuning`` by name; others keep their value."""
        t = _lib.Tuning()
        check(_lib.lib().ugc_get_tuning(self._h, replica_id, C.byref(t)))
        for k, v in kw.items():
            if not hasattr(t, k):
                raise KeyError(k)
            setattr(t, k, v)
        check(_lib.lib().ugc_set_tuning(self._h, replica_id, C.byref(t)))

    def profile_begin(self, replica_id, max_lookups):
        check(_lib.lib().ugc_profile_begin(self._h, replica_id, max_lookups))

    def profile_end(self, replica_id):
        """(lookup_group ms, gather ms, lookups) summed over the profiled lookups."""
        a, b, n = C.c_double(), C.c_double(), C.c_uint64()
        check(_lib.lib().ugc_profile_end(self._h, replica_id, C.byref(a), C.byref(b), C.byref(n)))
        return a.value, b.value, n.value

    def table_words(self, replica_id, keys_u32, stream=None):
        import torch
        words = torch.empty(keys_u32.numel(), dtype=torch.int32, device=keys_u32.device)
        s = torch.cuda.current_stream(keys_u32.device).cuda_stream if stream is None else stream
        check(_lib.lib().ugc_table_words(self._h, replica_id, C.c_void_p(keys_u32.data_ptr()),
                                         keys_u32.numel(), C.c_void_p(words.data_ptr()),
                                         C.c_void_p(s)))
        return words


def gen_table(dst_ptr, seed, row_begin, n_rows, dim, elem_bytes, stream=0):
    check(_lib.lib().ugc_gen_table(C.c_void_p(dst_ptr), seed, row_begin, n_rows, dim, elem_bytes,
                                   C.c_void_p(stream)))


def host_register(host_ptr, nbytes):
    """Pins and maps caller-owned host memory; returns the device-side address."""
    d = C.c_void_p()
    check(_lib.lib().ugc_host_register(C.c_void_p(host_ptr), nbytes, C.byref(d)))
    return d.value


def host_unregister(host_ptr, nbytes=1):
    check(_lib.lib().ugc_host_unregister_sized(C.c_void_p(host_ptr), nbytes))


def host_alloc(nbytes):
    """Pinned GPU-mapped host memory; returns (host address, device-side address)."""
    h, d = C.c_void_p(), C.c_void_p()
    check(_lib.lib().ugc_host_alloc(nbytes, C.byref(h), C.byref(d)))
    return h.value, d.value


def host_free(host_ptr):
    check(_lib.lib().ugc_host_free(C.c_void_p(host_ptr)))


def host_is_large_page(host_ptr):
    return bool(_lib.lib().ugc_host_is_large_page(C.c_void_p(host_ptr)))
