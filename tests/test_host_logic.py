"""CPU-only checks of the shipped library: it loads without a GPU, exports every symbol
the headers declare, its host-side logic (placement heuristics, key classification,
validation) agrees with the oracle, and device entry points fail with a status (never a
crash, never a silent CPU fallback) when no GPU is present."""
import ctypes as C
import glob
import os
import re

import numpy as np
import pytest

from oracle import oracle as orc
from tests.conftest import ROOT, oracle_solver
from tests.helpers import case_workload, digest


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        names |= set(re.findall(r"\b((?:ugc|coll_cache)_[a-z0-9_]+)\s*\(", text))
    return sorted(n for n in names if not n.endswith("_fn"))


def test_library_exports_every_declared_symbol(built_lib):
    lib = C.CDLL(built_lib)
    syms = declared_symbols()
    assert len(syms) >= 20
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, missing


def test_binding_covers_header(built_lib):
    from ugache_b200 import _lib
    ugc = [s for s in declared_symbols() if s.startswith("ugc_")]
    assert sorted(_lib.SIGNATURES) == ugc


def test_placement_solvers_match_oracle(built_lib, golden_cases):
    from ugache_b200 import runtime as rt
    for case in golden_cases:
        w_prod = case_workload(case)                 # product solver (C++ in the library)
        w_orc = case_workload(case, oracle_solver)   # oracle solver
        for f in ("nid_to_block", "block_placement", "block_access_from", "block_density"):
            assert np.array_equal(getattr(w_prod.placement, f), getattr(w_orc.placement, f)), \
                (case["name"], f)
        assert digest(w_prod.placement.nid_to_block) + digest(w_prod.placement.block_access_from) \
            == case["placement"]
    # a few more shapes, all three policies, G = 1..8
    rng = np.random.default_rng(0)
    for G in (1, 2, 3, 5, 8):
        N = 3000 + 17 * G
        ids = rng.permutation(N).astype(np.uint32)
        freqs = np.sort(rng.zipf(1.3, N).astype(np.uint32))[::-1].copy()
        for pol in ("intuitive", "rep", "clique_part"):
            for pct in (0.0, 1.0, 7.5, 40.0, 100.0):
                a = rt.solve_placement(pol, G, ids, freqs, pct)
                b = oracle_solver(pol, G, ids, freqs, pct)
                assert np.array_equal(a.nid_to_block, b.nid_to_block), (G, pol, pct)
                assert np.array_equal(a.block_access_from, b.block_access_from)
                assert np.array_equal(a.block_placement, b.block_placement)
                assert np.allclose(a.block_density, b.block_density)


def test_classification_matches_oracle(built_lib, golden_cases):
    from ugache_b200 import runtime as rt
    for case in golden_cases:
        w = case_workload(case)
        cache = rt.Cache(case["G"], case["N"], w.row_bytes, case["pct"], max_batch=1 << 14)
        cache.set_placement(w.placement)
        for r in range(case["G"]):
            counts, lists = cache.classify_keys(r, want_keys=True)
            words, cnt, slot_of = orc.model_build(w.placement, r, w.capacity)
            assert [int(x) for x in counts] == case["ranks"][str(r)]["per_src"]
            for s in range(case["G"]):
                want = np.nonzero((words != 0xFFFFFFFF) & ((words >> 28) == s))[0]
                assert np.array_equal(lists[s], want.astype(np.uint32))
                if s == r:  # slot = position in the ascending list
                    assert np.array_equal(slot_of[r][lists[s]], np.arange(len(lists[s])))
        cache.close()


def test_config_and_placement_validation(built_lib):
    from ugache_b200 import _lib, runtime as rt
    with pytest.raises(_lib.UgcError):
        rt.Cache(9, 1000, 512, 0.1)
    with pytest.raises(_lib.UgcError):
        rt.Cache(1, 1000, 510, 0.1)           # row size not a multiple of 4
    with pytest.raises(_lib.UgcError):
        rt.Cache(1, 1000, 512, 1.5)           # fraction, not percent
    with pytest.raises(_lib.UgcError):
        rt.Cache(1, 1 << 31, 512, 0.1)        # key space too large for 31-bit table keys
    cache = rt.Cache(2, 1000, 512, 0.1)
    ids = np.arange(1000, dtype=np.uint32)
    good = rt.solve_placement("rep", 2, ids, None, 10.0)
    cache.set_placement(good)
    bad = rt.PlacementArrays(good.nid_to_block, good.block_placement,
                             good.block_access_from.copy(), good.block_density)
    bad.block_access_from[0, 0] = 1           # GPU 0 stores block 0 but reads it from GPU 1
    with pytest.raises(_lib.UgcError):
        cache.set_placement(bad)
    bad2 = rt.PlacementArrays(good.nid_to_block.copy(), good.block_placement,
                              good.block_access_from, good.block_density)
    bad2.nid_to_block[5] = 99                 # block id out of range
    with pytest.raises(_lib.UgcError):
        cache.set_placement(bad2)
    with pytest.raises(_lib.UgcError):        # lookup before build
        cache.lookup_ptr(0, 1, 8, 1, 1)
    cache.close()


def test_device_entry_points_fail_loudly_without_gpu(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from ugache_b200 import _lib, runtime as rt
    cache = rt.Cache(1, 1000, 512, 0.1)
    cache.set_placement(rt.solve_placement("rep", 1, np.arange(1000, dtype=np.uint32), None, 10.0))
    table = np.zeros((1000, 128), dtype=np.float32)
    with pytest.raises(_lib.UgcError) as e:
        cache.build(0, 0, table.ctypes.data)
    assert e.value.status == 2               # UGC_ERR_CUDA: no silent fallback
    cache.close()


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    from ugache_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.lib()


def test_workload_generators_match_oracle():
    from ugache_b200 import workload as wl
    for dt in (np.float32, np.float16):
        a = wl.table(21, 300, 24, dt, row_begin=5)
        b = orc.gen_rows(21, 5, 300, 24, dt)
        assert a.tobytes() == b.tobytes()
    u = np.random.default_rng(4).random(50000)
    for N, alpha in ((10 ** 8, 1.2), (4 * 10 ** 8, 1.05), (10 ** 6, 1.0), (10 ** 6, 0.8), (10 ** 6, 1.4)):
        r = wl.zipf_ranks(u, N, alpha)
        assert np.array_equal(r, orc.zipf_ranks(u, N, alpha))
        A, B = wl.bijection(N)
        assert np.array_equal(wl.rank_to_id(r, N), orc.rank_to_id(r, N, A, B))
        ids = wl.rank_to_id(np.arange(1000), N)
        assert len(np.unique(ids)) == 1000


@pytest.mark.parametrize("G,alpha,pct", [(1, 1.2, 10.0), (2, 1.2, 10.0), (4, 1.2, 10.0), (8, 1.2, 10.0),
                                         (8, 1.05, 5.0), (4, 1.01, 2.0), (2, 1.5, 20.0), (3, 1.1, 30.0)])
def test_split_search_is_never_costlier_than_the_heuristics(built_lib, G, alpha, pct):
    """The split-search policy (the stand-in for the reference's MILP on a switch-connected
    box) yields a placement the runtime accepts, within the cache capacity, whose modelled cost
    is at most that of every heuristic policy, under the nominal link model and under the one
    with the measured host-row rate."""
    from ugache_b200 import runtime as rt, workload as wl
    N = 400_000
    ids, freqs = wl.analytic_hotness(N, alpha)
    cache = rt.Cache(G, N, 512, pct / 100.0)
    for row_bytes in (None, 512, 128):
        tl, tr, tc = rt.link_model(G, row_bytes)
        costs = {}
        for pol in ("rep", "clique_part", "intuitive", "split_search"):
            p = rt.solve_placement(pol, G, ids, freqs, pct, tl, tr, tc)
            costs[pol] = float(rt.placement_cost(p, ids, freqs, tl, tr, tc).max())
            if pol == "split_search":
                cache.set_placement(p)                      # validated by the runtime
                stored = (p.block_placement[p.nid_to_block][:, None] >> np.arange(G)) & 1
                assert stored.sum(axis=0).max() <= int(N * (pct / 100.0 + 0.001))
                # hotter ids are never placed worse than colder ones: replicated, then
                # partitioned, then host, along the hotness order
                kind = np.where(p.block_placement[p.nid_to_block[ids]] == (1 << G) - 1, 0,
                                np.where(p.block_placement[p.nid_to_block[ids]] != 0, 1, 2))
                assert (np.diff(kind) >= 0).all()
        best_other = min(v for k, v in costs.items() if k != "split_search")
        assert costs["split_search"] <= best_other * (1 + 1e-6), (row_bytes, costs)
    cache.close()


def test_placement_cost_rejects_bad_arrays(built_lib):
    from ugache_b200 import _lib, runtime as rt
    ids = np.arange(1000, dtype=np.uint32)
    freqs = np.arange(1000, 0, -1).astype(np.uint32)
    p = rt.solve_placement("rep", 2, ids, None, 10.0)
    c = rt.placement_cost(p, ids, freqs)
    assert c.shape == (2,) and c[0] == c[1] and c[0] > 0
    bad = rt.PlacementArrays(p.nid_to_block.copy(), p.block_placement, p.block_access_from,
                             p.block_density)
    bad.nid_to_block[3] = 77
    with pytest.raises(_lib.UgcError):
        rt.placement_cost(bad, ids, freqs)
    with pytest.raises(_lib.UgcError):
        rt.solve_placement("split_search", 2, ids, None, 10.0)   # needs frequencies


def test_lookup_unique_helper_reassembles_the_batch(built_lib):
    """The dedup-aware adapter on CPU tensors with a stand-in lookup: the distinct keys are
    looked up once, in ascending order, and rows_unique[inverse] is the per-key result."""
    torch = pytest.importorskip("torch")
    from ugache_b200.collcache.torch import lookup_unique
    from ugache_b200 import workload as wl
    N, dim = 5000, 8
    table = torch.from_numpy(wl.table(3, N, dim))
    calls = []

    def fake_lookup(u):
        calls.append(u.clone())
        out = torch.zeros((u.numel() + 5, dim))       # a larger reusable buffer, as the real one
        out[:u.numel()] = table[u]
        return out

    for keys in (torch.from_numpy(wl.zipf_keys(9, 4000, N, 1.3)), torch.tensor([7, 7, 7], dtype=torch.int64),
                 torch.zeros(0, dtype=torch.int64)):
        rows, inverse = lookup_unique(keys, fake_lookup)
        u = calls[-1]
        assert rows.shape == (u.numel(), dim)
        assert torch.equal(u, torch.unique(keys)) and (u.numel() < 2 or bool((u[1:] > u[:-1]).all()))
        assert torch.equal(rows[inverse], table[keys])


def test_link_description_follows_the_number_of_gpus(built_lib):
    """The B200 link description: no peers with one GPU; the host share per GPU shrinks as more
    GPUs read the host side together; small rows are bound by the scattered-row rate; the CTA
    budgets of the far links follow bandwidth x latency."""
    from ugache_b200 import runtime as rt
    d1, d2, d8 = (rt.link_desc(g, 512) for g in (1, 2, 8))
    assert d1["bw_remote_gbs"] == 0 and d2["bw_remote_gbs"] == d8["bw_remote_gbs"] == 900
    assert d1["bw_host_gbs"] >= d2["bw_host_gbs"] >= d8["bw_host_gbs"] > 0
    assert d8["bw_host_gbs"] <= d8["host_total_gbs"] / 8 + 1e-9
    small = rt.link_desc(1, 128)
    assert abs(small["bw_host_gbs"] - small["host_rows_per_s"] * 128 / 1e9) < 1e-9   # row-rate bound
    assert rt.link_desc(1, 0)["bw_host_gbs"] == 64                                   # bandwidth only
    # Little's law: CTAs = 2 * ceil(bw * latency / 16 KiB in flight per CTA)
    import math
    assert d8["remote_ctas"] == 2 * math.ceil(900e3 * d8["lat_remote_us"] / 16384)
    assert d8["host_ctas"] == 2 * math.ceil(64e3 * d8["lat_host_us"] / 16384)
    assert d8["per_peer_ctas"] == d8["remote_ctas"] // 7
    assert d8["t_cpu"] > d1["t_cpu"] > d8["t_remote"] > d8["t_local"] == 1.0
    tl, tr, tc = rt.link_model(8, 512)
    assert (tl, tr, tc) == (d8["t_local"], d8["t_remote"], d8["t_cpu"])
    assert rt.link_model(8) == (1.0, 8000.0 / 900.0, 8000.0 / 64.0)                  # solver defaults


def test_ctypes_structs_follow_the_header(built_lib):
    """Field names and order of every struct in include/ugache_b200.h against the ctypes
    declarations, and their sizes against the loaded library (ugc_abi_sizes)."""
    import ctypes as C
    import os
    import re
    from tests.conftest import ROOT
    from ugache_b200 import _lib
    header = open(os.path.join(ROOT, "include", "ugache_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    pairs = (("ugc_config", _lib.Config), ("ugc_peer_handle", _lib.PeerHandle), ("ugc_stats_t", _lib.Stats),
             ("ugc_tuning", _lib.Tuning), ("ugc_link_desc_t", _lib.LinkDesc))
    for cname, cls in pairs:
        end = header.index("} %s;" % cname)
        body = header[header.rindex("typedef struct {", 0, end) + len("typedef struct {"):end]
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                names.append(re.sub(r"\[.*\]", "", part.strip().split()[-1].lstrip("*")))
        assert names == [f[0] for f in cls._fields_], cname
    sizes = (C.c_uint32 * 5)()
    assert _lib.lib().ugc_abi_sizes(C.byref(sizes)) == 0
    assert list(sizes) == [C.sizeof(cls) for _, cls in pairs]


def test_oracle_pool_is_a_sequential_fp32_sum():
    """The pooled-lookup restatement: per bag, rows added in key order in fp32 from +0; fp16 rows
    widened first; the mean divides once; ids outside the table add nothing; empty bags are zero."""
    from oracle import oracle as orc
    rng = np.random.default_rng(5)
    for dtype in (np.float32, np.float16):
        table = (rng.standard_normal((500, 12)) * 100).astype(dtype)
        keys = rng.integers(0, 500, 300)
        keys[5], keys[77] = -3, 500
        offsets = np.array([0, 0, 7, 7, 40, 41, 300])
        for mean in (False, True):
            got = orc.pool(table, keys, offsets=offsets, mean=mean)
            want = np.zeros((6, 12), np.float32)
            for b in range(6):
                acc = np.zeros(12, np.float32)
                for i in range(offsets[b], offsets[b + 1]):
                    if 0 <= keys[i] < 500:
                        acc = (acc + table[keys[i]].astype(np.float32)).astype(np.float32)
                n = offsets[b + 1] - offsets[b]
                want[b] = acc / np.float32(n) if (mean and n) else acc
            assert got.dtype == np.float32 and got.view(np.uint32).tobytes() == want.view(np.uint32).tobytes()
        fixed = orc.pool(table, keys, bag_size=7)
        assert fixed.shape == (300 // 7, 12)
        assert np.array_equal(fixed[3], orc.pool(table, keys[21:28], bag_size=7)[0])
