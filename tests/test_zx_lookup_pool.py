"""Pooled lookup (ugc_lookup_pool): lookup, row fetch and per-bag sum in one kernel, compared bit
for bit with the oracle's sequential fp32 restatement (oracle.pool).  The reference has no such
call; the rows a bag sums are the rows its lookup returns (coll_cache_lib/facade.cc:431-480)."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import case_workload

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _pool(cache, r, keys, dev, elem, tdt=None, **kw):
    with torch.cuda.device(dev):
        k = torch.from_numpy(np.ascontiguousarray(keys)).to(dev)
        if tdt is not None:
            k = k.to(tdt)
        if kw.get("offsets") is not None:
            kw["offsets"] = torch.from_numpy(np.asarray(kw["offsets"], dtype=np.int64)).to(dev)
        out = cache.lookup_pool(r, k, elem=elem, **kw)
        torch.cuda.synchronize(dev)
        return out.cpu().numpy()


CASES = [
    # name of a golden case (sources: local + peers + host), element type
    ("g2_intuitive", "f32"),
    ("g8_intuitive", "f32"),
]


@pytest.mark.parametrize("case_name,elem", CASES)
@pytest.mark.parametrize("key_dtype,piece", [("int64", 0), ("int32", 16), ("int64", 4)])
def test_pooled_lookup_matches_the_oracle(built_lib, golden_cases, case_name, elem, key_dtype, piece):
    from tests.test_gpu_parity import make_cache
    case = next(c for c in golden_cases if c["name"] == case_name)
    w = case_workload(case)
    assert w.dtype == np.float32
    cache = make_cache(w)
    ndev = torch.cuda.device_count()
    tdt = torch.int64 if key_dtype == "int64" else torch.int32
    rng = np.random.default_rng(7)
    for r in range(min(w.G, 3)):
        dev = torch.device("cuda", r % ndev)
        cache.tune(r, pool_vec_bytes=piece)       # 16- or 4-byte pieces per lane, or the launcher's choice
        keys = w.keys(rank=r)
        n = len(keys)
        before = cache.stats(r)
        # fixed bags of 1, 4 and 37 keys (the last one leaves keys over), sum and mean
        for bag, mode in ((1, "sum"), (4, "sum"), (37, "mean")):
            got = _pool(cache, r, keys, dev, elem, tdt, bag_size=bag, mode=mode)
            want = orc.pool(w.table, keys, bag_size=bag, mean=mode == "mean")
            assert got.shape == want.shape == (n // bag, w.dim)
            assert np.array_equal(_bits(got), _bits(want)), (case_name, r, bag, mode)
        # ragged bags with empty ones, one long bag (several passes of the lane group)
        cuts = np.sort(rng.integers(0, n, 300))
        cuts[100:110] = cuts[100]                      # empty bags
        offsets = np.concatenate([[0], cuts, [n]]).astype(np.int64)
        for mode in ("sum", "mean"):
            got = _pool(cache, r, keys, dev, elem, tdt, offsets=offsets, mode=mode)
            want = orc.pool(w.table, keys, offsets=offsets, mean=mode == "mean")
            assert np.array_equal(_bits(got), _bits(want)), (case_name, r, "ragged", mode)
        # many short ragged bags (a lane group walks through several bags per tile), empty ones among them
        cuts = np.sort(rng.integers(0, n, n // 3))
        small = np.concatenate([[0], cuts, [n]]).astype(np.int64)
        got = _pool(cache, r, keys, dev, elem, tdt, offsets=small, mode="mean")
        want = orc.pool(w.table, keys, offsets=small, mean=True)
        assert np.array_equal(_bits(got), _bits(want)), (case_name, r, "short ragged")
        st = cache.stats(r)
        assert st["lookups_pooled"] - before["lookups_pooled"] == 6
        rows = [a - b for a, b in zip(st["pool_rows"], before["pool_rows"])]
        assert sum(rows) == (n // 1) + (n // 4) * 4 + (n // 37) * 37 + 3 * n
        assert rows[0] > 0 and rows[2] > 0 and (w.G == 1 or rows[1] > 0)
        assert st["err_key_range"] == before["err_key_range"]
    cache.close()


@pytest.mark.parametrize("dim,dtype", [(64, "float16"), (100, "float32"), (256, "float32"), (8, "float16")])
def test_pooled_lookup_row_shapes(built_lib, dim, dtype):
    """fp16 rows (widened, summed in fp32), rows whose number of 16-byte pieces is no power of
    two, rows wider than one pass of a lane group (1 KiB), 16-byte rows; ids outside the key
    space add nothing and are counted."""
    from ugache_b200 import runtime as rt, workload as wl
    from tests.test_gpu_parity import pinned_table
    N, G = 30000, 2
    dt = np.dtype(dtype)
    table = wl.table(11, N, dim, dt)
    ids, freqs = wl.analytic_hotness(N, 1.1)
    cache = rt.Cache(G, N, dim * dt.itemsize, 0.1, max_batch=1 << 15)
    cache.set_placement(rt.solve_placement("intuitive", G, ids, freqs, 10.0))
    host = pinned_table(table)
    for r in range(G):
        cache.build(r, 0, host.data_ptr())
    cache.connect_local()
    for r in range(G):
        cache.attach_peers(r)
    dev = torch.device("cuda", 0)
    elem = "f16" if dt == np.float16 else "f32"
    keys = wl.zipf_keys(5, 20000, N, 1.1)
    keys[17], keys[4000], keys[19999] = -1, N, N + 12345
    for piece in (16, 4):
        cache.tune(1, pool_vec_bytes=piece)
        for bag, mode in ((8, "sum"), (50, "mean")):
            got = _pool(cache, 1, keys, dev, elem, bag_size=bag, mode=mode)
            want = orc.pool(table, keys, bag_size=bag, mean=mode == "mean")
            assert np.array_equal(_bits(got), _bits(want)), (dim, dtype, bag, mode, piece)
    assert cache.stats(1)["err_key_range"] == 12
    cache.tune(1, pool_vec_bytes=0)
    # the sum of bags of one key is the widened row itself
    got = _pool(cache, 1, keys[:1000], dev, elem, bag_size=1)
    ok = (keys[:1000] >= 0) & (keys[:1000] < N)
    assert np.array_equal(_bits(got[ok]), _bits(table[keys[:1000][ok]].astype(np.float32) + np.float32(0)))
    assert not got[~ok].any()
    cache.close()


def test_pooled_lookup_argument_errors(built_lib):
    from ugache_b200 import _lib, runtime as rt, workload as wl
    from tests.test_gpu_parity import pinned_table
    N, dim = 5000, 5                       # 20-byte rows: not a multiple of 16
    table = wl.table(3, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    cache = rt.Cache(1, N, dim * 4, 0.1, max_batch=1 << 12)
    cache.set_placement(rt.solve_placement("rep", 1, ids, freqs, 10.0))
    host = pinned_table(table)
    cache.build(0, 0, host.data_ptr())
    k = torch.arange(64, device="cuda")
    with pytest.raises(_lib.UgcError):
        cache.lookup_pool(0, k, bag_size=4)
    with pytest.raises(ValueError):
        cache.lookup_pool(0, k)
    cache.close()
