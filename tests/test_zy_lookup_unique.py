"""Dedup-aware lookup on the GPU: the distinct keys of a skewed batch are looked up once and the
batch is reassembled through the inverse index.  (Collected near the end on purpose: it is the
newest test of the suite.)"""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import case_workload

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_lookup_unique_on_the_gpu(built_lib, golden_cases):
    from tests.test_gpu_parity import make_cache
    from ugache_b200.collcache.torch import lookup_unique
    case = next(c for c in golden_cases if c["name"] == "g2_intuitive")
    w = case_workload(case)
    cache = make_cache(w)
    ndev = torch.cuda.device_count()
    for r in range(w.G):
        dev = torch.device("cuda", r % ndev)
        keys = w.keys(rank=r)
        with torch.cuda.device(dev):
            k = torch.from_numpy(keys).to(dev)
            rows, inverse = lookup_unique(k, lambda u: cache.lookup(r, u))
            torch.cuda.synchronize(dev)
            assert rows.shape[0] == len(np.unique(keys))
            got = rows[inverse].cpu().numpy()
        want = orc.gather(w.table, keys).view(np.uint8).reshape(len(keys), -1)
        assert np.array_equal(got, want), r
        assert cache.stats(r)["last_keys"] == len(np.unique(keys))
    cache.close()


@pytest.mark.parametrize("key_dtype", ["int64", "int32"])
def test_fused_unique_lookup(built_lib, golden_cases, key_dtype):
    """ugc_lookup_unique through the C ABI: distinct keys found on the GPU, each row extracted
    once, the batch reassembled by the inverse index; repeated calls (epochs of the stamps),
    out-of-range ids, a batch without duplicates and an empty batch."""
    from tests.test_gpu_parity import make_cache
    case = next(c for c in golden_cases if c["name"] == "g2_intuitive")
    w = case_workload(case)
    cache = make_cache(w)
    ndev = torch.cuda.device_count()
    tdt = torch.int64 if key_dtype == "int64" else torch.int32
    for r in range(w.G):
        dev = torch.device("cuda", r % ndev)
        with torch.cuda.device(dev):
            for it in range(3):
                keys = w.keys(rank=r, it=it)
                k = torch.from_numpy(keys).to(dev).to(tdt)
                rows, uniq, inverse, n_unique = cache.lookup_unique(r, k)
                torch.cuda.synchronize(dev)
                nu = int(n_unique.item())
                assert nu == len(np.unique(keys))
                u = uniq[:nu].cpu().numpy().astype(np.int64)
                assert np.array_equal(np.sort(u), np.unique(keys))
                inv = inverse.cpu().numpy()
                assert np.array_equal(u[inv], keys)
                got = rows[:nu][inverse.long()].cpu().numpy()
                want = orc.gather(w.table, keys).view(np.uint8).reshape(len(keys), -1)
                assert np.array_equal(got, want), (r, it)
                st = cache.stats(r)
                assert st["last_local"] + st["last_remote"] + st["last_host"] == nu
            # ids outside the key space: flagged in the inverse index, counted, rest exact
            keys = w.keys(rank=r, it=5)[:2000].copy()
            keys[7], keys[8] = w.N + 3, -5
            rows, uniq, inverse, n_unique = cache.lookup_unique(r, torch.from_numpy(keys).to(dev).to(tdt))
            torch.cuda.synchronize(dev)
            inv = inverse.cpu().numpy()
            good = np.ones(len(keys), dtype=bool)
            good[[7, 8]] = False
            assert (inv[~good] == -1).all() and (inv[good] >= 0).all()
            nu = int(n_unique.item())
            assert nu == len(np.unique(keys[good]))
            got = rows[:nu][inverse.long()[torch.from_numpy(good).to(dev)]].cpu().numpy()
            assert np.array_equal(got, orc.gather(w.table, keys[good]).view(np.uint8).reshape(int(good.sum()), -1))
            assert cache.stats(r)["err_key_range"] == 2
            # no duplicates at all, then nothing at all
            perm = np.random.default_rng(3).permutation(w.N)[:3000].astype(np.int64)
            rows, uniq, inverse, n_unique = cache.lookup_unique(r, torch.from_numpy(perm).to(dev).to(tdt))
            torch.cuda.synchronize(dev)
            assert int(n_unique.item()) == 3000
            assert np.array_equal(rows[inverse.long()].cpu().numpy(),
                                  orc.gather(w.table, perm).view(np.uint8).reshape(3000, -1))
            rows, uniq, inverse, n_unique = cache.lookup_unique(r, torch.zeros(0, dtype=tdt, device=dev))
            torch.cuda.synchronize(dev)
            assert int(n_unique.item()) == 0
    cache.close()


def test_stamp_epochs_wrap(built_lib):
    """More than 255 deduplicated lookups on one replica: the stamps are cleared when the epoch
    counter comes round and the results stay exact."""
    from ugache_b200 import runtime as rt, workload as wl
    N, dim = 5000, 8
    table = wl.table(71, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    cache = rt.Cache(1, N, dim * 4, 0.2, max_batch=4096)
    cache.set_placement(rt.solve_placement("rep", 1, ids, freqs, 20.0))
    host = torch.from_numpy(table).pin_memory()
    cache.build(0, 0, host.data_ptr())
    for it in range(300):
        keys = wl.zipf_keys(900 + it, 700, N, 1.2)
        rows, uniq, inverse, n_unique = cache.lookup_unique(0, torch.from_numpy(keys).cuda())
        if it % 37 == 0 or it > 250:
            torch.cuda.synchronize()
            nu = int(n_unique.item())
            assert nu == len(np.unique(keys)), it
            assert np.array_equal(rows[:nu][inverse.long()].cpu().numpy(),
                                  table[keys].view(np.uint8).reshape(len(keys), -1)), it
    cache.close()
