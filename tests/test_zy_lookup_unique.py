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
