"""Parity of the CUDA path (through the C ABI) against the CPU oracle, bit for bit.

Replicas are spread over the visible GPUs round-robin; on a one-GPU box all of them sit on
device 0, where a "peer" slice is simply another allocation on the same device: the
multi-replica logic (placement, tables, peer resolve, grouped gather) is exercised in
full, only the NVLink hop is missing.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from tests.conftest import oracle_solver
from tests.helpers import case_workload, digest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(autouse=True, params=["grouped", "grouped_static", "direct", "direct_early", "auto"])
def extract_mode(request, monkeypatch):
    """Every test of this module runs once per extraction mode (index lists + per-source CTA
    groups / one fused kernel / chosen per lookup from the previous lookup's counts)."""
    # the two main shapes run everywhere; the other two on the tests that exercise the gather
    # and the mode switch (keeps the suite short)
    wide = {"test_golden_cases_bit_exact", "test_ragged_batch_sizes", "test_auto_mode_follows_the_host_share",
            "test_auto_mode_stays_direct_when_peers_serve_more_rows_than_the_host",
            "test_duplicates_and_single_source_batches", "test_out_of_range_keys_are_counted_and_skipped",
            "test_unaligned_output_and_host_table", "test_refresh_keeps_results_identical",
            "test_host_list_in_address_order"}
    if request.param in ("auto", "grouped_static", "direct_early") and request.node.originalname not in wide:
        pytest.skip("covered by the grouped and direct runs")
    monkeypatch.setenv("UGC_EXTRACT_MODE", request.param)
    return request.param


def pinned_table(np_table):
    t = torch.from_numpy(np_table.view(np.uint8).reshape(np_table.shape[0], -1).copy()).pin_memory()
    return t


def make_cache(w, table_kind=0, max_batch=1 << 16, **kw):
    from ugache_b200 import runtime as rt
    ndev = torch.cuda.device_count()
    cache = rt.Cache(w.G, w.N, w.row_bytes, w.pct, max_batch=max_batch, table_kind=table_kind, **kw)
    cache.set_placement(w.placement)
    host = pinned_table(w.table)
    for r in range(w.G):
        cache.build(r, r % ndev, host.data_ptr())
    cache.connect_local()
    for r in range(w.G):
        cache.attach_peers(r)
    cache._host_keepalive = host
    return cache


def lookup_np(cache, r, keys_np, dtype=torch.int64):
    ndev = torch.cuda.device_count()
    dev = torch.device("cuda", r % ndev)
    with torch.cuda.device(dev):
        k = torch.from_numpy(np.ascontiguousarray(keys_np)).to(dev)
        if dtype != torch.int64:
            k = k.to(dtype)
        out = torch.full((len(keys_np), cache.cfg.row_bytes), 0xCD, dtype=torch.uint8, device=dev)
        cache.lookup(r, k, out=out)
        torch.cuda.synchronize(dev)
        return out.cpu().numpy()


@pytest.mark.parametrize("table_kind", [0, 1, 2])
def test_golden_cases_bit_exact(built_lib, golden_cases, table_kind):
    for case in golden_cases:
        w = case_workload(case)
        cache = make_cache(w, table_kind=table_kind)
        for r in range(w.G):
            keys = w.keys(rank=r)
            want = orc.gather(w.table, keys)
            got = lookup_np(cache, r, keys)
            assert got.tobytes() == want.tobytes(), (case["name"], r)
            assert digest(got) == case["ranks"][str(r)]["out"]
            st = cache.stats(r)
            assert st["err_key_range"] == 0 and st["err_table"] == 0
            # per-source split of the batch against the oracle's model
            words, _, _ = orc.model_build(w.placement, r, w.capacity)
            kw = words[keys]
            n_host = int((kw == 0xFFFFFFFF).sum())
            n_local = int(((kw != 0xFFFFFFFF) & ((kw >> 28) == r)).sum())
            assert (st["last_local"], st["last_remote"], st["last_host"]) == \
                (n_local, len(keys) - n_local - n_host, n_host)
            assert st["last_keys"] == len(keys)
        cache.close()


def test_table_words_match_oracle_model(built_lib, golden_cases):
    for case in golden_cases:
        w = case_workload(case)
        for kind in (1, 2):
            cache = make_cache(w, table_kind=kind)
            allk = torch.arange(w.N, dtype=torch.int32)
            for r in range(w.G):
                dev = torch.device("cuda", r % torch.cuda.device_count())
                got = cache.table_words(r, allk.to(dev))
                torch.cuda.synchronize(dev)
                words, _, _ = orc.model_build(w.placement, r, w.capacity)
                assert np.array_equal(got.cpu().numpy().view(np.uint32), words), (case["name"], r, kind)
                assert digest(got.cpu().numpy().view(np.uint32)) == case["ranks"][str(r)]["words"]
            cache.close()


def test_u32_keys_and_int64_agree(built_lib, golden_cases):
    case = golden_cases[2]
    w = case_workload(case)
    cache = make_cache(w)
    keys = w.keys(rank=1)
    a = lookup_np(cache, 1, keys)
    b = lookup_np(cache, 1, keys, dtype=torch.int32)
    assert a.tobytes() == b.tobytes() == orc.gather(w.table, keys).tobytes()
    cache.close()


@pytest.mark.parametrize("n", [0, 1, 2, 31, 32, 33, 255, 256, 257, 1023, 1024, 1025, 4097])
def test_ragged_batch_sizes(built_lib, golden_cases, n):
    case = golden_cases[4]   # 8 replicas
    w = case_workload(case)
    cache = make_cache(w)
    keys = w.keys(rank=3)[:n]
    got = lookup_np(cache, 3, keys)
    assert got.tobytes() == orc.gather(w.table, keys).tobytes()
    cache.close()


def test_duplicates_and_single_source_batches(built_lib, golden_cases):
    case = golden_cases[2]
    w = case_workload(case)
    cache = make_cache(w)
    words, _, _ = orc.model_build(w.placement, 0, w.capacity)
    local = np.nonzero((words != 0xFFFFFFFF) & ((words >> 28) == 0))[0]
    remote = np.nonzero((words != 0xFFFFFFFF) & ((words >> 28) == 1))[0]
    host = np.nonzero(words == 0xFFFFFFFF)[0]
    rng = np.random.default_rng(0)
    for name, pool in (("local", local), ("remote", remote), ("host", host)):
        keys = rng.choice(pool, size=3000).astype(np.int64)      # with duplicates
        got = lookup_np(cache, 0, keys)
        assert got.tobytes() == orc.gather(w.table, keys).tobytes(), name
    same = np.full(2000, int(local[0]), dtype=np.int64)          # one key repeated
    assert lookup_np(cache, 0, same).tobytes() == orc.gather(w.table, same).tobytes()
    cache.close()


def test_out_of_range_keys_are_counted_and_skipped(built_lib, golden_cases):
    case = golden_cases[1]
    w = case_workload(case)
    cache = make_cache(w)
    keys = w.keys(rank=0)[:1000].copy()
    keys[10] = w.N           # first id past the table
    keys[20] = -1
    keys[30] = 1 << 40
    got = lookup_np(cache, 0, keys)
    want = orc.gather(w.table, np.where((keys >= 0) & (keys < w.N), keys, 0))
    good = np.ones(1000, dtype=bool)
    good[[10, 20, 30]] = False
    assert got[good].tobytes() == want.view(np.uint8).reshape(1000, -1)[good].tobytes()
    assert (got[~good] == 0xCD).all()          # rows of bad keys are left untouched
    st = cache.stats(0)
    assert st["err_key_range"] == 3
    assert st["last_local"] + st["last_remote"] + st["last_host"] == 997
    cache.close()


def test_host_buffer_lookup(built_lib, golden_cases):
    case = golden_cases[2]
    w = case_workload(case)
    cache = make_cache(w)
    keys = w.keys(rank=0)
    out = np.zeros((len(keys), w.row_bytes), dtype=np.uint8)
    cache.lookup_host(0, keys, out)
    assert out.tobytes() == orc.gather(w.table, keys).tobytes()
    k32 = keys.astype(np.uint32)
    out2 = np.zeros_like(out)
    cache.lookup_host(0, k32, out2)
    assert out2.tobytes() == out.tobytes()
    cache.close()


def test_mock_host_table(built_lib):
    """empty_feat: host rows wrap to key mod 2^k, cached rows are filled from the wrapped row
    too (the reference's SAMGRAPH_EMPTY_FEAT)."""
    from ugache_b200 import runtime as rt, workload as wl
    N, dim, k = 30000, 32, 10
    small = wl.table(9, 1 << k, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    p = rt.solve_placement("rep", 1, ids, freqs, 10.0)
    cache = rt.Cache(1, N, dim * 4, 0.10, max_batch=1 << 14, empty_feat=k)
    cache.set_placement(p)
    host = pinned_table(small)
    cache.build(0, 0, host.data_ptr())
    keys = wl.zipf_keys(5, 5000, N, 1.2)
    got = lookup_np(cache, 0, keys)
    assert got.tobytes() == orc.gather(small, keys, empty_feat=k).tobytes()
    cache.close()


def test_gen_table_matches_oracle(built_lib):
    from ugache_b200 import runtime as rt
    for dt, eb in ((np.float32, 4), (np.float16, 2)):
        n_rows, dim, row0 = 1000, 64, 12345
        buf = torch.empty(n_rows * dim * eb, dtype=torch.uint8, device="cuda")
        rt.gen_table(buf.data_ptr(), 77, row0, n_rows, dim, eb, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert buf.cpu().numpy().tobytes() == orc.gen_rows(77, row0, n_rows, dim, dt).tobytes()
    # straight into pinned host memory (how the benchmark fills its table)
    host = torch.empty(256 * 128 * 4, dtype=torch.uint8).pin_memory()
    rt.gen_table(host.data_ptr(), 3, 0, 256, 128, 4, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert host.numpy().tobytes() == orc.gen_rows(3, 0, 256, 128).tobytes()


def test_refresh_keeps_results_identical(built_lib):
    """Lookups before, between the phases of, and after a refresh all return the table's
    rows; the per-replica stored set follows the new placement."""
    from ugache_b200 import runtime as rt, workload as wl
    N, dim, G = 40000, 32, 4
    table = wl.table(31, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    p_old = rt.solve_placement("intuitive", G, ids, freqs, 8.0)
    shifted = np.roll(ids, 1500)              # hotness drifts: a different hot set
    p_new = rt.solve_placement("intuitive", G, shifted, freqs, 8.0)
    for kind in (1, 2):
        cache = rt.Cache(G, N, dim * 4, 0.08, max_batch=1 << 14, table_kind=kind)
        cache.set_placement(p_old)
        host = pinned_table(table)
        ndev = torch.cuda.device_count()
        for r in range(G):
            cache.build(r, r % ndev, host.data_ptr())
        cache.connect_local()
        for r in range(G):
            cache.attach_peers(r)
        keys = [wl.zipf_keys(100 + r, 6000, N, 1.2) for r in range(G)]
        want = [orc.gather(table, k).tobytes() for k in keys]

        def check(tag):
            for r in range(G):
                assert lookup_np(cache, r, keys[r]).tobytes() == want[r], (tag, r, kind)

        check("before")
        cache.refresh_set_placement(p_new)
        for r in range(G):
            cache.refresh_evict(r)
        check("after evict")                  # evicted keys fall back to the host
        for r in range(G):
            cache.refresh_fill(r)
        check("after fill")
        for r in range(G):
            cache.refresh_attach(r)
        cache.refresh_commit()
        check("after refresh")
        o_new = orc.Placement(p_new.nid_to_block, p_new.block_placement, p_new.block_access_from,
                              p_new.block_density)
        allk = torch.arange(N, dtype=torch.int32)
        for r in range(G):
            dev = torch.device("cuda", r % ndev)
            got = cache.table_words(r, allk.to(dev)).cpu().numpy().view(np.uint32)
            words, cnt, _ = orc.model_build(o_new, r, int(N * 0.081))
            # same source per key as the model; slots differ after a refresh by design
            assert np.array_equal(got == 0xFFFFFFFF, words == 0xFFFFFFFF)
            live = got != 0xFFFFFFFF
            assert np.array_equal(got[live] >> 28, words[live] >> 28)
            st = cache.stats(r)
            assert st["err_table"] == 0
            assert st["num_local_rows"] == int(cnt[r])
            assert st["free_rows"] == st["capacity_rows"] - st["num_local_rows"]
            # every stored row sits in its own slot
            mine = got[live & ((got >> 28) == r)] & 0x0FFFFFFF
            assert len(np.unique(mine)) == len(mine)
        # a second refresh back to the old placement
        cache.refresh_all_local(p_old, list(range(G)))
        check("after second refresh")
        cache.close()


def test_refresh_repoints_keys_that_move_to_a_peer_in_place(built_lib):
    """A key that was stored here and is read from a peer under the new placement, the peer
    holding the row already, never falls back to the host during the refresh: its entry is
    re-pointed in the evict phase.  With the tuning field cleared it is removed there and
    attached later (the reference's order), and is served by the host in between."""
    from ugache_b200 import runtime as rt, workload as wl
    N, dim, G = 40000, 32, 2
    table = wl.table(41, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.05)
    p_old = rt.solve_placement("intuitive", G, ids, freqs, 20.0)
    p_new = rt.solve_placement("intuitive", G, np.roll(ids, 800), freqs, 20.0)
    src_old = np.asarray(p_old.block_access_from).reshape(G, -1)[0][p_old.nid_to_block]
    src_new = np.asarray(p_new.block_access_from).reshape(G, -1)[0][p_new.nid_to_block]
    held = (np.asarray(p_old.block_placement)[p_old.nid_to_block] >> 1) & 1
    moved = np.nonzero((src_old == 0) & (src_new == 1) & (held == 1))[0]
    assert len(moved) > 100                  # rows leaving the replicated set
    keys = np.random.default_rng(3).choice(moved, 4000).astype(np.int64)
    want = orc.gather(table, keys).tobytes()
    for kind in (1, 2):
        for early in (1, 0):
            cache = rt.Cache(G, N, dim * 4, 0.2, max_batch=1 << 14, table_kind=kind)
            cache.set_placement(p_old)
            host = pinned_table(table)
            for r in range(G):
                cache.build(r, 0, host.data_ptr())
            cache.connect_local()
            for r in range(G):
                cache.attach_peers(r)
                cache.tune(r, refresh_early_repoint=early)
            assert lookup_np(cache, 0, keys).tobytes() == want
            assert cache.stats(0)["last_local"] == len(keys)
            cache.refresh_set_placement(p_new)
            for r in range(G):
                cache.refresh_evict(r)
            assert lookup_np(cache, 0, keys).tobytes() == want
            st = cache.stats(0)
            if early:
                assert (st["last_remote"], st["last_host"]) == (len(keys), 0), (kind, st)
            else:
                assert (st["last_remote"], st["last_host"]) == (0, len(keys)), (kind, st)
            for r in range(G):
                cache.refresh_fill(r)
            for r in range(G):
                cache.refresh_attach(r)
            cache.refresh_commit()
            assert lookup_np(cache, 0, keys).tobytes() == want
            st = cache.stats(0)
            assert (st["last_remote"], st["last_host"], st["err_table"]) == (len(keys), 0, 0)
            # every key has the source the new placement names
            allk = torch.arange(N, dtype=torch.int32, device="cuda")
            got = cache.table_words(0, allk).cpu().numpy().view(np.uint32)
            live = got != 0xFFFFFFFF
            assert np.array_equal(live, src_new < G)
            assert np.array_equal(got[live] >> 28, src_new[live].astype(np.uint32))
            cache.close()


def test_gnn_shaped_batches(built_lib):
    """Deduplicated, variable-size node-id batches from the sampled R-MAT graph, cache ordered
    by degree (the GNN configuration at small scale)."""
    from ugache_b200 import runtime as rt, workload as wl, workload_gnn as wg
    N, dim, G = 50000, 128, 4
    g = wg.GnnWorkload(N, 15, 9)
    ids, freqs = g.hotness()
    table = wl.table(13, N, dim)
    cache = rt.Cache(G, N, dim * 4, 0.05, max_batch=1 << 12)
    cache.set_placement(rt.solve_placement("intuitive", G, ids, freqs, 5.0))
    host = pinned_table(table)
    ndev = torch.cuda.device_count()
    for r in range(G):
        cache.build(r, r % ndev, host.data_ptr())
    cache.connect_local()
    for r in range(G):
        cache.attach_peers(r)
    for r in range(G):
        for it in range(2):
            keys = g.batch(r, it, num_seeds=200).numpy()
            assert len(np.unique(keys)) == len(keys)
            cache.reserve_batch(r, len(keys))
            got = lookup_np(cache, r, keys)
            assert got.tobytes() == orc.gather(table, keys).tobytes()
    cache.close()


def test_device_hotness_recording_drives_a_refresh(built_lib):
    """Access counts recorded on the GPU equal a host bincount; ranking them and refreshing
    moves the cache to the recorded hot set, with lookups exact before and after."""
    from ugache_b200 import runtime as rt, workload as wl
    N, dim = 30000, 32
    table = wl.table(3, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    cache = rt.Cache(1, N, dim * 4, 0.10, max_batch=1 << 14)
    cache.set_placement(rt.solve_placement("rep", 1, ids, freqs, 10.0))
    host = pinned_table(table)
    cache.build(0, 0, host.data_ptr())
    rng = np.random.default_rng(5)
    perm = rng.permutation(N)                      # a different popularity order
    want = np.zeros(N, dtype=np.int64)
    for i in range(6):
        keys = perm[wl.zipf_ranks(rng.random(12000), N, 1.2)].astype(np.int64)
        k = torch.from_numpy(keys).cuda()
        cache.record(0, k if i % 2 else k.to(torch.int32))
        want += np.bincount(keys, minlength=N)
    got = cache.hotness_read(0, reset=True)
    assert np.array_equal(got.astype(np.int64), want)
    assert cache.hotness_read(0).sum() == 0        # reset took effect
    rank_ids, rank_freqs = rt.Cache.rank_hotness(got)
    keys = perm[wl.zipf_ranks(rng.random(8000), N, 1.2)].astype(np.int64)
    before = lookup_np(cache, 0, keys)
    host_before = cache.stats(0)["last_host"]
    cache.refresh_all_local(rt.solve_placement("rep", 1, rank_ids, rank_freqs, 10.0), [0])
    after = lookup_np(cache, 0, keys)
    assert before.tobytes() == after.tobytes() == orc.gather(table, keys).tobytes()
    assert cache.stats(0)["last_host"] < host_before / 2      # the recorded hot set is cached now
    cache.close()


def test_full_batch_size_against_regenerated_rows(built_lib):
    """The benchmark's batch size (212,992 keys, 512-byte rows) over a table too large to hold
    twice: the table is written by the GPU generator into library-owned pinned memory and the
    expected rows are regenerated key by key by the oracle's counter-based generator.  Also:
    a second lookup of the same keys gives the same bytes (idempotence) and rows past the
    batch stay untouched."""
    from ugache_b200 import runtime as rt, workload as wl
    N, dim, B = 8_000_000, 128, 8192 * 26
    seed = 1234
    hptr, dptr = rt.host_alloc(N * dim * 4)
    try:
        s = torch.cuda.current_stream().cuda_stream
        rt.gen_table(dptr, seed, 0, N, dim, 4, s)
        torch.cuda.synchronize()
        ids, freqs = wl.analytic_hotness(N, 1.2)
        for G, kind in ((1, 0), (4, 2)):
            ndev = torch.cuda.device_count()
            cache = rt.Cache(G, N, dim * 4, 0.10, max_batch=B, table_kind=kind, register_host=False)
            cache.set_placement(rt.solve_placement("intuitive", G, ids, freqs, 10.0))
            for r in range(G):
                cache.build(r, r % ndev, hptr)
            cache.connect_local()
            for r in range(G):
                cache.attach_peers(r)
            r = G - 1
            dev = torch.device("cuda", r % ndev)
            keys = wl.zipf_keys(77 + G, B, N, 1.2)
            want = orc.gen_rows_for_keys(seed, keys, dim).view(np.uint8).reshape(B, dim * 4)
            with torch.cuda.device(dev):
                k = torch.from_numpy(keys).to(dev)
                out = torch.full((B + 64, dim * 4), 0x5A, dtype=torch.uint8, device=dev)
                cache.lookup(r, k, out=out)
                torch.cuda.synchronize(dev)
                first = out.cpu().numpy()
                cache.lookup(r, k, out=out)
                torch.cuda.synchronize(dev)
                second = out.cpu().numpy()
            assert first[:B].tobytes() == want.tobytes()
            assert second.tobytes() == first.tobytes()
            assert (first[B:] == 0x5A).all()
            st = cache.stats(r)
            assert st["last_local"] + st["last_remote"] + st["last_host"] == B
            assert st["err_table"] == 0 and st["err_key_range"] == 0
            cache.close()
    finally:
        rt.host_free(hptr)


def test_probing_table_churn(built_lib):
    """Evict / re-insert cycles on the probing table (tombstones, slot reuse, chains that cross
    lines): after every refresh the word of every key equals the model's source, every stored
    row has its own slot, and lookups stay exact."""
    from ugache_b200 import runtime as rt, workload as wl
    N, dim = 20000, 8
    table = wl.table(8, N, dim)
    rng = np.random.default_rng(11)
    cache = rt.Cache(1, N, dim * 4, 0.30, max_batch=1 << 13, table_kind=2)
    order = rng.permutation(N).astype(np.uint32)
    cache.set_placement(rt.solve_placement("rep", 1, order, None, 30.0))
    host = pinned_table(table)
    cache.build(0, 0, host.data_ptr())
    allk = torch.arange(N, dtype=torch.int32, device="cuda")
    for round_ in range(8):
        order = np.roll(order, int(rng.integers(500, 5000)))
        p = rt.solve_placement("rep", 1, order, None, 30.0)
        cache.refresh_all_local(p, [0])
        words = cache.table_words(0, allk).cpu().numpy().view(np.uint32)
        stored = p.nid_to_block == 0
        assert np.array_equal(words != 0xFFFFFFFF, stored), round_
        slots = words[stored] & 0x0FFFFFFF
        assert len(np.unique(slots)) == stored.sum()
        keys = rng.integers(0, N, 5000).astype(np.int64)
        assert lookup_np(cache, 0, keys).tobytes() == orc.gather(table, keys).tobytes()
        st = cache.stats(0)
        assert st["err_table"] == 0 and st["free_rows"] == st["capacity_rows"] - stored.sum()
    cache.close()


@pytest.mark.parametrize("G,row_bytes_model", [(4, None), (2, 512), (8, 128)])
def test_split_search_placement_serves_exact_rows(built_lib, G, row_bytes_model):
    """Build and look up under the split-search policy: every reader gets exactly the host
    table's rows, and the per-source counts follow the placement."""
    from ugache_b200 import runtime as rt, workload as wl

    def solver(policy, G_, ids, freqs, pct):
        tl, tr, tc = rt.link_model(G_, row_bytes_model)
        return rt.solve_placement(policy, G_, ids, freqs, pct, tl, tr, tc)

    w = wl.Workload(N=60_000, dim=32, dtype="float32", G=G, pct=0.08, alpha=1.1, n_keys=20_000,
                    policy="split_search", seed=41, dedup=False, solver=solver)
    cache = make_cache(w)
    for r in range(G):
        keys = w.keys(rank=r)
        got = lookup_np(cache, r, keys)
        assert np.array_equal(got, orc.gather(w.table, keys).view(np.uint8).reshape(len(keys), -1)), r
        st = cache.stats(r)
        src = w.placement.block_access_from[r][w.placement.nid_to_block[keys]]
        assert st["last_local"] == int((src == r).sum())
        assert st["last_host"] == int((src == G).sum())
        assert st["last_remote"] == int(((src != r) & (src != G)).sum())
    cache.close()


@pytest.mark.parametrize("kind", [1, 2])
def test_lookups_stay_exact_while_a_refresh_runs(built_lib, kind):
    """Lookups issued from other threads, on their own streams, while a background thread takes
    the cache through whole refreshes back and forth: every batch must still be the host
    table's rows (evicted keys come from the host, reused slots are never read by an older
    lookup, new entries appear only with their rows)."""
    import threading
    from ugache_b200 import runtime as rt, workload as wl
    N, dim, G = 120_000, 32, 2
    table = wl.table(51, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.1)
    p_a = rt.solve_placement("intuitive", G, ids, freqs, 10.0)
    p_b = rt.solve_placement("intuitive", G, np.roll(ids, 9000), freqs, 10.0)
    cache = rt.Cache(G, N, dim * 4, 0.10, max_batch=1 << 15, table_kind=kind)
    cache.set_placement(p_a)
    host = pinned_table(table)
    ndev = torch.cuda.device_count()
    for r in range(G):
        cache.build(r, r % ndev, host.data_ptr())
    cache.connect_local()
    for r in range(G):
        cache.attach_peers(r)
    stop = threading.Event()
    failures, done = [], [0] * G

    def reader(r):
        dev = torch.device("cuda", r % ndev)
        try:
            with torch.cuda.device(dev):
                stream = torch.cuda.Stream(dev)
                out = torch.empty((20_000, dim * 4), dtype=torch.uint8, device=dev)
                it = 0
                while not stop.is_set() or it < 4:
                    keys = wl.zipf_keys(1000 * r + it, 20_000, N, 1.1)
                    with torch.cuda.stream(stream):
                        k = torch.from_numpy(keys).to(dev, non_blocking=False)
                        out.fill_(0xEE)
                        cache.lookup(r, k, out=out)
                        stream.synchronize()
                        got = out.cpu().numpy()
                    if got.tobytes() != orc.gather(table, keys).tobytes():
                        failures.append((r, it))
                        return
                    it += 1
                    done[r] = it
        except Exception as e:  # surfaces in the main thread's assert
            failures.append((r, repr(e)))

    threads = [threading.Thread(target=reader, args=(r,)) for r in range(G)]
    for t in threads:
        t.start()
    try:
        # the refresh runs on each device's default stream; the readers' streams do not
        # synchronise with it (torch creates non-blocking streams)
        for round_ in range(6):
            cache.refresh_all_local(p_b if round_ % 2 == 0 else p_a, list(range(G)))
    finally:
        stop.set()
        for t in threads:
            t.join(timeout=120)
    assert not failures, failures
    assert min(done) >= 4
    for r in range(G):
        assert cache.stats(r)["err_table"] == 0
    cache.close()


@pytest.mark.parametrize("out_off,table_off,vec", [(4, 0, 32), (16, 0, 32), (0, 4, 16), (8, 16, 32), (0, 0, 32)])
def test_unaligned_output_and_host_table(built_lib, out_off, table_off, vec):
    """`out` and the host table may start at any multiple of 4 bytes: the kernels then fall
    back to narrower vector loads instead of faulting on a misaligned address.  Checked for
    lookups (local and host rows) and for the build-time fill."""
    from ugache_b200 import runtime as rt, workload as wl
    N, dim = 30000, 32                        # 128-byte rows
    rb = dim * 4
    table = wl.table(77, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    raw = torch.empty(N * rb + 64, dtype=torch.uint8).pin_memory()
    raw[table_off:table_off + N * rb] = torch.from_numpy(table.view(np.uint8).reshape(-1))
    cache = rt.Cache(1, N, rb, 0.10, max_batch=1 << 14, gather_vec_bytes=vec)
    cache.set_placement(rt.solve_placement("rep", 1, ids, freqs, 10.0))
    cache.build(0, 0, raw.data_ptr() + table_off)
    keys = wl.zipf_keys(3, 9000, N, 1.1)
    k = torch.from_numpy(keys).cuda()
    buf = torch.full((len(keys) * rb + 64,), 0x77, dtype=torch.uint8, device="cuda")
    out = buf[out_off:out_off + len(keys) * rb]
    cache.lookup_ptr(0, k.data_ptr(), 8, len(keys), out.data_ptr(),
                     torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    got = buf.cpu().numpy()
    assert got[out_off:out_off + len(keys) * rb].tobytes() == orc.gather(table, keys).tobytes()
    assert (got[:out_off] == 0x77).all() and (got[out_off + len(keys) * rb:] == 0x77).all()
    st = cache.stats(0)
    assert st["err_table"] == 0 and st["last_host"] > 0 and st["last_local"] > 0
    cache.close()


def test_host_buffers_in_place_and_staged(built_lib, golden_cases):
    """ugc_lookup_host with pinned buffers the GPU has mapped (read and written in place by the
    kernel) and with the staging copies forced: same bytes either way, int64 and uint32 keys."""
    case = golden_cases[2]
    w = case_workload(case)
    cache = make_cache(w)
    keys = w.keys(rank=0)
    want = orc.gather(w.table, keys).tobytes()
    kpin = torch.from_numpy(keys).pin_memory()
    k32 = torch.from_numpy(keys.astype(np.int32)).pin_memory()
    for zc in (3, 2, 1, 0):
        cache.tune(0, host_zero_copy=zc)
        for kt, kb in ((kpin, 8), (k32, 4)):
            opin = torch.full((len(keys), w.row_bytes), 0x11, dtype=torch.uint8).pin_memory()
            cache.lookup_host_ptr(0, kt.data_ptr(), kb, len(keys), opin.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
            assert opin.numpy().tobytes() == want, (zc, kb)
    cache.close()


def test_auto_mode_follows_the_host_share(built_lib, extract_mode):
    """In auto mode the first lookup is grouped; later ones go direct once a finished lookup
    has shown few host rows, and back when there are many.  A direct lookup's counts
    reach the library with the start of the next lookup, so the switch back takes one lookup
    longer than the switch forth."""
    if extract_mode != "auto":
        pytest.skip("only meaningful in auto mode")
    from ugache_b200 import runtime as rt, workload as wl
    N, dim = 40000, 32
    table = wl.table(5, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    cache = rt.Cache(1, N, dim * 4, 0.25, max_batch=1 << 14)
    p = rt.solve_placement("rep", 1, ids, freqs, 25.0)
    cache.set_placement(p)
    host = pinned_table(table)
    cache.build(0, 0, host.data_ptr())
    cache.tune(0, direct_max_host_rows=1000)      # direct while a lookup took <= 1000 host rows
    cached = np.nonzero(np.asarray(p.block_access_from).reshape(1, -1)[0][p.nid_to_block] == 0)[0]
    missing = np.nonzero(np.asarray(p.block_access_from).reshape(1, -1)[0][p.nid_to_block] != 0)[0]
    rng = np.random.default_rng(1)
    hot = rng.choice(cached, 6000).astype(np.int64)
    cold = rng.choice(missing, 6000).astype(np.int64)
    for keys in (hot, hot, hot):
        assert lookup_np(cache, 0, keys).tobytes() == orc.gather(table, keys).tobytes()
    st = cache.stats(0)
    assert st["lookups"] == 3 and st["lookups_direct"] == 2 and st["kernel_launches"] == 4
    for keys in (cold, cold, cold):  # two more direct ones (the mirror still shows hot batches)
        got = lookup_np(cache, 0, keys)
        assert got.tobytes() == orc.gather(table, keys).tobytes()
        st = cache.stats(0)
        assert (st["last_local"], st["last_remote"], st["last_host"], st["last_keys"]) == (0, 0, 6000, 6000)
    assert st["lookups_direct"] == 4 and st["kernel_launches"] == 8
    assert lookup_np(cache, 0, hot).tobytes() == orc.gather(table, hot).tobytes()   # still grouped
    st = cache.stats(0)
    assert st["lookups_direct"] == 4 and st["kernel_launches"] == 10 and st["last_local"] == 6000
    cache.close()


def test_auto_mode_stays_direct_when_peers_serve_more_rows_than_the_host(built_lib, extract_mode):
    """Auto mode goes grouped only when the host rows of the last finished lookup exceed both the
    threshold and the peer rows."""
    if extract_mode != "auto":
        pytest.skip("only meaningful in auto mode")
    from ugache_b200 import runtime as rt, workload as wl
    N, dim, G = 40000, 32, 2
    table = wl.table(6, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    cache = rt.Cache(G, N, dim * 4, 0.25, max_batch=1 << 14)
    p = rt.solve_placement("clique_part", G, ids, freqs, 25.0)
    cache.set_placement(p)
    host = pinned_table(table)
    for r in range(G):
        cache.build(r, 0, host.data_ptr())
    cache.connect_local()
    for r in range(G):
        cache.attach_peers(r)
    cache.tune(0, direct_max_host_rows=1000)
    src = np.asarray(p.block_access_from).reshape(G, -1)[0][p.nid_to_block]
    peer, far = np.nonzero(src == 1)[0], np.nonzero(src == G)[0]
    assert len(peer) > 0 and len(far) > 0
    rng = np.random.default_rng(2)
    peer_heavy = np.concatenate([rng.choice(peer, 6000), rng.choice(far, 2000)]).astype(np.int64)
    host_heavy = np.concatenate([rng.choice(peer, 500), rng.choice(far, 2000)]).astype(np.int64)
    for keys in (peer_heavy,) * 3:      # grouped (no record yet), then direct twice
        assert lookup_np(cache, 0, keys).tobytes() == orc.gather(table, keys).tobytes()
    st = cache.stats(0)
    assert st["lookups_direct"] == 2 and (st["last_remote"], st["last_host"]) == (6000, 2000)
    for keys in (host_heavy,) * 3:      # direct twice more (the record lags), then grouped
        assert lookup_np(cache, 0, keys).tobytes() == orc.gather(table, keys).tobytes()
    st = cache.stats(0)
    assert st["lookups_direct"] == 4 and (st["last_remote"], st["last_host"]) == (500, 2000)
    cache.close()


def test_golden_cases_at_configuration_sizes(built_lib, golden_cases_large, extract_mode):
    """Full-size cases: 1 M x 128 fp32 with every row on the host and one deduplicated batch of
    65,536 draws; 2 M x 64 fp16 (128-byte rows) on 4 replicas with 20 % cached each."""
    if extract_mode in ("auto", "grouped_static"):
        pytest.skip("grouped and direct cover it")
    for case in golden_cases_large:
        w = case_workload(case)
        cache = make_cache(w, max_batch=1 << 17)
        for r in range(w.G):
            keys = w.keys(rank=r)
            got = lookup_np(cache, r, keys)
            assert digest(got) == case["ranks"][str(r)]["out"], (case["name"], r)
            st = cache.stats(r)
            assert st["err_key_range"] == 0 and st["err_table"] == 0
            per_src = case["ranks"][str(r)]["per_src"]
            assert st["num_local_rows"] == per_src[r]
            if w.G == 1 and w.pct == 0.0:
                assert (st["last_local"], st["last_remote"], st["last_host"]) == (0, 0, len(keys))
        cache.close()


def test_host_list_in_address_order(built_lib, extract_mode):
    """Grouped extraction with the host list put in address order (counting sort between lookup
    and gather) once a finished lookup has shown enough host rows: same bytes, and the stats say
    the ordered path ran.  Batches with duplicates, with one bucket only, and with no host row."""
    if extract_mode not in ("grouped", "grouped_static"):
        pytest.skip("the ordering belongs to the grouped path")
    from ugache_b200 import runtime as rt, workload as wl
    N, dim = 300_000, 32
    table = wl.table(61, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.05)
    cache = rt.Cache(1, N, dim * 4, 0.05, max_batch=1 << 16)
    p = rt.solve_placement("rep", 1, ids, freqs, 5.0)
    cache.set_placement(p)
    host = pinned_table(table)
    cache.build(0, 0, host.data_ptr())
    cache.tune(0, host_order_min_rows=100)
    rng = np.random.default_rng(7)
    missing = np.nonzero(np.asarray(p.block_access_from).reshape(1, -1)[0][p.nid_to_block] != 0)[0]
    cached = np.nonzero(np.asarray(p.block_access_from).reshape(1, -1)[0][p.nid_to_block] == 0)[0]
    batches = [wl.zipf_keys(1, 50_000, N, 1.05),                       # mixed, many host rows
               wl.zipf_keys(2, 50_000, N, 1.05),
               rng.choice(missing, 20_000).astype(np.int64),           # host only, duplicates
               np.sort(rng.choice(missing[:500], 3_000)).astype(np.int64),   # one address bucket
               rng.choice(cached, 5_000).astype(np.int64),             # no host row at all
               wl.zipf_keys(3, 65_536, N, 1.05)]                       # follows a batch without host rows: not ordered
    for i, keys in enumerate(batches):
        got = lookup_np(cache, 0, keys)
        assert got.tobytes() == orc.gather(table, keys).tobytes(), i
    st = cache.stats(0)
    assert st["err_table"] == 0 and st["err_key_range"] == 0
    # lookups 2..5 followed a lookup with >= 100 host rows; the one after the cached-only batch did not
    assert st["lookups_host_ordered"] == 4
    cache.reserve_batch(0, 1 << 17)                                    # drops and re-makes the ordered buffer
    keys = wl.zipf_keys(4, 100_000, N, 1.05)
    assert lookup_np(cache, 0, keys).tobytes() == orc.gather(table, keys).tobytes()
    assert cache.stats(0)["lookups_host_ordered"] == 5
    cache.close()


def test_refresh_with_a_fill_of_several_batches(built_lib, extract_mode):
    """A refresh that brings in more rows than one fill batch: the batches run on the
    library's low-priority stream and take consecutive windows of the free-slot ring, also across
    its wrap-around; lookups are exact afterwards and every stored row has its own slot."""
    if extract_mode not in ("grouped", "direct"):
        pytest.skip("one grouped and one direct run are enough")
    from ugache_b200 import runtime as rt, workload as wl
    N, dim = 600_000, 16
    table = wl.table(91, N, dim)
    rng = np.random.default_rng(17)
    order = rng.permutation(N).astype(np.uint32)
    cache = rt.Cache(1, N, dim * 4, 0.30, max_batch=1 << 15, table_kind=1)
    cache.set_placement(rt.solve_placement("rep", 1, order, None, 30.0))
    host = pinned_table(table)
    cache.build(0, 0, host.data_ptr())
    allk = torch.arange(N, dtype=torch.int32, device="cuda")
    for round_ in range(3):                      # each round replaces 150,000 of the 180,000 rows
        order = np.roll(order, 150_000)
        p = rt.solve_placement("rep", 1, order, None, 30.0)
        cache.refresh_all_local(p, [0])
        words = cache.table_words(0, allk).cpu().numpy().view(np.uint32)
        stored = p.nid_to_block == 0
        assert np.array_equal(words != 0xFFFFFFFF, stored), round_
        slots = words[stored] & 0x0FFFFFFF
        assert len(np.unique(slots)) == int(stored.sum())
        assert slots.max() < int(N * 0.301)
        keys = rng.integers(0, N, 20_000).astype(np.int64)
        assert lookup_np(cache, 0, keys).tobytes() == orc.gather(table, keys).tobytes()
        st = cache.stats(0)
        assert st["err_table"] == 0 and st["free_rows"] == st["capacity_rows"] - int(stored.sum())
    cache.close()
