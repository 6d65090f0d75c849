"""Shared helpers of the test-suite."""
import hashlib

import numpy as np


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def case_workload(case, solver=None):
    from ugache_b200 import workload as wl
    kw = {k: v for k, v in case.items()
          if k in ("N", "dim", "dtype", "G", "pct", "alpha", "n_keys", "policy", "seed", "dedup")}
    if case.get("large"):
        # full-size cases: the rows come from the oracle's C generator (same definition as
        # workload.table, checked on the small cases; numpy needs GBs of temporaries here)
        from oracle import oracle as orc
        kw["table_array"] = orc.gen_rows(case["seed"], 0, case["N"], case["dim"], np.dtype(case["dtype"]))
    return wl.Workload(solver=solver, **kw)


def ref_table_scenario(seed, N, n_ins, n_ev, n_re):
    """Operation list for the reference's table kernels: unique keys inserted with location
    i mod 3 and a random 28-bit offset, the first ``n_ev`` of them evicted, the first ``n_re``
    of those inserted again at location 1 with new offsets.  Only present keys are evicted and
    only absent keys inserted — the reference's kernels assume both."""
    rng = np.random.default_rng(seed)
    keys = rng.choice(N, size=n_ins, replace=False).astype(np.uint32)
    locs = (np.arange(n_ins) % 3).astype(np.uint32)
    offs = rng.integers(0, 1 << 28, n_ins).astype(np.uint32)
    evict = keys[:n_ev].copy()
    rk = evict[:n_re].copy()
    ro = rng.integers(0, 1 << 28, n_re).astype(np.uint32)
    return keys, locs, offs, evict, rk, ro


def write_ref_table_scenario(path, N, fallback, scenario):
    keys, locs, offs, evict, rk, ro = scenario
    with open(path, "wb") as f:
        np.array([N, keys.size, evict.size, rk.size, fallback], dtype=np.uint32).tofile(f)
        for a in (keys, locs, offs, evict, rk, ro):
            a.tofile(f)


def oracle_table_words(orc, N, fallback, scenario):
    """The oracle's answer for the scenario: (words of the probing table, words of the
    direct-index table) for every key 0..N-1."""
    keys, locs, offs, evict, rk, ro = scenario
    t = orc.SimpleTable(keys.size)
    for loc in range(3):
        for k, o in zip(keys[locs == loc], offs[locs == loc]):
            t.insert(int(k), orc.pack_loc_off(loc, int(o)))
    for k in evict:
        t.evict(int(k))
    for k, o in zip(rk, ro):
        t.insert(int(k), orc.pack_loc_off(1, int(o)))
    allk = np.arange(N, dtype=np.int64)
    rec = t.lookup(allk, fallback_loc=fallback)
    simple = ((rec["loc"].astype(np.uint64) << 28) + rec["off"]).astype(np.uint32)
    flat = np.full(N, 0xFFFFFFFF, dtype=np.uint32)
    flat[keys] = (locs << 28) + offs
    flat[evict] = 0xFFFFFFFF
    flat[rk] = (1 << 28) + ro
    rec2 = orc.lookup_flat(flat, allk, fallback_loc=fallback)
    return simple, ((rec2["loc"].astype(np.uint64) << 28) + rec2["off"]).astype(np.uint32)


# Cases run through the reference's own extraction kernels (oracle/ref_extract_pin.cu).
REF_EXTRACT_CASES = [
    dict(name="g4_intuitive_f32x128", N=60_000, dim=128, dtype="float32", G=4, pct=0.10, alpha=1.2,
         n_keys=26_000, policy="intuitive", seed=21, dedup=False, rank=1, flat=1),
    dict(name="g8_clique_f16x64", N=80_000, dim=64, dtype="float16", G=8, pct=0.05, alpha=1.05,
         n_keys=40_000, policy="clique_part", seed=22, dedup=False, rank=5, flat=1),
    dict(name="g2_rep_probing_f32x24", N=50_000, dim=24, dtype="float32", G=2, pct=0.04, alpha=1.2,
         n_keys=9_000, policy="rep", seed=23, dedup=False, rank=0, flat=0),
    dict(name="g3_intuitive_f32x5_dedup", N=30_000, dim=5, dtype="float32", G=3, pct=0.10, alpha=1.1,
         n_keys=7_000, policy="intuitive", seed=24, dedup=True, rank=2, flat=0),
    dict(name="g1_host_only_f32x32", N=20_000, dim=32, dtype="float32", G=1, pct=0.0, alpha=1.2,
         n_keys=5_000, policy="rep", seed=25, dedup=False, rank=0, flat=1),
]


def ref_extract_case(orc, solver, case):
    """Builds, from the oracle's cache model of one reader, the input of the reference
    extraction pin and the oracle's expectation of its three outputs.

    Returns (file_bytes, want) with want = dict(out=uint8[n, row_bytes], records=uint64[n]
    sorted as the reference groups them, groups=uint32[G + 2])."""
    w = case_workload(case, solver)
    G, rank = w.G, case["rank"]
    words, cnt, slot_of = orc.model_build(w.placement, rank, w.capacity)
    loc = (words >> 28).astype(np.uint32)
    off = (words & ((1 << 28) - 1)).astype(np.uint32)
    cached = np.nonzero(words != 0xFFFFFFFF)[0].astype(np.uint32)   # host keys have no entry
    tab = w.table.view(np.uint8).reshape(w.N, w.row_bytes)
    sources, rows = [], []
    for g in range(G):
        own = np.nonzero(slot_of[g] != 0xFFFFFFFF)[0]
        n_rows = int(slot_of[g][own].max()) + 1 if own.size else 0
        sl = np.zeros((n_rows, w.row_bytes), dtype=np.uint8)
        sl[slot_of[g][own]] = tab[own]
        sources.append(sl)
        rows.append(n_rows)
    sources.append(tab)
    rows.append(w.N)
    keys = w.keys(rank=rank)
    hdr = np.array([w.N, cached.size, keys.size, G + 1, w.row_bytes, case["flat"]], dtype=np.uint32)
    parts = [hdr, cached, loc[cached], off[cached], np.array(rows, dtype=np.uint32),
             keys.astype(np.uint32)] + sources
    blob = b"".join(np.ascontiguousarray(p).tobytes() for p in parts)

    if case["flat"]:
        rec = orc.lookup_flat(words, keys, fallback_loc=G)
    else:
        t = orc.SimpleTable(cached.size)
        for g in range(G):          # the pin inserts location by location, in list order
            for k in cached[loc[cached] == g]:
                t.insert(int(k), int(words[k]))
        rec = t.lookup(keys, fallback_loc=G)
    out = orc.extract_records(rec, sources, w.row_bytes)
    assert np.array_equal(out, orc.gather(tab, keys))
    # the reference's record is {u32 dst; u32 (loc << 28) + off}, grouped by sorting it as one u64
    r64 = (((rec["loc"].astype(np.uint64) << np.uint64(28)) + rec["off"].astype(np.uint64))
           << np.uint64(32)) | rec["dst"].astype(np.uint64)
    r64.sort()
    groups = np.zeros(G + 2, dtype=np.uint32)
    groups[1:] = np.cumsum(np.bincount(rec["loc"].astype(np.int64), minlength=G + 1))
    return blob, dict(out=out, records=r64, groups=groups)


REF_FILL_CASES = [
    dict(name="f32x128", seed=31, N=40_000, dim=128, dtype="float32", n_build=5_000, slice_rows=6_000,
         n_scatter=5_500),
    dict(name="f16x64", seed=32, N=30_000, dim=64, dtype="float16", n_build=9_000, slice_rows=9_000,
         n_scatter=8_200),
    dict(name="f32x5", seed=33, N=10_000, dim=5, dtype="float32", n_build=1_000, slice_rows=1_500,
         n_scatter=700),
    dict(name="scatter_only", seed=34, N=10_000, dim=32, dtype="float32", n_build=0, slice_rows=4_100,
         n_scatter=4_093),
]


def ref_fill_case(orc, case):
    """(file_bytes, expected slice as uint8[slice_rows, row_bytes]) for the reference fill pin:
    a build fill of ``n_build`` rows in list order, then a refresh scatter of ``n_scatter`` rows
    to distinct slots (some overwrite build rows, some take free rows)."""
    rng = np.random.default_rng(case["seed"])
    dt = np.dtype(case["dtype"])
    N, rb = case["N"], case["dim"] * dt.itemsize
    tab = orc.gen_rows(case["seed"], 0, N, case["dim"], dt).view(np.uint8).reshape(N, rb)
    bkeys = rng.choice(N, size=case["n_build"], replace=False).astype(np.uint32)
    skeys = rng.choice(N, size=case["n_scatter"], replace=False).astype(np.uint32)
    sdst = rng.choice(case["slice_rows"], size=case["n_scatter"], replace=False).astype(np.uint32)
    hdr = np.array([N, bkeys.size, rb, case["slice_rows"], skeys.size], dtype=np.uint32)
    blob = b"".join(np.ascontiguousarray(p).tobytes() for p in (hdr, bkeys, skeys, sdst, tab))
    want = orc.fill(tab, bkeys, None, case["slice_rows"])
    sc = orc.fill(tab, skeys, sdst, case["slice_rows"])
    want[sdst] = sc[sdst]
    return blob, want
