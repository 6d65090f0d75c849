"""Shared helpers of the test-suite."""
import hashlib

import numpy as np


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def case_workload(case, solver=None):
    from ugache_b200 import workload as wl
    kw = {k: v for k, v in case.items()
          if k in ("N", "dim", "dtype", "G", "pct", "alpha", "n_keys", "policy", "seed", "dedup")}
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
