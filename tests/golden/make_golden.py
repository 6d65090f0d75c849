"""Regenerates the committed fixtures in this folder.

  ref_pin.json    known answers printed by the reference's OWN code: its hashtable header
                  and sources are compiled in place from the reference tree by
                  ``make -C oracle ref`` (needs the reference tree and nvcc; runs on the
                  host, no GPU).  Pins the oracle's murmur3 hash, the packed
                  (location, offset) word and the probing-table sizing rule.
  cases.json      small seeded end-to-end cases with digests of the oracle's answers
                  (table rows, Zipf keys, placement arrays, per-key (location, offset)
                  words, gathered output).  The CUDA path and the oracle are both
                  checked against these.

Run from the repository root:  python tests/golden/make_golden.py [--reference /path]
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def make_ref_pin(reference):
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "ref",
                           "REF=" + reference])
    env = dict(os.environ, USER=os.environ.get("USER", "root"))
    out = subprocess.check_output([os.path.join(ROOT, "oracle", "_ref", "ref_pin")], env=env)
    data = json.loads(out)
    with open(os.path.join(HERE, "ref_pin.json"), "w") as f:
        json.dump(data, f, separators=(",", ":"))
    print("ref_pin.json:", {k: len(v) for k, v in data.items()})


# The small end-to-end cases.  Everything is derived from these parameters by
# ugache_b200/workload.py (shared with the tests), so a case is reproducible from its dict.
CASES = [
    dict(name="c1_host_only", N=20000, dim=128, dtype="float32", G=1, pct=0.0, alpha=1.2,
         n_keys=4096, policy="rep", seed=11, dedup=True),
    dict(name="g1_rep_10", N=50000, dim=128, dtype="float32", G=1, pct=0.10, alpha=1.2,
         n_keys=8192, policy="intuitive", seed=12, dedup=False),
    dict(name="g2_intuitive", N=40000, dim=128, dtype="float32", G=2, pct=0.10, alpha=1.2,
         n_keys=8192, policy="intuitive", seed=13, dedup=False),
    dict(name="g4_clique_f16", N=60000, dim=64, dtype="float16", G=4, pct=0.20, alpha=1.05,
         n_keys=10000, policy="clique_part", seed=14, dedup=False),
    dict(name="g8_intuitive", N=80000, dim=128, dtype="float32", G=8, pct=0.05, alpha=1.2,
         n_keys=6000, policy="intuitive", seed=15, dedup=False),
    dict(name="g3_dim24", N=30000, dim=24, dtype="float32", G=3, pct=0.08, alpha=0.8,
         n_keys=5000, policy="intuitive", seed=16, dedup=False),
]


# Cases at the sizes the benchmark configurations name: the CPU-runnable configuration in full
# (1,000,000 x 128 fp32 rows, one batch of 65,536 Zipf-1.2 draws deduplicated, every row on the
# host) and the fp16 x 64 row shape of the flat-skew configuration over more than a million
# rows with 20 % cached per GPU.  Kept in cases_large.json.
LARGE_CASES = [
    dict(name="c1_full_1Mx128_host_only", N=1_000_000, dim=128, dtype="float32", G=1, pct=0.0,
         alpha=1.2, n_keys=65_536, policy="rep", seed=101, dedup=True, large=True),
    dict(name="c4_shape_2Mx64f16_4gpu", N=2_000_000, dim=64, dtype="float16", G=4, pct=0.20,
         alpha=1.05, n_keys=100_000, policy="intuitive", seed=102, dedup=False, large=True),
]


def oracle_solver(policy, G, rank_ids, rank_freqs, cache_percent):
    """Placement through the ORACLE's restatement of the reference heuristics, with the
    B200 time ratios local : peer : host = 1 : 8000/900 : 8000/64."""
    from oracle import oracle as orc
    if policy == "intuitive":
        return orc.solve_intuitive(G, rank_ids, rank_freqs, cache_percent, 1.0, 8000.0 / 900.0,
                                   8000.0 / 64.0)
    if policy == "rep":
        return orc.solve_rep(G, rank_ids, cache_percent)
    return orc.solve_clique_part(G, rank_ids, cache_percent)


def make_cases(cases=None, fname="cases.json"):
    from ugache_b200 import workload as wl
    from oracle import oracle as orc
    out = []
    for c in (CASES if cases is None else cases):
        kw = {k: v for k, v in c.items() if k not in ("name", "large")}
        if c.get("large"):
            kw["table_array"] = orc.gen_rows(c["seed"], 0, c["N"], c["dim"], np.dtype(c["dtype"]))
        w = wl.Workload(solver=oracle_solver, **kw)
        entry = dict(c)
        entry["table_head"] = digest(w.table[:64])
        entry["table"] = digest(w.table)
        entry["placement"] = digest(w.placement.nid_to_block) + digest(w.placement.block_access_from)
        ranks = {}
        for r in range(c["G"]):
            keys = w.keys(rank=r, it=0)
            words, cnt, _ = orc.model_build(w.placement, r, w.capacity)
            ranks[str(r)] = dict(keys=digest(keys), words=digest(words),
                                 per_src=[int(x) for x in cnt],
                                 out=digest(orc.gather(w.table, keys)))
        entry["ranks"] = ranks
        out.append(entry)
    with open(os.path.join(HERE, fname), "w") as f:
        json.dump(out, f, indent=1)
    print(fname + ":", [c["name"] for c in out])


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("UGACHE_REFERENCE", ""),
                    help="root of the reference's source tree (or $UGACHE_REFERENCE); needed for "
                         "ref_pin.json only")
    ap.add_argument("--skip-ref", action="store_true")
    a = ap.parse_args()
    if not a.skip_ref:
        if not a.reference:
            ap.error("--reference (or $UGACHE_REFERENCE) is required unless --skip-ref is given")
        make_ref_pin(a.reference)
    make_cases()
    make_cases(LARGE_CASES, "cases_large.json")
