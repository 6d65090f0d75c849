"""Makes tests/golden/ref_solver.json: what THE REFERENCE'S OWN placement heuristics
(IntuitiveSolver, RepSolver, CliquePartSolver of coll_cache_lib/coll_cache/optimal_solver_class.cc,
compiled in place into oracle/_ref/ref_solver_pin by `make -C oracle ref-solver REF=...`) answer
on seeded hotness rankings, as SHA-256 digests of the complete placement arrays.  The CPU suite
holds the oracle's solvers (and, through tests/test_host_logic.py, the library's) to these.

    python tests/golden/make_solver_pin.py            # needs oracle/_ref/ref_solver_pin

No GPU is needed.  Test infrastructure only.
"""
import hashlib
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

POLICY = {"intuitive": 0, "rep": 1, "clique_part": 2}

# name, policy, G, N, cache percent, alpha of the ranking's frequencies, T_local, T_remote, T_cpu
CASES = [
    ("intuitive_g1", "intuitive", 1, 50_000, 10.0, 1.2, 1.0, 8.9, 125.0),
    ("intuitive_g2_zipf12", "intuitive", 2, 60_000, 10.0, 1.2, 1.0, 8.9, 125.0),
    ("intuitive_g4_zipf08", "intuitive", 4, 100_000, 5.0, 0.8, 1.0, 8.9, 125.0),
    ("intuitive_g8_zipf12", "intuitive", 8, 200_000, 10.0, 1.2, 1.0, 8.9, 125.0),
    ("intuitive_g8_zipf105_20pct", "intuitive", 8, 150_000, 20.0, 1.05, 1.0, 8.9, 125.0),
    ("intuitive_g8_flat_hotness", "intuitive", 8, 80_000, 2.0, 0.3, 1.0, 8.9, 125.0),
    ("intuitive_g4_cheap_host", "intuitive", 4, 70_000, 8.0, 1.0, 1.0, 8.9, 6.0),   # mu < 1: replicate only
    ("intuitive_g3_odd", "intuitive", 3, 33_333, 7.5, 1.1, 1.0, 4.0, 60.0),
    ("rep_g4", "rep", 4, 50_000, 12.5, 1.2, 1.0, 8.9, 125.0),
    ("rep_g8_tiny", "rep", 8, 1_000, 0.3, 1.2, 1.0, 8.9, 125.0),
    ("clique_g2", "clique_part", 2, 60_000, 10.0, 1.2, 1.0, 8.9, 125.0),
    ("clique_g8", "clique_part", 8, 120_000, 5.0, 1.05, 1.0, 8.9, 125.0),
    ("clique_g4_covers_all", "clique_part", 4, 10_000, 30.0, 1.2, 1.0, 8.9, 125.0),
]


def ranking(name, N, alpha):
    """A seeded hotness ranking: ids in random order, frequencies descending ~ rank^-alpha with
    ties (integer counts), as a recorded workload would give."""
    seed = int.from_bytes(hashlib.sha256(name.encode()).digest()[:4], "little")
    rng = np.random.default_rng(seed)
    ids = rng.permutation(N).astype(np.uint32)
    w = (np.arange(1, N + 1, dtype=np.float64)) ** (-alpha)
    freqs = np.maximum(1, np.floor(w / w[-1] * 3.0)).astype(np.uint64)
    freqs = np.minimum(freqs, 2 ** 31 - 1).astype(np.uint32)
    return ids, freqs


def digest_placement(nid_to_block, placement, access, density):
    h = hashlib.sha256()
    h.update(np.ascontiguousarray(nid_to_block, dtype=np.uint32).tobytes())
    h.update(np.ascontiguousarray(placement, dtype=np.uint8).tobytes())
    h.update(np.ascontiguousarray(access, dtype=np.uint8).tobytes())
    h.update(np.ascontiguousarray(density, dtype=np.float64).tobytes())
    return h.hexdigest()


def run_reference(binary, case):
    name, policy, G, N, pct, alpha, tl, tr, tc = case
    ids, freqs = ranking(name, N, alpha)
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "solver_case.bin"), "wb") as f:
            f.write(struct.pack("<4I", G, N, POLICY[policy], 0))
            f.write(struct.pack("<4d", pct, tl, tr, tc))
            ids.tofile(f)
            freqs.tofile(f)
        env = dict(os.environ, OMP_NUM_THREADS="4", USER=os.environ.get("USER", "pin"))
        r = subprocess.run([binary, d], capture_output=True, text=True, env=env)
        if r.returncode != 0:
            raise SystemExit("%s failed on %s:\n%s" % (binary, name, r.stderr[-2000:]))
        n2b = np.fromfile(os.path.join(d, "ref_nid_to_block.bin"), dtype=np.uint32)
        with open(os.path.join(d, "ref_blocks.bin"), "rb") as f:
            (B,) = struct.unpack("<I", f.read(4))
            placement = np.frombuffer(f.read(B), dtype=np.uint8)
            access = np.frombuffer(f.read(G * B), dtype=np.uint8).reshape(G, B)
            density = np.frombuffer(f.read(8 * B), dtype=np.float64)
    return n2b, placement, access, density


def oracle_placement(case):
    from oracle import oracle as orc
    name, policy, G, N, pct, alpha, tl, tr, tc = case
    ids, freqs = ranking(name, N, alpha)
    if policy == "intuitive":
        p = orc.solve_intuitive(G, ids, freqs, pct, tl, tr, tc)
    elif policy == "rep":
        p = orc.solve_rep(G, ids, pct)
    else:
        p = orc.solve_clique_part(G, ids, pct)
    return p.nid_to_block, p.block_placement, p.block_access_from, p.block_density


def main():
    binary = os.path.join(ROOT, "oracle", "_ref", "ref_solver_pin")
    if not os.path.exists(binary):
        raise SystemExit("build it first: make -C oracle ref-solver REF=/path/to/reference")
    out = {"note": "SHA-256 over nid_to_block (u32), block_placement (u8), block_access_from (u8, "
                   "[G, B]) and block_density (f64) as the reference's solver classes produce them",
           "cases": []}
    for case in CASES:
        ref = run_reference(binary, case)
        mine = oracle_placement(case)
        same = digest_placement(*ref) == digest_placement(*mine)
        print("%-28s blocks %d  reference %s  oracle %s" % (case[0], len(ref[1]), digest_placement(*ref)[:12],
                                                             "identical" if same else "DIFFERS"))
        if not same:
            for nm, a, b in zip(("nid_to_block", "placement", "access", "density"), ref, mine):
                a, b = np.asarray(a), np.asarray(b)
                if a.shape != b.shape or not np.array_equal(a, b):
                    print("   ", nm, "differs:", a.shape, b.shape, a.ravel()[:8], b.ravel()[:8])
        out["cases"].append({"name": case[0], "policy": case[1], "G": case[2], "N": case[3], "cache_percent": case[4],
                             "alpha": case[5], "T_local": case[6], "T_remote": case[7], "T_cpu": case[8],
                             "num_block": int(len(ref[1])), "digest": digest_placement(*ref)})
    with open(os.path.join(HERE, "ref_solver.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", os.path.join(HERE, "ref_solver.json"))


if __name__ == "__main__":
    main()
