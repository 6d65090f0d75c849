"""Writes tests/golden/ref_tables.npz: the output of the REFERENCE's own GPU table kernels.

Needs a GPU and ``oracle/_ref/ref_pin`` (``make -C oracle ref`` where the reference tree is
available).  The binary runs the reference's SimpleHashTable and FlatHashTable — its insert,
evict and lookup kernels, unmodified — over the scenario of ``tests.helpers.ref_table_scenario``
and prints the packed word its lookup returns for every key of the id space.

    python tests/golden/make_ref_tables.py [out.npz]

The committed file was produced on a B200.  It stores only the scenario's parameters and the
words, so the CPU test-suite regenerates the scenario from the seed and compares the oracle."""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from tests.helpers import ref_table_scenario, write_ref_table_scenario  # noqa: E402

PARAMS = dict(seed=77, N=60_000, n_ins=20_000, n_ev=3_000, n_re=1_000, fallback=5)


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_tables.npz")
    binary = os.path.join(ROOT, "oracle", "_ref", "ref_pin")
    p = PARAMS
    sc = ref_table_scenario(p["seed"], p["N"], p["n_ins"], p["n_ev"], p["n_re"])
    with tempfile.TemporaryDirectory() as d:
        write_ref_table_scenario(os.path.join(d, "scenario.bin"), p["N"], p["fallback"], sc)
        env = dict(os.environ, USER=os.environ.get("USER", "root"))
        r = subprocess.run([binary, "--gpu", d], env=env, capture_output=True, text=True, timeout=300)
        if r.returncode != 0 or "ref tables ok" not in r.stdout:
            raise SystemExit(r.stdout + r.stderr[-2000:])
        simple = np.fromfile(os.path.join(d, "words_simple.bin"), dtype=np.uint32)
        flat = np.fromfile(os.path.join(d, "words_flat.bin"), dtype=np.uint32)
    np.savez_compressed(out, simple=simple, flat=flat, **{k: np.int64(v) for k, v in p.items()})
    print("wrote", out, simple.size, "words")


if __name__ == "__main__":
    main()
