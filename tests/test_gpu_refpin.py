"""The reference's OWN table kernels, run on the GPU, against the CPU oracle.

``oracle/_ref/ref_pin`` is built (by ``make -C oracle ref``, where the reference tree is
available) from the reference's unmodified sources: its SimpleHashTable / FlatHashTable, its
insert / evict kernels and its ``lookup_hashmap_with_helper`` kernel with its own ``EmbedVal``
helper.  This test feeds it a seeded scenario (insert per location, evict, re-insert, look up
the whole id space) and requires the oracle's restatement to return exactly the same packed
word for every key.  Skipped where the binary is absent."""
import os
import subprocess

import numpy as np
import pytest

from oracle import oracle as orc
from tests.conftest import ROOT
from tests.helpers import oracle_table_words, ref_table_scenario, write_ref_table_scenario

pytestmark = pytest.mark.gpu

REF_PIN = os.path.join(ROOT, "oracle", "_ref", "ref_pin")


@pytest.mark.skipif(not os.path.exists(REF_PIN), reason="reference pin binary not built")
@pytest.mark.parametrize("seed,N,n_ins,n_ev,n_re,fallback", [
    (2025, 200_000, 50_000, 5_000, 2_000, 3),
    (7, 4_096, 4_000, 4_000, 4_000, 8),      # nearly every id cached, all evicted and re-inserted
    (11, 1_000_000, 300_000, 0, 0, 1),       # insert-only, larger than one probe window
])
def test_reference_table_kernels_agree_with_oracle(tmp_path, seed, N, n_ins, n_ev, n_re, fallback):
    sc = ref_table_scenario(seed, N, n_ins, n_ev, n_re)
    write_ref_table_scenario(tmp_path / "scenario.bin", N, fallback, sc)
    env = dict(os.environ, USER=os.environ.get("USER", "root"))
    p = subprocess.run([REF_PIN, "--gpu", str(tmp_path)], env=env, capture_output=True, text=True,
                       timeout=300)
    assert p.returncode == 0 and "ref tables ok" in p.stdout, p.stdout + p.stderr[-2000:]
    got_simple = np.fromfile(tmp_path / "words_simple.bin", dtype=np.uint32)
    got_flat = np.fromfile(tmp_path / "words_flat.bin", dtype=np.uint32)
    want_simple, want_flat = oracle_table_words(orc, N, fallback, sc)
    assert np.array_equal(want_simple, want_flat)
    assert np.array_equal(got_simple, want_simple)
    assert np.array_equal(got_flat, want_flat)
