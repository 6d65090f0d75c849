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
from tests.conftest import ROOT, oracle_solver
from tests.helpers import (REF_EXTRACT_CASES, REF_FILL_CASES, oracle_table_words, ref_extract_case,
                           ref_fill_case, ref_table_scenario, write_ref_table_scenario)

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


REF_EXTRACT = os.path.join(ROOT, "oracle", "_ref", "ref_extract_pin")


def run_ref_extract(binary, workdir, blob):
    with open(os.path.join(workdir, "extract.bin"), "wb") as f:
        f.write(blob)
    env = dict(os.environ, USER=os.environ.get("USER", "root"))
    p = subprocess.run([binary, str(workdir)], env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "ref extract ok" in p.stdout, p.stdout + p.stderr[-2000:]
    return dict(out=np.fromfile(os.path.join(workdir, "out.bin"), dtype=np.uint8),
                records=np.fromfile(os.path.join(workdir, "records.bin"), dtype=np.uint64),
                groups=np.fromfile(os.path.join(workdir, "groups.bin"), dtype=np.uint32))


@pytest.mark.skipif(not os.path.exists(REF_EXTRACT), reason="reference pin binary not built")
@pytest.mark.parametrize("case", REF_EXTRACT_CASES, ids=[c["name"] for c in REF_EXTRACT_CASES])
def test_reference_extraction_kernels_agree_with_oracle(tmp_path, case):
    """Lookup -> sort -> boundaries -> per-location row copy, all by the reference's device
    code, on the oracle's cache model of one reader: records, group boundaries and output
    bytes must be the oracle's."""
    blob, want = ref_extract_case(orc, oracle_solver, case)
    got = run_ref_extract(REF_EXTRACT, tmp_path, blob)
    assert np.array_equal(got["groups"], want["groups"])
    assert np.array_equal(got["records"], want["records"])
    assert np.array_equal(got["out"], want["out"].reshape(-1))


@pytest.mark.skipif(not os.path.exists(REF_EXTRACT), reason="reference pin binary not built")
@pytest.mark.parametrize("mode", ["grouped", "direct"])
@pytest.mark.parametrize("case", REF_EXTRACT_CASES, ids=[c["name"] for c in REF_EXTRACT_CASES])
def test_product_lookup_equals_reference_extraction(built_lib, tmp_path, case, mode, monkeypatch):
    """The shipped library (through its C ABI) against the reference's device code directly:
    same table, same placement, same reader, same key batch -> same output bytes, in both
    extraction modes."""
    monkeypatch.setenv("UGC_EXTRACT_MODE", mode)
    from tests.helpers import case_workload
    from tests.test_gpu_parity import lookup_np, make_cache
    blob, _ = ref_extract_case(orc, oracle_solver, case)
    ref = run_ref_extract(REF_EXTRACT, tmp_path, blob)
    w = case_workload(case)                      # placement solved by the library's own solver
    cache = make_cache(w, table_kind=1 if case["flat"] else 2)
    got = lookup_np(cache, case["rank"], w.keys(rank=case["rank"]))
    st = cache.stats(case["rank"])
    cache.close()
    assert np.array_equal(got.reshape(-1), ref["out"])
    g = ref["groups"]
    r = case["rank"]
    assert st["last_local"] == int(g[r + 1] - g[r])
    assert st["last_host"] == int(g[-1] - g[-2])
    assert st["last_remote"] == int(g[-2]) - st["last_local"]


def run_ref_fill(binary, workdir, blob):
    with open(os.path.join(workdir, "fill.bin"), "wb") as f:
        f.write(blob)
    env = dict(os.environ, USER=os.environ.get("USER", "root"))
    p = subprocess.run([binary, "--fill", str(workdir)], env=env, capture_output=True, text=True,
                       timeout=300)
    assert p.returncode == 0 and "ref fill ok" in p.stdout, p.stdout + p.stderr[-2000:]
    return np.fromfile(os.path.join(workdir, "slice.bin"), dtype=np.uint8)


@pytest.mark.skipif(not os.path.exists(REF_EXTRACT), reason="reference pin binary not built")
@pytest.mark.parametrize("case", REF_FILL_CASES, ids=[c["name"] for c in REF_FILL_CASES])
def test_reference_fill_kernels_agree_with_oracle(tmp_path, case):
    """The reference's build fill (slice[j] = host[key[j]]) and refresh scatter
    (slice[dst[j]] = host[key[j]], 4092-row batches) against the oracle's fill."""
    blob, want = ref_fill_case(orc, case)
    got = run_ref_fill(REF_EXTRACT, tmp_path, blob)
    assert np.array_equal(got, want.reshape(-1))
