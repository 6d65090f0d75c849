"""The CPU oracle against (a) known answers printed by the reference's own code and
(b) the committed digests of its answers on the small seeded cases."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.conftest import oracle_solver
from tests.helpers import case_workload, digest


def test_murmur3_matches_reference(ref_pin):
    for key, want in ref_pin["murmur3_32"]:
        assert orc.murmur3_32(key) == want


def test_packed_word_matches_reference(ref_pin):
    for loc, off, data, rloc, roff in ref_pin["emb_cache_off"]:
        w = orc.pack_loc_off(loc, off)
        assert w == data
        assert orc.lib().orc_word_loc(w) == rloc
        assert orc.lib().orc_word_off(w) == roff


def test_table_size_matches_reference(ref_pin):
    for num, want in ref_pin["table_size"]:
        assert orc.table_size(num) == want


def test_constants_match_reference(ref_pin):
    assert ref_pin["constants"]["kEmptyKey"] == 0xFFFFFFFF
    assert ref_pin["constants"]["kEmptyPos"] == 0xFFFFFFFF


def test_table_choice_rule():
    # sizes worked out from the reference rule: flat iff TableSize(entries) > N/2
    N = 100_000_000
    assert orc.use_flat_table(80_000_000, N)       # 8 GPUs x 10 %
    assert orc.use_flat_table(40_000_000, N)       # 8 GPUs x 5 %
    assert not orc.use_flat_table(10_000_000, N)   # 1 GPU x 10 %
    assert orc.cache_capacity(N, 0.10) == 10_100_000


def test_probing_table_semantics():
    rng = np.random.default_rng(1)
    keys = rng.choice(1 << 20, size=5000, replace=False).astype(np.uint32)
    t = orc.SimpleTable(len(keys))
    ref = {}
    for i, k in enumerate(keys):
        t.insert(int(k), orc.pack_loc_off(i % 8, i))
        ref[int(k)] = orc.pack_loc_off(i % 8, i)
    for k in keys[:500]:
        pos = t.search(int(k))
        assert pos != 0xFFFFFFFF and t.buckets[pos]["val"] == ref[int(k)]
    absent = np.setdiff1d(np.arange(1 << 20, dtype=np.uint32), keys)[:500]
    for k in absent:
        assert t.search(int(k)) == 0xFFFFFFFF
    # evict then re-insert elsewhere in the chain: searches walk past tombstones
    for k in keys[:1000]:
        t.evict(int(k))
    for k in keys[:1000]:
        assert t.search(int(k)) == 0xFFFFFFFF
    for k in keys[1000:1500]:
        assert t.search(int(k)) != 0xFFFFFFFF
    for k in keys[:200]:
        t.insert(int(k), 7)
        assert t.buckets[t.search(int(k))]["val"] == 7
    rec = t.lookup(np.concatenate([keys[:10], absent[:10]]).astype(np.int64), fallback_loc=8)
    assert (rec["loc"][10:] == 8).all() and (rec["off"][10:] == absent[:10]).all()


def test_records_gather_equals_plain_gather():
    case = dict(N=5000, dim=16, dtype="float32", G=4, pct=0.1, alpha=1.2, n_keys=3000,
                policy="intuitive", seed=5, dedup=False)
    w = case_workload(case, oracle_solver)
    for r in range(4):
        words, cnt, slot_of = orc.model_build(w.placement, r, w.capacity)
        # per-GPU slices as the model places them
        slices = []
        for g in range(4):
            sl = np.zeros((w.capacity, w.dim), dtype=np.float32)
            own = np.nonzero(slot_of[g] != 0xFFFFFFFF)[0]
            sl[slot_of[g][own]] = w.table[own]
            slices.append(sl)
        keys = w.keys(rank=r)
        rec = orc.lookup_flat(words, keys, fallback_loc=4)
        out = orc.extract_records(rec, slices + [w.table], w.row_bytes)
        assert (out.view(np.float32) == orc.gather(w.table, keys)).all()


def test_golden_cases(golden_cases):
    for case in golden_cases:
        w = case_workload(case, oracle_solver)
        assert digest(w.table) == case["table"], case["name"]
        assert digest(orc.gen_rows(case["seed"], 0, 64, case["dim"], np.dtype(case["dtype"]))) \
            == case["table_head"]
        assert digest(w.placement.nid_to_block) + digest(w.placement.block_access_from) \
            == case["placement"]
        for r, want in case["ranks"].items():
            keys = w.keys(rank=int(r))
            assert digest(keys) == want["keys"]
            words, cnt, _ = orc.model_build(w.placement, int(r), w.capacity)
            assert digest(words) == want["words"]
            assert [int(x) for x in cnt] == want["per_src"]
            assert digest(orc.gather(w.table, keys)) == want["out"]


def test_golden_cases_at_configuration_sizes(golden_cases_large):
    """The CPU-runnable configuration in full (1 M x 128 fp32, 65,536 draws deduplicated, all
    rows on the host) and the fp16 x 64 row shape over 2 M rows: keys, placement, per-key words
    and gathered bytes against the committed digests."""
    for case in golden_cases_large:
        w = case_workload(case, oracle_solver)
        assert digest(w.table) == case["table"], case["name"]
        assert digest(w.placement.nid_to_block) + digest(w.placement.block_access_from) \
            == case["placement"]
        for r, want in case["ranks"].items():
            keys = w.keys(rank=int(r))
            assert digest(keys) == want["keys"]
            if case["dedup"]:
                assert len(np.unique(keys)) == len(keys) <= case["n_keys"]
            words, cnt, _ = orc.model_build(w.placement, int(r), w.capacity)
            assert digest(words) == want["words"]
            assert [int(x) for x in cnt] == want["per_src"]
            assert digest(orc.gather(w.table, keys)) == want["out"]
    c1 = golden_cases_large[0]
    assert c1["N"] == 1_000_000 and c1["dim"] == 128 and c1["n_keys"] == 65_536 and c1["pct"] == 0.0
    assert c1["ranks"]["0"]["per_src"][0] == 0            # nothing cached: every key is a host row


def test_refresh_slot_model():
    N, G = 4000, 2
    ids = np.arange(N, dtype=np.uint32)
    old = orc.solve_rep(G, ids, 10.0)
    new = orc.solve_rep(G, np.roll(ids, 100), 10.0)
    cap = orc.cache_capacity(N, 0.10)
    _, _, slot_of = orc.model_build(old, 0, cap)
    slots = slot_of[0].copy()
    free = np.arange(int((slots != 0xFFFFFFFF).sum()), cap, dtype=np.uint32)
    free2, ev, ins = orc.model_refresh_slots(0, old, new, slots, free)
    assert ev == 100 and ins == 100
    stored = np.nonzero(new.block_placement[new.nid_to_block] & 1)[0]
    assert (slots[stored] != 0xFFFFFFFF).all()
    assert len(np.unique(slots[stored])) == len(stored)
    assert len(free2) == len(free)


def test_empty_and_ragged_gather():
    t = orc.gen_rows(3, 0, 100, 8)
    assert orc.gather(t, np.zeros(0, dtype=np.int64)).shape == (0, 8)
    for n in (1, 7, 33):
        k = np.arange(n, dtype=np.int64) * 3 % 100
        assert (orc.gather(t, k) == t[k]).all()
    assert (orc.gather(t, np.array([5, 69]), empty_feat=6) == t[[5, 5]]).all()


def test_oracle_tables_match_reference_gpu_kernels():
    """tests/golden/ref_tables.npz holds what the reference's own SimpleHashTable and
    FlatHashTable kernels returned on a B200 (tests/golden/make_ref_tables.py): insert per
    location, evict, re-insert, then a lookup of every id with its EmbedVal helper."""
    import os
    from tests.helpers import oracle_table_words, ref_table_scenario
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_tables.npz"))
    N, fb = int(z["N"]), int(z["fallback"])
    sc = ref_table_scenario(int(z["seed"]), N, int(z["n_ins"]), int(z["n_ev"]), int(z["n_re"]))
    simple, flat = oracle_table_words(orc, N, fb, sc)
    assert np.array_equal(simple, z["simple"])
    assert np.array_equal(flat, z["flat"])
    # the fixture is not trivial: hits at three locations, evicted ids and misses all occur
    loc = z["simple"] >> 28
    assert {0, 1, 2, fb} <= set(np.unique(loc).tolist())


def test_oracle_extraction_matches_reference_gpu_kernels():
    """tests/golden/ref_extract.json: digests of what the reference's own lookup-helper, sort,
    boundary and extract_data kernels produced on a B200 for REF_EXTRACT_CASES
    (tests/golden/make_ref_extract.py)."""
    import json
    import os
    from tests.helpers import REF_EXTRACT_CASES, ref_extract_case
    with open(os.path.join(os.path.dirname(__file__), "golden", "ref_extract.json")) as f:
        gold = json.load(f)
    from tests.helpers import REF_FILL_CASES, ref_fill_case
    assert set(gold) == {c["name"] for c in REF_EXTRACT_CASES} | {"fill_" + c["name"] for c in REF_FILL_CASES}
    for case in REF_FILL_CASES:
        _, want = ref_fill_case(orc, case)
        assert digest(want) == gold["fill_" + case["name"]]["slice"], case["name"]
    for case in REF_EXTRACT_CASES:
        _, want = ref_extract_case(orc, oracle_solver, case)
        g = gold[case["name"]]
        assert [int(x) for x in want["groups"]] == g["groups"], case["name"]
        assert digest(want["records"]) == g["records"], case["name"]
        assert digest(want["out"]) == g["out"], case["name"]


def test_placement_heuristics_match_the_reference_solver_classes(built_lib):
    """The oracle's Intuitive / Rep / CliquePart solvers AND the library's own produce, array for
    array (nid_to_block, block_placement, block_access_from, block_density), what the reference's
    solver classes (coll_cache_lib/coll_cache/optimal_solver_class.cc:1251-1404, :1869-2058,
    compiled in place into oracle/_ref/ref_solver_pin) produced for the same seeded rankings;
    their digests are kept in tests/golden/ref_solver.json (made by tests/golden/make_solver_pin.py)."""
    import json
    import os
    import sys
    from ugache_b200 import runtime as rt
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, here)
    try:
        import make_solver_pin as pin
    finally:
        sys.path.remove(here)
    with open(os.path.join(here, "ref_solver.json")) as f:
        want = {c["name"]: c for c in json.load(f)["cases"]}
    assert len(want) == len(pin.CASES) >= 13
    for case in pin.CASES:
        name, policy, G, N, pct, alpha, tl, tr, tc = case
        assert pin.digest_placement(*pin.oracle_placement(case)) == want[name]["digest"], name
        ids, freqs = pin.ranking(name, N, alpha)
        p = rt.solve_placement(policy, G, ids, freqs, pct, t_local=tl, t_remote=tr, t_cpu=tc)
        ours = (p.nid_to_block, p.block_placement, np.asarray(p.block_access_from).reshape(G, -1), p.block_density)
        assert pin.digest_placement(*ours) == want[name]["digest"], ("library", name)

