import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def built_lib():
    """The in-tree CUDA library, compiled on demand (nvcc cross-compiles without a GPU)."""
    from ugache_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def ref_pin():
    with open(os.path.join(GOLDEN, "ref_pin.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def golden_cases():
    with open(os.path.join(GOLDEN, "cases.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def golden_cases_large():
    """Cases at the sizes the benchmark configurations name (tests/golden/make_golden.py)."""
    with open(os.path.join(GOLDEN, "cases_large.json")) as f:
        return json.load(f)


def oracle_solver(policy, G, rank_ids, rank_freqs, cache_percent):
    """Placement through the oracle's restatement of the reference heuristics."""
    from oracle import oracle as orc
    if policy == "intuitive":
        return orc.solve_intuitive(G, rank_ids, rank_freqs, cache_percent, 1.0, 8000.0 / 900.0,
                                   8000.0 / 64.0)
    if policy == "rep":
        return orc.solve_rep(G, rank_ids, cache_percent)
    return orc.solve_clique_part(G, rank_ids, cache_percent)
