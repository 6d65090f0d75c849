"""Writes tests/golden/ref_extract.json: digests of what the REFERENCE's own extraction device
code produced for the cases of ``tests.helpers.REF_EXTRACT_CASES``.

Needs a GPU and ``oracle/_ref/ref_extract_pin`` (``make -C oracle ref`` where the reference
tree is available): the reference's table lookup with its record helper, its radix-sort
grouping, its boundary kernel and its ``extract_data`` row-copy kernel, run in the order its
extraction session runs them.  Inputs are built from the oracle's cache model; the file keeps,
per case, the SHA-256 of the output bytes and of the sorted records, and the group boundaries,
so the CPU test-suite can hold the oracle to them without the reference.  The ``fill_*``
entries are the same for the reference's build fill and refresh scatter (REF_FILL_CASES).

    python tests/golden/make_ref_extract.py [out.json]

The committed file was produced on a B200."""
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402
from tests.conftest import oracle_solver  # noqa: E402
from tests.helpers import (REF_EXTRACT_CASES, REF_FILL_CASES, digest, ref_extract_case,  # noqa: E402
                           ref_fill_case)
from tests.test_gpu_refpin import REF_EXTRACT, run_ref_extract, run_ref_fill  # noqa: E402


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_extract.json")
    res = {}
    for case in REF_EXTRACT_CASES:
        blob, _ = ref_extract_case(orc, oracle_solver, case)
        with tempfile.TemporaryDirectory() as d:
            got = run_ref_extract(REF_EXTRACT, d, blob)
        res[case["name"]] = dict(out=digest(got["out"]), records=digest(got["records"]),
                                 groups=[int(x) for x in got["groups"]])
    for case in REF_FILL_CASES:
        blob, _ = ref_fill_case(orc, case)
        with tempfile.TemporaryDirectory() as d:
            res["fill_" + case["name"]] = dict(slice=digest(run_ref_fill(REF_EXTRACT, d, blob)))
    with open(out_path, "w") as f:
        json.dump(res, f, indent=1, sort_keys=True)
    print("wrote", out_path, len(res), "cases")


if __name__ == "__main__":
    main()
