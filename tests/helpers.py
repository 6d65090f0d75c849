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
