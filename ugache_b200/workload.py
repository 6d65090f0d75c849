"""Seeded synthetic inputs with the shapes and skew of the reference's workloads.

The reference measures on Criteo-TB, a synthetic Zipf DLR set and large graphs; none of those
datasets is available offline, so these generators stand in for them:

* table:  value(row, col) uniform in [-1, 1) from a counter-based generator keyed by
          (seed, row*dim + col), so any row can be regenerated on demand;
* keys:   Zipf ranks through the bounded-Pareto inverse CDF the reference's generator uses
          (eval/dlr/common/ds_generator.py:11-15 called with alpha-1,
          datagen/dlr/syn.py:43), mapped to ids by a fixed bijection on [0, N);
* hotness for the placement: the analytic rank order (frequency ~ rank^-alpha).
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return x ^ (x >> np.uint64(31))


def table_rows(seed, rows, dim, dtype=np.float32):
    """Rows `rows` (int array) of the synthetic table, shape [len(rows), dim]."""
    rows = np.asarray(rows, dtype=np.uint64)
    with np.errstate(over="ignore"):
        e = rows[:, None] * np.uint64(dim) + np.arange(dim, dtype=np.uint64)[None, :]
        x = _splitmix64(np.uint64(seed) ^ _splitmix64(e))
    if np.dtype(dtype) == np.float32:
        return ((x >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 8388608.0)
                - np.float32(1.0))
    v = (x >> np.uint64(53)).astype(np.int64) - 1024
    return (v.astype(np.float32) * np.float32(1.0 / 1024.0)).astype(np.float16)


def table(seed, n_rows, dim, dtype=np.float32, row_begin=0):
    return table_rows(seed, np.arange(row_begin, row_begin + n_rows), dim, dtype)


def zipf_ranks(u, N, alpha):
    """Zero-based Zipf ranks for uniform draws u in [0, 1)."""
    a = alpha - 1.0
    H = float(N)
    if abs(a) < 1e-12:
        x = np.power(H, u)
    else:
        Ha = H ** a
        x = np.power((-Ha) / (u * (Ha - 1.0) - Ha), 1.0 / a)
    r = x.astype(np.int64) - 1
    return np.clip(r, 0, N - 1)


def bijection(N):
    """(A, B) of the rank -> id map id = (A*rank + B) mod N with gcd(A, N) = 1."""
    A = 2654435761 % N
    if A < 2:
        A = 1
    while np.gcd(A, N) != 1:
        A += 1
    return int(A), int(12345 % N)


def rank_to_id(rank0, N):
    A, B = bijection(N)
    return ((np.asarray(rank0).astype(object) * A + B) % N).astype(np.int64) if N > (1 << 31) \
        else ((np.asarray(rank0, dtype=np.uint64) * np.uint64(A) + np.uint64(B))
              % np.uint64(N)).astype(np.int64)


def zipf_keys(seed, n, N, alpha):
    """n int64 ids, Zipf(alpha) over one hashed id space of N rows, not deduplicated."""
    u = np.random.Generator(np.random.Philox(seed)).random(n)
    return rank_to_id(zipf_ranks(u, N, alpha), N)


def analytic_hotness(N, alpha, top=4.0e9):
    """(rank_ids, rank_freqs): ids by descending expected frequency and 32-bit integer
    counts proportional to rank^-alpha, the input the placement solvers take.  The hottest id
    gets `top` counts (close to the 32-bit ceiling) so that the tail keeps non-zero counts as
    far down as the integer format allows."""
    ranks = np.arange(N, dtype=np.uint64)
    ids = rank_to_id(ranks, N).astype(np.uint32)
    w = (np.arange(1, N + 1, dtype=np.float64)) ** (-alpha)
    freqs = np.floor(w * top).astype(np.uint32)
    return ids, freqs


class Workload:
    """A small seeded case: table, hotness, placement (through `solver`) and key batches."""

    def __init__(self, N, dim, dtype, G, pct, alpha, n_keys, policy, seed, dedup=False,
                 solver=None, table_array=None):
        self.N, self.dim, self.G, self.pct = N, dim, G, pct
        self.dtype = np.dtype(dtype)
        self.alpha, self.n_keys, self.policy, self.seed, self.dedup = alpha, n_keys, policy, seed, dedup
        self.row_bytes = dim * self.dtype.itemsize
        # large cases hand in the rows from a faster generator with the same definition
        self.table = table(seed, N, dim, self.dtype) if table_array is None else table_array
        self.rank_ids, self.rank_freqs = analytic_hotness(N, alpha)
        self.capacity = int(N * (pct + 0.001))
        if solver is None:
            from . import runtime
            solver = runtime.solve_placement
        self.placement = solver(policy, G, self.rank_ids, self.rank_freqs, pct * 100.0)

    def keys(self, rank=0, it=0):
        k = zipf_keys(self.seed * 1000003 + rank * 1009 + it, self.n_keys, self.N, self.alpha)
        if self.dedup:
            k = np.unique(k)
        return k
