"""Seeded count-matrix generators.

Every generator returns a ``P x P`` ``int64`` matrix ``C`` with ``C[s, d]`` = number of elements rank
``s`` sends to rank ``d``.  All are deterministic in ``seed`` (the reference seeds from the wall clock or
``std::random_device``, e.g. examples/twophaseLayer_example.cpp:59-67, examples/other_distributions.cpp:70-71,
so its runs cannot be repeated).

Reference drivers whose patterns are reproduced: examples/rbruckv_example.cpp:58-66 (constant, shuffled),
examples/twophaseLayer_example.cpp:58-67 (uniform random), examples/other_distributions.cpp:69-104 (normal,
power law), examples/FFT_distribution.cpp:66-87 (FFT-like), examples/balanced_benchmark.cpp:58-63,123-128,
examples/MLinputs_example.cpp:119-145 (matrix file).
"""
from __future__ import annotations

from pathlib import Path

import numpy as np


def _rng(seed: int) -> np.random.Generator:
    return np.random.default_rng(np.random.SeedSequence(int(seed)))


def constant(P: int, n: int, seed: int = 0) -> np.ndarray:
    return np.full((P, P), int(n), dtype=np.int64)


def uniform(P: int, hi: int, seed: int = 0, lo: int = 0) -> np.ndarray:
    """Counts uniform in [lo, hi] (inclusive)."""
    return _rng(seed).integers(lo, hi + 1, size=(P, P), dtype=np.int64)


def uniform_fraction(P: int, n: int, seed: int = 0) -> np.ndarray:
    """``n * (k % 100) / 100`` with random k, shuffled per row: the reference's default random pattern."""
    k = _rng(seed).integers(0, 100, size=(P, P))
    return (int(n) * k // 100).astype(np.int64)


def zipf(P: int, max_elems: int, s: float = 1.2, zero_frac: float = 0.10, seed: int = 0) -> np.ndarray:
    """Zipf-skewed block sizes: size = max_elems / k**s with k a random rank in 1..P*P, then a fraction
    ``zero_frac`` of the blocks set to zero."""
    rng = _rng(seed)
    ranks = rng.permutation(P * P) + 1
    sizes = np.floor(max_elems / ranks.astype(np.float64) ** s).astype(np.int64)
    sizes = np.maximum(sizes, 1)
    zero = rng.random(P * P) < zero_frac
    sizes[zero] = 0
    return sizes.reshape(P, P)


def normal(P: int, mean: float, sd_frac: float = 0.25, seed: int = 0, max_value: int | None = None) -> np.ndarray:
    """Normal(mean, sd_frac*mean), clipped at 0 (and at ``max_value`` when given)."""
    v = _rng(seed).normal(mean, sd_frac * mean, size=(P, P))
    v = np.clip(np.rint(v), 0, max_value if max_value is not None else None)
    return v.astype(np.int64)


def power_law(P: int, max_value: int, x: float, seed: int = 0) -> np.ndarray:
    """``max_value * x**i`` for i = 0..P-1, shuffled per sender."""
    rng = _rng(seed)
    base = (max_value * np.power(float(x), np.arange(P))).astype(np.int64)
    return np.stack([rng.permutation(base) for _ in range(P)])


def jitter(P: int, n: int, frac: float = 0.05, seed: int = 0) -> np.ndarray:
    """Near-balanced counts: n * (1 + U[-frac, frac])."""
    u = _rng(seed).uniform(-frac, frac, size=(P, P))
    return np.rint(n * (1.0 + u)).astype(np.int64)


def fft_pattern(P: int, number: int, xzero: float = 0.0, yzero: float = 0.0, last: int = 0) -> np.ndarray:
    """The two count patterns of the reference's FFT driver (no FFT is computed there)."""
    Cm = np.zeros((P, P), dtype=np.int64)
    if last == 0:
        rows = int((1.0 - yzero) * P)
        cols = int((1.0 - xzero) * P)
        Cm[:rows, :cols] = number
    else:
        Cm[:, :] = number
        Cm[:, P - 1] = last
    return Cm


def sparse_groups(P: int, n: int, ncores: int, transpose: bool = False) -> np.ndarray:
    """Send only to ranks whose index is a multiple of ``ncores`` (or the transposed pattern)."""
    Cm = np.zeros((P, P), dtype=np.int64)
    Cm[:, ::ncores] = n
    return Cm.T.copy() if transpose else Cm


def leaders_only(P: int, n: int, ncores: int) -> np.ndarray:
    """Only the first rank of every group of ``ncores`` talks, to the other groups' first ranks, ``n`` elements each:
    the second pattern of the reference's gather driver (examples/gather_benchmark.cpp:120-125)."""
    Cm = np.zeros((P, P), dtype=np.int64)
    idx = np.arange(0, P, max(ncores, 1))
    Cm[np.ix_(idx, idx)] = n
    return Cm


def merge_pattern(P: int, csize: int, lsize: int, ncores: int) -> np.ndarray:
    """Small blocks of ``csize`` elements everywhere, large blocks of ``lsize`` between the first ranks of the groups
    of ``ncores``: the setting the reference's merge_alltoallv is written for (local rank 0 carries the large
    messages and stays out of the merge, benchmarks/merge_benchmark.cpp:155-332)."""
    Cm = np.full((P, P), csize, dtype=np.int64)
    idx = np.arange(0, P, max(ncores, 1))
    Cm[np.ix_(idx, idx)] = lsize
    return Cm


def read_matrix(path: str | Path) -> np.ndarray:
    """A whitespace-separated P x P byte-count matrix; row r holds rank r's send counts."""
    vals = np.loadtxt(str(path), dtype=np.int64, ndmin=2)
    if vals.shape[0] != vals.shape[1]:
        flat = vals.reshape(-1)
        P = int(round(flat.size ** 0.5))
        if P * P != flat.size:
            raise ValueError(f"{path}: {flat.size} values do not form a square matrix")
        vals = flat.reshape(P, P)
    return vals


def write_matrix(path: str | Path, Cm: np.ndarray) -> None:
    np.savetxt(str(path), np.asarray(Cm, dtype=np.int64), fmt="%d")


def synthetic_ml_trace(P: int, seed: int = 0, mean_bytes: float = 29.1e6, zero_diag: bool = True,
                       zero_frac: float = 0.0) -> np.ndarray:
    """A heavy-tailed byte matrix shaped like the recorded all-to-all traces that ship with the reference
    (zero diagonal, log-normal skew); used when the trace files are not at hand."""
    rng = _rng(seed)
    v = rng.lognormal(mean=0.0, sigma=1.0, size=(P, P))
    v = v / v.mean() * mean_bytes
    if zero_frac > 0:
        v[rng.random((P, P)) < zero_frac] = 0
    if zero_diag:
        np.fill_diagonal(v, 0)
    return v.astype(np.int64)


def by_name(name: str, P: int, seed: int = 0, **kw) -> np.ndarray:
    table = {
        "constant": lambda: constant(P, kw.get("n", 256), seed),
        "uniform": lambda: uniform(P, kw.get("hi", 256), seed),
        "uniform_fraction": lambda: uniform_fraction(P, kw.get("n", 256), seed),
        "zipf": lambda: zipf(P, kw.get("max_elems", 16384), kw.get("s", 1.2), kw.get("zero_frac", 0.10), seed),
        "normal": lambda: normal(P, kw.get("mean", 1024), kw.get("sd_frac", 0.25), seed),
        "power_law": lambda: power_law(P, kw.get("max_value", 4096), kw.get("x", 0.9), seed),
        "jitter": lambda: jitter(P, kw.get("n", 1024), kw.get("frac", 0.05), seed),
    }
    return table[name]()
