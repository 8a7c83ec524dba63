"""Direct-copy oracle and test-problem construction.

The reference's own self check (src/utils.cpp:31-46) only verifies that a received value is non-zero and
that ``value % 10 == rank % 10``; a permutation of equally sized source blocks passes it.  Here the
expected receive buffer is built byte by byte and compared exactly, with canary bytes in every gap and
behind the last block.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

CANARY = 0xA5


@dataclass
class Problem:
    P: int
    type_size: int
    counts: np.ndarray      # [P, P] elements, counts[s, d]
    sdispls: np.ndarray     # [P, P] elements, rank s's send displacements
    rdispls: np.ndarray     # [P, P] elements, rank d's receive displacements, rdispls[d, s]
    send_bytes: np.ndarray  # [P] send buffer sizes in bytes
    recv_bytes: np.ndarray  # [P] receive buffer sizes in bytes

    @property
    def recvcounts(self) -> np.ndarray:
        return self.counts.T.copy()


def _layout(sizes: np.ndarray, rng, packed: bool, max_gap: int):
    """Displacements (elements) for one rank's blocks: packed rank order, or shuffled with holes."""
    P = sizes.shape[0]
    disp = np.zeros(P, dtype=np.int64)
    order = np.arange(P) if packed else rng.permutation(P)
    cur = 0 if packed else int(rng.integers(0, max_gap + 1))
    for i in order:
        disp[i] = cur
        cur += int(sizes[i]) + (0 if packed else int(rng.integers(0, max_gap + 1)))
    return disp, cur


def make_problem(counts: np.ndarray, type_size: int, seed: int = 0, packed: bool = True,
                 max_gap: int = 3) -> Problem:
    counts = np.asarray(counts, dtype=np.int64)
    P = counts.shape[0]
    rng = np.random.default_rng(seed + 7919)
    sd = np.zeros((P, P), dtype=np.int64)
    rd = np.zeros((P, P), dtype=np.int64)
    sb = np.zeros(P, dtype=np.int64)
    rb = np.zeros(P, dtype=np.int64)
    for r in range(P):
        sd[r], tot = _layout(counts[r], rng, packed, max_gap)
        sb[r] = tot * type_size
        rd[r], tot = _layout(counts[:, r], rng, packed, max_gap)
        rb[r] = tot * type_size
    return Problem(P, type_size, counts, sd, rd, sb, rb)


def fill_send(prob: Problem, seed: int = 0):
    """Send buffers with position-dependent pseudo-random bytes (every byte identifies its place)."""
    bufs = []
    for s in range(prob.P):
        rng = np.random.default_rng(seed * 1000003 + s)
        bufs.append(rng.integers(0, 256, size=max(int(prob.send_bytes[s]), 1), dtype=np.uint8))
    return bufs


def empty_recv(prob: Problem, tail: int = 64):
    return [np.full(int(prob.recv_bytes[d]) + tail, CANARY, dtype=np.uint8) for d in range(prob.P)]


def expected_recv(prob: Problem, sendbufs, tail: int = 64):
    ts = prob.type_size
    out = empty_recv(prob, tail)
    for d in range(prob.P):
        for s in range(prob.P):
            n = int(prob.counts[s, d]) * ts
            if n:
                so = int(prob.sdispls[s, d]) * ts
                ro = int(prob.rdispls[d, s]) * ts
                out[d][ro:ro + n] = sendbufs[s][so:so + n]
    return out


def first_mismatch(got, want):
    """``None`` when all buffers agree, else ``(rank, byte offset)`` of the first difference."""
    for d, (g, w) in enumerate(zip(got, want)):
        g = np.asarray(g).reshape(-1)
        w = np.asarray(w).reshape(-1)
        if g.shape != w.shape:
            return (d, -1)
        bad = np.nonzero(g != w)[0]
        if bad.size:
            return (d, int(bad[0]))
    return None


def reference_value_fill(prob: Problem):
    """The reference drivers' payload: element i-block of sender s holds ``dest + 10 * s``
    (examples/rbruckv_example.cpp:88-92); 8-byte elements."""
    assert prob.type_size == 8
    bufs = []
    for s in range(prob.P):
        b = np.zeros(max(int(prob.send_bytes[s]) // 8, 1), dtype=np.int64)
        for d in range(prob.P):
            o, n = int(prob.sdispls[s, d]), int(prob.counts[s, d])
            b[o:o + n] = d + 10 * s
        bufs.append(b.view(np.uint8))
    return bufs


def check_errors(recvcounts, recv_buffer, rank: int, nprocs: int) -> int:
    """Same rule as the reference's ``check_errors`` (src/utils.cpp:31-46) on a packed receive buffer."""
    errors = 0
    idx = 0
    vals = np.asarray(recv_buffer).view(np.int64)
    for p in range(nprocs):
        n = int(recvcounts[p])
        seg = vals[idx:idx + n]
        if p != 0 or rank != 0:
            errors += int(np.count_nonzero(seg == 0))
        errors += int(np.count_nonzero((seg % 10) != (rank % 10)))
        idx += n
    return errors
