"""Algorithm selection from measured timings.

The reference has no selection logic beyond a hard-coded table of batch limits by rank count and block size
(examples/twophaseLayer_example2.cpp:136-152) and sweeps of the batch parameter in its drivers
(examples/twophaseLayer_example.cpp:120-144, twophaseLayer_example2.cpp:96-191).  Here a table of measured
timings, keyed by (ranks, processes, message-size class, skew class), decides algorithm, group size, radix, batch
and protocol.  ``sweep`` fills the table on the machine at hand (batch and group size are swept too); ``choose``
reads it and falls back to the built-in rule.  Candidates are listed simplest first and a later candidate only
replaces the current winner when it is more than ``MARGIN`` faster, so that differences inside the measurement
noise never put an exotic schedule into the table.  The table is the only state the library persists (JSON
under ``$RBV_TUNER_CACHE`` or the package folder); the C API reads the same file (``csrc/api/tuner_native.cpp``).
"""
from __future__ import annotations

import json
import math
import os
from pathlib import Path
from typing import Dict, List, Optional

_TABLE: Optional[Dict[str, dict]] = None

# size classes by mean block bytes: class k covers [2^k, 2^(k+1))
def size_class(mean_block_bytes: float) -> int:
    return max(0, int(math.floor(math.log2(max(mean_block_bytes, 1.0)))))


def _cache_path() -> Path:
    p = os.environ.get("RBV_TUNER_CACHE")
    return Path(p) if p else Path(__file__).resolve().parent / "tuner_table.json"


MARGIN = 0.03          # a candidate must beat the current winner by more than this fraction to replace it ...
MIN_GAIN_US = 0.5      # ... and by more than this: CUDA event times on B200 come in steps of about one microsecond
MIN_STEPS = 30         # timed steps per candidate in a sweep
SKEW_CV = 0.5          # coefficient of variation of the block sizes from which an exchange counts as skewed


def skew_class(cv: float) -> int:
    """0: balanced (block sizes within about +-50 % of the mean), 1: skewed (Zipf-like, many empty blocks)."""
    return 1 if cv >= SKEW_CV else 0


def block_stats(counts, type_size: int = 1):
    """(mean block bytes, coefficient of variation) of a count matrix."""
    import numpy as np
    a = np.asarray(counts, dtype=np.float64).ravel() * type_size
    if a.size == 0 or a.mean() <= 0:
        return 0.0, 0.0
    return float(a.mean()), float(a.std() / a.mean())


def _key(P: int, nproc: int, cls: int, skew: int = 0) -> str:
    return f"P{P}-G{nproc}-c{cls}" + (f"-s{skew}" if skew else "")


def load_table() -> Dict[str, dict]:
    global _TABLE
    if _TABLE is None:
        _TABLE = {}
        path = _cache_path()
        if path.exists():
            try:
                _TABLE = json.loads(path.read_text())
            except Exception:
                _TABLE = {}
    return _TABLE


def save_table() -> None:
    path = _cache_path()
    tmp = path.with_suffix(".tmp")
    tmp.write_text(json.dumps(load_table(), indent=1, sort_keys=True))
    os.replace(tmp, path)


def record(P: int, nproc: int, mean_block_bytes: float, choice: dict, us: float, cv: float = 0.0,
           replace: bool = False) -> None:
    """Enters a measurement.  An existing entry is replaced only by one that is more than ``MARGIN`` faster
    (``replace=True``: unconditionally, for a fresh sweep whose winner was chosen by the same rule)."""
    tab = load_table()
    k = _key(P, nproc, size_class(mean_block_bytes), skew_class(cv))
    if replace or k not in tab or (us < tab[k]["us"] * (1.0 - MARGIN) and tab[k]["us"] - us > MIN_GAIN_US):
        tab[k] = {"choice": choice, "us": us}


def pick_winner(timings) -> tuple:
    """``timings``: (choice, microseconds) in order of preference, simplest first.  Returns the first entry that no
    later entry beats by more than ``MARGIN``: the simplest configuration within the margin of the best."""
    best = None
    for choice, us in timings:
        if us is None:
            continue
        if best is None or (us < best[1] * (1.0 - MARGIN) and best[1] - us > MIN_GAIN_US):
            best = (choice, us)
    return best


def robust_us(samples_ms) -> float:
    """Microseconds of one candidate from its per-step times: the mean of the fastest 80 % of the steps.  A median
    would sit on one of the timer's one-microsecond steps; the mean of many steps resolves finer differences, and
    dropping the slowest fifth keeps stragglers out."""
    import numpy as np
    t = np.sort(np.asarray(samples_ms, dtype=np.float64))
    keep = max(1, int(round(0.8 * len(t))))
    return float(t[:keep].mean()) * 1e3


def default_choice(P: int, nproc: int, mean_block_bytes: float) -> dict:
    """Built-in rule for configurations the table has no measurement for.  On a flat NVSwitch fabric every extra
    Bruck digit costs one more cross-GPU synchronisation and forwards data twice, so the single-hop spread-out
    order wins whenever ranks are on different GPUs; Bruck variants remain selectable explicitly.  Blocks up to
    64 KB go through the eager protocol (faster in every measured configuration: 1, 2, 4 and 8 GPUs), larger ones
    through rendezvous."""
    return {"algo": "spreadout", "protocol": "eager" if mean_block_bytes <= (64 << 10) else "rendezvous"}


def choose(P: int, nproc: int, mean_block_bytes: float, cv: float = 0.0) -> dict:
    """The table's entry for this size and skew class; neighbours (other skew class first, then the adjacent size
    classes) stand in for classes that were not measured; then the built-in rule."""
    tab = load_table()
    cls, sk = size_class(mean_block_bytes), skew_class(cv)
    for c in (cls, cls - 1, cls + 1):
        for s in (sk, 1 - sk):
            hit = tab.get(_key(P, nproc, c, s))
            if hit:
                return dict(hit["choice"])
    return default_choice(P, nproc, mean_block_bytes)


def _pow2_upto(limit: int) -> List[int]:
    out, b = [], 1
    while b < limit:
        out.append(b)
        b *= 2
    return out


def native_choose(P: int, nproc: int, mean_block_bytes: float, cv: float = 0.0, path=None) -> dict:
    """The same lookup done by the native reader that serves the C API (``csrc/api/tuner_native.cpp``), on the table
    file on disk (not on entries recorded in this process and not yet saved)."""
    from .. import _native
    from .plan import ALGOS
    lib = _native.host_lib()
    lib.rbv_tuner_set_table(str(path or _cache_path()).encode())
    ch = _native.Choice()
    lib.rbv_tuner_choose(P, nproc, float(mean_block_bytes), float(cv), ch)
    out = {"algo": ALGOS[ch.algo], "protocol": "eager" if ch.eager else "rendezvous"}
    for k in ("n", "r", "r2", "b", "b2"):
        out[k] = int(getattr(ch, k))
    return out


def candidates(P: int, groups: Optional[List[int]] = None, full: bool = True) -> List[dict]:
    """The configurations a sweep tries, simplest first (single hop, then flat Bruck by decreasing radix, then the
    two-layer schedules).  Batch parameters run over 1, 2, 4, ... like the reference's drivers sweep them
    (0 = everything in flight at once); ``full=False`` keeps one batch value per schedule."""
    out: List[dict] = [{"algo": "spreadout"}, {"algo": "linear"}, {"algo": "pairwise"}]
    if P & (P - 1) == 0:
        out.append({"algo": "xor"})
    for b in (_pow2_upto(P) if full else [max(1, P // 2)]):
        out.append({"algo": "scattered", "b": b})
    for r in sorted({2, 3, 4, P}, reverse=True):
        if 2 <= r <= P:
            out.append({"algo": "rbruck", "r": r})
            rt = min(r, max(2, P - 1))
            for b in ([0] + _pow2_upto(rt - 1) if full else [0]):
                out.append({"algo": "tuna2", "r": rt, "b": b})
    for n in (groups or [g for g in (2, 4, 8, 16) if P % g == 0 and g < P]):
        G = P // n
        for b in ([0] + _pow2_upto(P) if full else [0]):
            out.append({"algo": "ttpl_bt_s1", "n": n, "r": 2, "b": b})
        for b in ([0] + _pow2_upto(G) if full else [0]):
            out.append({"algo": "ttpl_bt", "n": n, "r": 2, "b": b})
    seen, uniq = set(), []
    for c in out:
        k = tuple(sorted(c.items()))
        if k not in seen:
            seen.add(k)
            uniq.append(c)
    return uniq


def sweep(comm, mean_block_bytes=(16, 256, 4096, 65536, 1 << 20, 4 << 20), type_size: int = 2, skew: str = "normal",
          steps: int = MIN_STEPS, warmup: int = 3, seed: int = 0, groups=None, verbose: bool = True,
          full: bool = True) -> List[dict]:
    """Times every candidate (both protocols where the blocks fit the eager cells) for each size class on
    ``comm`` and records the winners in the table: at least ``MIN_STEPS`` timed steps per candidate, median, and
    the simplest candidate within ``MARGIN`` of the best wins (:func:`pick_winner`).  Collective: every process of
    the communicator calls it."""
    steps = max(int(steps), MIN_STEPS)
    import numpy as np
    import torch

    from ..utils import distributions as D
    from ..utils.timing import L2Flusher, RankAligner, time_steps

    dev = f"cuda:{comm.device}"
    flush, align = L2Flusher(dev), RankAligner(comm)
    L, P, mine = comm.L, comm.P, comm.local_ranks
    rows = []
    for nbytes in mean_block_bytes:
        elems = max(1, nbytes // type_size)
        counts = D.zipf(P, 4 * elems, seed=seed) if skew == "zipf" else D.normal(P, elems, 0.25, seed=seed)
        sc = counts[mine].astype(np.int32)
        rc = counts.T[mine].astype(np.int32)
        send = [torch.zeros(max(int(sc[i].sum()), 1) * type_size, dtype=torch.uint8, device=dev) for i in range(L)]
        recv = [comm.symm_empty(max(int(rc[i].sum()), 1) * type_size, torch.uint8) for i in range(L)]
        emax = comm.max_block_bytes(sc, type_size)
        cell_room = comm.arena_bytes // (2 * max(emax, 8) + 16)
        mean_b, cv = block_stats(counts, type_size)
        row = {"mean_block_bytes": nbytes, "skew": skew, "cv": round(cv, 3), "max_block_bytes": emax, "us": {}}
        timings = []
        for cand in candidates(P, groups, full):
            for eager in (True, False):
                kw = dict(cand)
                if eager:
                    if emax > (256 << 10) or cell_room < P + 64:
                        continue
                    kw["eager_max_bytes"] = emax
                name = "/".join(f"{k}={v}" for k, v in kw.items() if k != "eager_max_bytes") + ("/eager" if eager else "")
                try:
                    call = comm.prepare(send, recv, sc, None, rc, None, type_size=type_size, **kw)
                except Exception:
                    row["us"][name] = None
                    continue
                t = time_steps(call.launch, steps, warmup, flush=flush, align=align)
                if comm.status()["code"]:
                    comm.reset()
                    row["us"][name] = None
                    continue
                us = robust_us(t)
                row["us"][name] = round(us, 2)
                timings.append((dict(cand, protocol="eager" if eager else "rendezvous"), us))
        win = pick_winner(timings)
        if win is not None:
            record(P, comm.nproc, mean_b, win[0], win[1], cv=cv, replace=True)
            row["best"] = win[0]
            row["best_us"] = round(win[1], 2)
            row["fastest_us"] = round(min(u for _, u in timings), 2)
        rows.append(row)
        if verbose and comm.proc == 0:
            print(json.dumps(row), flush=True)
        del send, recv
    return rows
