"""Algorithm selection from measured timings.

The reference has no selection logic beyond a hard-coded table of batch limits by rank count
(examples/twophaseLayer_example2.cpp:136-152).  Here a table of measured timings, keyed by
(ranks, processes, message-size class), decides algorithm, radix and batch.  ``sweep`` fills the table on
the machine at hand; ``choose`` reads it and falls back to the built-in defaults measured on 8 x B200.
The table is the only state the library persists (JSON under ``$RBV_TUNER_CACHE`` or the package folder).
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


def _key(P: int, nproc: int, cls: int) -> str:
    return f"P{P}-G{nproc}-c{cls}"


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


def record(P: int, nproc: int, mean_block_bytes: float, choice: dict, us: float) -> None:
    tab = load_table()
    k = _key(P, nproc, size_class(mean_block_bytes))
    if k not in tab or us < tab[k]["us"]:
        tab[k] = {"choice": choice, "us": us}


def default_choice(P: int, nproc: int, mean_block_bytes: float) -> dict:
    """Built-in rule for configurations the table has no measurement for.  On a flat NVSwitch fabric every extra
    Bruck digit costs one more cross-GPU synchronisation and forwards data twice, so the single-hop spread-out
    order wins whenever ranks are on different GPUs; Bruck variants remain selectable explicitly.  Blocks up to
    64 KB go through the eager protocol (faster in every measured configuration: 1, 2, 4 and 8 GPUs), larger ones
    through rendezvous."""
    return {"algo": "spreadout", "protocol": "eager" if mean_block_bytes <= (64 << 10) else "rendezvous"}


def choose(P: int, nproc: int, mean_block_bytes: float) -> dict:
    tab = load_table()
    cls = size_class(mean_block_bytes)
    for c in (cls, cls - 1, cls + 1):
        hit = tab.get(_key(P, nproc, c))
        if hit:
            return dict(hit["choice"])
    return default_choice(P, nproc, mean_block_bytes)


def candidates(P: int, groups: Optional[List[int]] = None) -> List[dict]:
    """The configurations a sweep tries."""
    out: List[dict] = [{"algo": "spreadout"}, {"algo": "linear"}, {"algo": "pairwise"},
                       {"algo": "scattered", "b": max(1, P // 2)}]
    if P & (P - 1) == 0:
        out.append({"algo": "xor"})
    for r in sorted({2, 3, 4, P}):
        if 2 <= r <= P:
            out.append({"algo": "rbruck", "r": r})
            out.append({"algo": "tuna2", "r": min(r, max(2, P - 1)), "b": 0})
    for n in (groups or [g for g in (2, 4) if P % g == 0 and g < P]):
        out.append({"algo": "ttpl_bt_s1", "n": n, "r": 2, "b": 0})
        out.append({"algo": "ttpl_bt", "n": n, "r": 2, "b": 0})
    return out


def sweep(comm, mean_block_bytes=(16, 256, 4096, 65536, 1 << 20, 4 << 20), type_size: int = 2, skew: str = "normal",
          steps: int = 10, warmup: int = 3, seed: int = 0, groups=None, verbose: bool = True) -> List[dict]:
    """Times every candidate (both protocols where the blocks fit the eager cells) for each size class on
    ``comm`` and records the winners in the table.  Collective: every process of the communicator calls it."""
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
        row = {"mean_block_bytes": nbytes, "skew": skew, "max_block_bytes": emax, "us": {}}
        best, best_us = None, float("inf")
        for cand in candidates(P, groups):
            for eager in (False, True):
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
                us = float(np.median(t)) * 1e3
                row["us"][name] = round(us, 2)
                if us < best_us:
                    best, best_us = dict(cand, protocol="eager" if eager else "rendezvous"), us
        if best is not None:
            record(P, comm.nproc, nbytes, best, best_us)
            row["best"] = best
            row["best_us"] = round(best_us, 2)
        rows.append(row)
        if verbose and comm.proc == 0:
            print(json.dumps(row), flush=True)
        del send, recv
    return rows
