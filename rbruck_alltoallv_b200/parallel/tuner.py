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
    """Built-in rule: on a flat NVSwitch fabric every extra Bruck digit costs one more cross-GPU
    synchronisation and forwards data twice, so the single-hop spread-out order wins whenever ranks are
    on different GPUs; Bruck variants remain selectable explicitly."""
    return {"algo": "spreadout"}


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
