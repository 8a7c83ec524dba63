"""Tuner table logic (no GPU)."""
import json

import pytest

from rbruck_alltoallv_b200.parallel import tuner


def test_choose_falls_back_and_reads_table(tmp_path, monkeypatch):
    monkeypatch.setenv("RBV_TUNER_CACHE", str(tmp_path / "t.json"))
    tuner._TABLE = None
    assert tuner.choose(8, 8, 1000)["algo"] == "spreadout"
    tuner.record(8, 8, 1000, {"algo": "rbruck", "r": 2, "protocol": "eager"}, 12.0)
    tuner.record(8, 8, 1000, {"algo": "tuna2", "r": 2}, 15.0)      # slower: must not replace the entry
    assert tuner.choose(8, 8, 1000) == {"algo": "rbruck", "r": 2, "protocol": "eager"}
    assert tuner.choose(8, 8, 600)["algo"] == "rbruck"               # neighbouring size class
    tuner.save_table()
    tuner._TABLE = None
    assert json.loads((tmp_path / "t.json").read_text())["P8-G8-c9"]["us"] == 12.0
    assert tuner.choose(8, 8, 1000)["algo"] == "rbruck"
    tuner._TABLE = None


def test_candidates_are_valid_plans():
    from rbruck_alltoallv_b200 import Plan
    for P in (2, 4, 6, 8, 16):
        for c in tuner.candidates(P):
            kw = {k: v for k, v in c.items() if k != "algo"}
            assert Plan(c["algo"], P, **kw).err == 0, (P, c)


def test_size_class():
    assert tuner.size_class(1) == 0 and tuner.size_class(1024) == 10 and tuner.size_class(1500) == 10


def test_environment_overrides_take_precedence(monkeypatch):
    """RBV_ALGO / RBV_RADIX / RBV_PROTOCOL win over the tuner table in automatic calls (no GPU needed: the
    choice is resolved against a stand-in communicator)."""
    from types import SimpleNamespace

    import numpy as np
    import torch

    from rbruck_alltoallv_b200.ops import alltoallv as A

    comm = SimpleNamespace(P=8, L=8, nproc=1, arena_bytes=8 << 20, max_block_bytes=lambda sc, ts: int(np.max(sc)) * ts)
    recv = [torch.empty(4, dtype=torch.float32)]
    sc = np.full((8, 8), 100, dtype=np.int32)
    for var in ("RBV_ALGO", "RBV_RADIX", "RBV_BATCH", "RBV_GROUP", "RBV_PROTOCOL"):
        monkeypatch.delenv(var, raising=False)
    base = A._auto_choice(comm, recv, sc, {}, agree_on_max=True)
    assert "algo" in base
    monkeypatch.setenv("RBV_ALGO", "tuna2")
    monkeypatch.setenv("RBV_RADIX", "3")
    monkeypatch.setenv("RBV_BATCH", "2")
    monkeypatch.setenv("RBV_PROTOCOL", "rendezvous")
    got = A._auto_choice(comm, recv, sc, {}, agree_on_max=True)
    assert got["algo"] == "tuna2" and got["r"] == 3 and got["b"] == 2 and "eager_max_bytes" not in got
    monkeypatch.setenv("RBV_PROTOCOL", "eager")
    got = A._auto_choice(comm, recv, sc, {}, agree_on_max=True)
    assert got["eager_max_bytes"] == 400
    # a keyword given by the caller still wins over the environment
    got = A._auto_choice(comm, recv, sc, {"r": 4}, agree_on_max=True)
    assert got["r"] == 4
    monkeypatch.setenv("RBV_PROTOCOL", "carrier-pigeon")
    with pytest.raises(ValueError):
        A._auto_choice(comm, recv, sc, {}, agree_on_max=True)


def test_default_choice_for_unmeasured_configurations():
    small = tuner.default_choice(16, 16, 1024)
    large = tuner.default_choice(16, 16, 4 << 20)
    assert small == {"algo": "spreadout", "protocol": "eager"}
    assert large == {"algo": "spreadout", "protocol": "rendezvous"}
