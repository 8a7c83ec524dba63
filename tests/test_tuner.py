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


def test_margin_keeps_the_simplest_candidate_within_three_percent():
    t = [({"algo": "spreadout"}, 22.50), ({"algo": "xor"}, 22.40), ({"algo": "ttpl_bt", "n": 4}, 22.10),
         ({"algo": "rbruck", "r": 2}, 30.0)]
    assert tuner.pick_winner(t)[0] == {"algo": "spreadout"}          # nobody is more than 3 % faster than the first
    t.append(({"algo": "scattered", "b": 4}, 21.0))                      # 6.7 % and 1.5 us faster: a real difference
    assert tuner.pick_winner(t)[0] == {"algo": "scattered", "b": 4}
    # 4 % faster but less than half a microsecond: below what the event timer resolves
    assert tuner.pick_winner([({"algo": "spreadout"}, 10.0), ({"algo": "xor"}, 9.6)])[0] == {"algo": "spreadout"}
    assert abs(tuner.robust_us([0.010, 0.010, 0.011, 0.010, 0.050]) - 10.25) < 1e-6
    assert tuner.pick_winner([({"algo": "a"}, None)]) is None


def test_skew_class_is_part_of_the_key(tmp_path, monkeypatch):
    import numpy as np
    from rbruck_alltoallv_b200.utils import distributions as D
    monkeypatch.setenv("RBV_TUNER_CACHE", str(tmp_path / "t.json"))
    tuner._TABLE = None
    mean_n, cv_n = tuner.block_stats(D.normal(8, 2048, 0.25, seed=1), 2)
    mean_z, cv_z = tuner.block_stats(D.zipf(8, 16384, seed=1), 4)
    assert tuner.skew_class(cv_n) == 0 and tuner.skew_class(cv_z) == 1
    tuner.record(8, 8, 4096, {"algo": "spreadout", "protocol": "eager"}, 15.0, cv=cv_n)
    tuner.record(8, 8, 4096, {"algo": "ttpl_bt_s1", "n": 4, "r": 2, "b": 2, "protocol": "rendezvous"}, 14.0, cv=cv_z)
    assert tuner.choose(8, 8, 4096, cv_n)["algo"] == "spreadout"
    assert tuner.choose(8, 8, 4096, cv_z)["algo"] == "ttpl_bt_s1"
    # an entry is replaced only by one that is more than the margin faster
    tuner.record(8, 8, 4096, {"algo": "xor", "protocol": "eager"}, 14.8, cv=cv_n)
    assert tuner.choose(8, 8, 4096, cv_n)["algo"] == "spreadout"
    tuner.record(8, 8, 4096, {"algo": "xor", "protocol": "eager"}, 13.0, cv=cv_n)
    assert tuner.choose(8, 8, 4096, cv_n)["algo"] == "xor"
    # a class without an entry of its own borrows the other skew class, then the neighbouring sizes
    tuner.record(4, 4, 1 << 20, {"algo": "pairwise", "protocol": "rendezvous"}, 30.0)
    assert tuner.choose(4, 4, 1 << 20, 0.9)["algo"] == "pairwise"
    assert tuner.choose(4, 4, 1 << 21, 0.9)["algo"] == "pairwise"
    # the native reader behind the C API's automatic entry points answers the same from the saved file
    tuner.save_table()
    for args in ((8, 8, 4096, cv_n), (8, 8, 4096, cv_z), (4, 4, 1 << 21, 0.9), (8, 8, 5000, 0.1), (16, 16, 100, 0.0),
                 (16, 16, 1 << 22, 0.0)):
        py, nat = tuner.choose(*args), tuner.native_choose(*args)
        assert nat["algo"] == py["algo"] and nat["protocol"] == py.get("protocol", "rendezvous"), (args, py, nat)
        for k in ("n", "r", "b", "b2"):
            if k in py:
                assert nat[k] == py[k]
    tuner._TABLE = None


def test_sweep_candidates_cover_batches_and_groupings():
    c8 = tuner.candidates(8)
    assert c8[0] == {"algo": "spreadout"}                                   # simplest first
    assert {c["b"] for c in c8 if c["algo"] == "scattered"} == {1, 2, 4}
    assert {c["n"] for c in c8 if c["algo"] == "ttpl_bt_s1"} == {2, 4}       # both groupings of 8 ranks
    assert {c["b"] for c in c8 if c["algo"] == "ttpl_bt_s1" and c["n"] == 4} == {0, 1, 2, 4}
    assert {c["b"] for c in c8 if c["algo"] == "ttpl_bt" and c["n"] == 2} == {0, 1, 2}
    assert len(tuner.candidates(8, full=False)) < len(c8)


def test_shipped_table_has_no_entry_that_the_native_reader_misreads():
    import json
    from rbruck_alltoallv_b200.parallel.plan import ALGOS
    path = tuner.Path(tuner.__file__).resolve().parent / "tuner_table.json"
    tab = json.loads(path.read_text())
    from rbruck_alltoallv_b200 import _native
    lib = _native.host_lib()
    lib.rbv_tuner_set_table(str(path).encode())
    assert lib.rbv_tuner_entries() == len(tab)
    for key, ent in tab.items():
        parts = key.split("-")
        P, G, cls = int(parts[0][1:]), int(parts[1][1:]), int(parts[2][1:])
        sk = int(parts[3][1:]) if len(parts) > 3 else 0
        nat = tuner.native_choose(P, G, 2.0 ** cls * 1.2, 0.9 if sk else 0.0, path=path)
        assert nat["algo"] == ent["choice"]["algo"], key
        assert nat["protocol"] == ent["choice"].get("protocol", "rendezvous"), key
