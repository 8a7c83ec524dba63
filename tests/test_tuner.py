"""Tuner table logic (no GPU)."""
import json

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
