import json

import pytest

from idrak_b200.runtime import Tuner, size_class


def _tuner(tmp_path, speeds, enabled=True, key="gpu-a"):
    """A tuner whose timer reads a table instead of a clock: candidate functions return their name through a cell."""
    cell = {}
    def timer(fn, flush):
        fn()
        base = speeds[cell["name"]]
        cell["n"] = cell.get("n", 0) + 1
        return base * (1.0 + 0.01 * (cell["n"] % 3))            # a little jitter, the same for every candidate in turn
    cands = {name: (lambda name=name: cell.__setitem__("name", name)) for name in speeds}
    return Tuner(str(tmp_path / "tuning.json"), enabled=enabled, key=key, timer=timer), cands


def test_winner_needs_a_margin_and_is_remembered(tmp_path):
    t, c = _tuner(tmp_path, {"1": 1.00, "4": 0.80, "8": 0.90})
    assert t.choose("gemm.splits", (64, 4096, 4096), c, default="1") == "4"
    entry = t.entries()["gemm.splits:64x4096x4096"]
    assert entry["choice"] == "4" and entry["default"] == "1" and abs(entry["ratios"]["4"] - 0.8) < 0.03
    # a 2 % gain is not enough to leave the default
    t2, c2 = _tuner(tmp_path, {"1": 1.00, "4": 0.98})
    assert t2.choose("gemm.splits", (64, 8192, 4096), c2, default="1") == "1"
    # remembered: another process (a new Tuner on the same file) does not measure again
    t3, c3 = _tuner(tmp_path, {"1": 0.1, "4": 5.0, "8": 5.0})
    assert t3.choose("gemm.splits", (64, 4096, 4096), c3, default="1") == "4" and t3.measured == 0
    doc = json.load(open(tmp_path / "tuning.json"))
    assert doc["format"] == "idrak-tuning/1" and set(doc["devices"]) == {"gpu-a"}


def test_decisions_are_per_device_and_tuning_can_be_off(tmp_path):
    t, c = _tuner(tmp_path, {"a": 1.0, "b": 0.5})
    assert t.choose("k", (1,), c, default="a") == "b"
    other, c2 = _tuner(tmp_path, {"a": 1.0, "b": 2.0}, key="gpu-b")
    assert other.lookup("k", (1,)) is None and other.choose("k", (1,), c2, default="a") == "a"
    assert set(json.load(open(tmp_path / "tuning.json"))["devices"]) == {"gpu-a", "gpu-b"}
    off, c3 = _tuner(tmp_path, {"a": 1.0, "b": 0.1}, enabled=False, key="gpu-c")
    assert off.choose("k", (2,), c3, default="a") == "a" and off.measured == 0
    # the cache is still honoured with tuning off
    assert _tuner(tmp_path, {"a": 1, "b": 1}, enabled=False)[0].choose("k", (1,), c, default="a") == "b"
    assert t.forget("k:") == 1 and t.lookup("k", (1,)) is None
    with pytest.raises(KeyError):
        t.choose("k", (3,), c, default="zzz")


def test_size_classes():
    assert [size_class(n) for n in (1, 2, 3, 48, 64, 65, 4096)] == [1, 2, 4, 64, 64, 128, 4096]
