"""The second group of commands: train / predict / runs, cluster init / inspect / sim / replay, env, completion, alias,
verify, bench-compare, train-tokenizer."""
import json
import os

import pytest

from idrak_b200.cli.__main__ import main


def run(capsys, *argv):
    rc = main(list(argv))
    return rc, capsys.readouterr().out


def test_train_predict_runs(tmp_path, capsys):
    csv = tmp_path / "d.csv"
    rows = ["a,b,y"] + [f"{i % 10},{(i * 7) % 5},{2 * (i % 10) - 3 * ((i * 7) % 5) + 1}" for i in range(200)]
    csv.write_text("\n".join(rows) + "\n")
    out = tmp_path / "runs" / "first"
    rc, text = run(capsys, "train", str(csv), "--target", "y", "-o", str(out), "--epochs", "150", "--batch", "64")
    assert rc == 0 and (out / "model.ikw").exists() and (out / "log.csv").exists()
    meta = json.loads((out / "run.json").read_text())
    assert meta["features"] == ["a", "b"] and meta["loss"] < 0.05
    rc, text = run(capsys, "predict", str(out), "4", "2")
    assert rc == 0 and abs(float(text.split()[0]) - 3.0) < 0.8
    rc, text = run(capsys, "runs", str(tmp_path / "runs"))
    assert "first" in text
    rc, text = run(capsys, "verify", str(out))
    assert rc == 0 and "tensors" in text


def test_cluster_commands(tmp_path, capsys, monkeypatch):
    monkeypatch.setenv("IDRAK_HOME", str(tmp_path / "home"))
    topo = tmp_path / "t.json"
    rc, _ = run(capsys, "cluster", "init", str(topo), "--nodes", "2", "--gpus", "4")
    assert rc == 0 and json.loads(topo.read_text())["format"] == "idrak-topology/1"
    rc, text = run(capsys, "cluster", "inspect", str(topo), "--bytes", str(1 << 26))
    assert "world 8" in text and "predicted ring" in text and "predicted hierarchical" in text
    csv = tmp_path / "m.csv"
    csv.write_text("bytes,seconds\n" + "\n".join(f"{n},{5e-5 + n / 5e9}" for n in (1024, 1 << 20, 1 << 26)) + "\n")
    rc, cal = run(capsys, "cluster", "calibrate", str(csv), "--link", "tcp")
    assert rc == 0 and "bandwidth 5.00 GB/s" in cal
    rc, again = run(capsys, "cluster", "inspect", str(topo), "--bytes", str(1 << 26))
    assert again != text                                       # the calibrated link changes the prediction
    log = tmp_path / "run.evlog"
    rc, text = run(capsys, "cluster", "sim", "--world", "3", "--steps", "6", "--failures", "slow-worker", "--rate", "0.9",
                   "--values", "1024", "--log", str(log), "--seed", "3")
    assert rc == 0 and "fault(s)" in text and log.exists()
    first = [l for l in text.splitlines() if l.startswith("  slow@")]
    rc, text = run(capsys, "cluster", "replay", str(log), "--world", "3", "--steps", "6", "--values", "1024")
    assert [l for l in text.splitlines() if l.startswith("  slow@")] == first and first


def test_env_completion_alias_transports(tmp_path, capsys, monkeypatch):
    monkeypatch.setenv("IDRAK_HOME", str(tmp_path))
    monkeypatch.setenv("IDRAK_GEMM_PAIR", "2")
    rc, text = run(capsys, "env")
    assert "IDRAK_GEMM_PAIR=2" in text
    rc, text = run(capsys, "env", "--all", "--export")
    assert "export IDRAK_TOKENIZER=library" in text
    rc, text = run(capsys, "completion", "bash")
    assert "complete -F _idrak idrak" in text and "train-tokenizer" in text
    assert run(capsys, "alias", "small", "/models/small")[0] == 0
    assert run(capsys, "alias", "small")[1].strip() == "/models/small"
    assert "small -> /models/small" in run(capsys, "alias")[1]
    assert run(capsys, "alias", "small", "--remove")[0] == 0
    with pytest.raises(SystemExit):
        main(["alias", "small"])
    capsys.readouterr()
    rc, text = run(capsys, "transports")
    assert "gloo" in text and "sim" in text


def test_bench_compare(tmp_path, capsys):
    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    a.write_text('{"case": "gemm", "ms": 1.0, "args": {"m": 8, "iters": 10}}\n{"case": "flash_fwd", "ms": 2.0, "args": {"seq": 4}}\n')
    b.write_text('{"case": "gemm", "ms": 1.2, "args": {"m": 8, "iters": 50}}\n{"case": "flash_fwd", "ms": 1.5, "args": {"seq": 4}}\n')
    rc, text = run(capsys, "bench-compare", str(a), str(b))
    assert rc == 1 and "WORSE gemm" in text and "(+20.0 %)" in text and "(-25.0 %)" in text
    assert run(capsys, "bench-compare", str(a), str(a))[0] == 0


def test_train_tokenizer_command(tmp_path, capsys):
    src = tmp_path / "c.txt"
    src.write_text("the cat sat on the mat\nthe dog sat on the log\n" * 30)
    rc, text = run(capsys, "train-tokenizer", str(src), "-o", str(tmp_path / "tok"), "--vocab", "300")
    assert rc == 0 and (tmp_path / "tok" / "tokenizer.json").exists()
    from idrak_b200.text.tokenizers_native import load_tokenizer_json
    tok = load_tokenizer_json(str(tmp_path / "tok" / "tokenizer.json"))
    assert tok.decode(tok.encode("the cat sat")) == "the cat sat"
