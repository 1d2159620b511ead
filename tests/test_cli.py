"""Command line: parsing, config table, inspect / convert / tokenize / template / complete / tune on tiny CPU models."""
import json
import os

import pytest
import torch

from idrak_b200.cli.__main__ import build_parser, main
from idrak_b200.config import Settings, describe
from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.models.pretrained import save_huggingface
from idrak_b200.text import train_tokenizer


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("model")
    tok = train_tokenizer("bpe", ["the quick brown fox jumps over the lazy dog"] * 20, 300, ["<|endoftext|>"])
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|endoftext|>"}))
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=tok.vocab_size, max_positions=128)
    save_huggingface(build_decoder(spec, seed=2).float(), d)
    return str(d)


def test_settings_table_and_validation():
    s = Settings({"IDRAK_MAX_BATCH": "12", "IDRAK_WORKSPACE": "64M", "IDRAK_TP_MULTIMEM": "off"})
    assert s.get("IDRAK_MAX_BATCH") == 12 and s.get("IDRAK_WORKSPACE") == 64 << 20 and s.get("IDRAK_TP_MULTIMEM") is False
    assert s.get("IDRAK_KEEP_ALIVE") == 300.0 and s.validate() == []
    bad = Settings({"IDRAK_MAX_BATCH": "many", "IDRAK_NO_SUCH": "1", "IDRAK_BENCH_DP": "mpi"})
    with pytest.raises(ValueError, match="IDRAK_MAX_BATCH='many'"):
        bad.get("IDRAK_MAX_BATCH")
    problems = bad.validate()
    assert len(problems) == 3 and any("IDRAK_NO_SUCH" in p for p in problems) and any("fused, nccl" in p for p in problems)
    assert "IDRAK_PREFILL_CHUNK" in describe(s) and "64M" not in describe(s)
    with pytest.raises(KeyError):
        s.get("IDRAK_NOPE")


def test_parser_knows_every_command_group():
    p = build_parser()
    names = set(p._subparsers._group_actions[0].choices)
    assert {"devices", "check", "doctor", "kernels", "memory", "bench", "inspect", "convert", "quantize", "merge", "package",
            "complete", "chat", "batch", "embed", "tokenize", "template", "tune", "pretrain", "perplexity", "serve",
            "ping", "cluster-bench", "config"} <= names
    with pytest.raises(SystemExit):
        p.parse_args(["complete"])                       # --model is required


def test_inspect_convert_tokenize_template_complete(model_dir, tmp_path, capsys):
    assert main(["inspect", os.path.join(model_dir, "model.safetensors"), "--tensors"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["kind"] == "safetensors" and out["tensor_count"] > 10 and "model.norm.weight" in out["tensors"]
    assert main(["convert", model_dir, str(tmp_path / "idrak"), "--to", "idrak"]) == 0
    assert (tmp_path / "idrak" / "spec.json").exists()
    capsys.readouterr()
    assert main(["tokenize", "--tokenizer", model_dir, "--text", "the quick fox"]) == 0
    t = json.loads(capsys.readouterr().out)
    assert t["count"] == len(t["ids"]) and "".join(t["pieces"]) == "the quick fox"
    text = tmp_path / "corpus.txt"
    text.write_text("the quick brown fox\n\njumps over the lazy dog\n\n" * 30)
    assert main(["tokenize", "--tokenizer", model_dir, "--output", str(tmp_path / "c.tokens"), str(text)]) == 0
    rec = json.loads(capsys.readouterr().out)
    assert rec["documents"] == 60 and rec["tokens"] > 100
    assert main(["template", "--tokenizer", model_dir, "--messages", '[{"role": "user", "content": "hi"}]']) == 0
    assert "<|im_start|>user\nhi" in capsys.readouterr().out
    assert main(["complete", "--model", model_dir, "--prompt", "the quick", "--max-tokens", "6", "--temperature", "0",
                 "--json", "--device", "cpu"]) == 0
    r = json.loads(capsys.readouterr().out)
    assert r["completion_tokens"] <= 6 and r["prompt_tokens"] >= 2
    assert main(["perplexity", "--model", model_dir, "--tokens", str(tmp_path / "c.tokens"), "--seq-len", "32",
                 "--windows", "4", "--device", "cpu"]) == 0
    assert json.loads(capsys.readouterr().out)["perplexity"] > 1
    assert main(["inspect", str(tmp_path / "nothing.bin")]) == 2
    assert "idrak inspect" in capsys.readouterr().err


def test_tune_and_package_commands(model_dir, tmp_path, capsys):
    data = tmp_path / "train.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": "the quick ", "response": "brown fox"}) for _ in range(6)))
    assert main(["tune", "--model", model_dir, "--data", str(data), "--out", str(tmp_path / "ad"), "--rank", "2", "--alpha",
                 "4", "--max-steps", "3", "--batch-tokens", "64", "--max-length", "32", "--device", "cpu", "--dtype",
                 "fp32"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert lines[-1]["steps"] == 3 and (tmp_path / "ad" / "adapter_config.json").exists()
    assert main(["merge", model_dir, str(tmp_path / "ad"), str(tmp_path / "merged")]) == 0
    assert (tmp_path / "merged" / "model.safetensors").exists()
    capsys.readouterr()
    assert main(["package", str(tmp_path / "m.ikm"), "--source", model_dir]) == 0
    assert main(["package", str(tmp_path / "m.ikm"), "--list"]) == 0
    listing = capsys.readouterr().out
    assert "Tokenizer" in listing and "Weights" in listing
    assert main(["config"]) in (0, 1)


def test_data_retrieval_onnx_and_page_commands(tmp_path, capsys):
    import json as _json
    from idrak_b200.cli.__main__ import main as run
    rows = tmp_path / "rows.jsonl"
    rows.write_text("\n".join(_json.dumps({"text": t}) for t in
                              ["the cat sat on the mat", "the cat sat on the mat", "dogs run in the park every day", "qubits power quantum computers"]))
    assert run(["data", "dedupe", str(rows), "-o", str(tmp_path / "u.jsonl")]) == 0
    assert _json.loads(capsys.readouterr().out)["kept"] == 3
    assert run(["data", "split", str(tmp_path / "u.jsonl"), "-o", str(tmp_path / "part.jsonl"), "--fraction", "0.67"]) == 0
    assert _json.loads(capsys.readouterr().out) == {"first": 2, "rest": 1}
    assert run(["index", str(tmp_path / "u.jsonl"), "-o", str(tmp_path / "idx")]) == 0
    capsys.readouterr()
    assert run(["search", str(tmp_path / "idx"), "quantum qubits", "-k", "1"]) == 0
    assert "qubits" in _json.loads(capsys.readouterr().out.splitlines()[0])["text"]
    from idrak_b200.nn import Network
    (tmp_path / "net.json").write_text(_json.dumps(Network.input(4).linear(3).relu().linear(2).to_json()))
    assert run(["onnx", "export", str(tmp_path / "net.json"), "-o", str(tmp_path / "net.onnx")]) == 0
    capsys.readouterr()
    assert run(["onnx", "inspect", str(tmp_path / "net.onnx")]) == 0
    info = _json.loads(capsys.readouterr().out)
    assert info["operators"]["Gemm"] == 2 and info["unsupported"] == [] and info["parameters"] >= 4 * 3 + 3 + 3 * 2 + 2
    import numpy as np
    np.save(tmp_path / "x.npy", np.ones((5, 4), np.float32))
    assert run(["onnx", "run", str(tmp_path / "net.onnx"), "--input", str(tmp_path / "x.npy")]) == 0
    assert _json.loads(capsys.readouterr().out)["shape"] == [5, 2]
    pytest.importorskip("PIL")
    assert run(["page", "a short page of text for the test", "-o", str(tmp_path / "p.png"), "--width", "300", "--height", "120",
                "--size", "16", "--margin", "10", "--effects", "gaussian_noise,rotate_small"]) == 0
    out = _json.loads(capsys.readouterr().out)
    assert out["words"] == 8 and (tmp_path / "p.words.jsonl").exists()
    from idrak_b200.imaging import decode
    assert decode((tmp_path / "p.png").read_bytes()).shape == (120, 300, 3)
    assert run(["image", "resize", str(tmp_path / "p.png"), "-o", str(tmp_path / "small.png"), "--width", "60", "--height", "24"]) == 0
    assert _json.loads(capsys.readouterr().out)["shape"] == [24, 60, 3]
