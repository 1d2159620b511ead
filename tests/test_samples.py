"""The sample programs run end to end at small sizes."""
import importlib.util
import os

import pytest
import torch

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "samples")


def _load(name):
    spec = importlib.util.spec_from_file_location(f"sample_{name}", os.path.join(ROOT, f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_gpt_training_sample_learns(tmp_path):
    out = _load("gpt_training").main(["--steps", "30", "--device", "cpu", "--eval-every", "30", "--quiet",
                                      "--save", str(tmp_path / "m.ikw")])
    assert out["final_loss"] < out["first_loss"] - 1.0
    assert out["held_out_loss"] < 5.0 and len(out["sample"]) == 84
    assert (tmp_path / "m.ikw").stat().st_size > 3_000_000


def test_xor_sample():
    out = _load("xor").main(quiet=True)
    p = out["predictions"]
    assert p[0] < 0.1 and p[1] > 0.9 and p[2] > 0.9 and p[3] < 0.1 and out["rebuilt_matches"]


def test_rag_sample():
    out = _load("rag").main(quiet=True)
    assert out["sources"][0] == "dp.txt"
    assert "reduce-scatter" in out["messages"][-1]["content"]


def test_house_prices_api_sample():
    pytest.importorskip("fastapi")
    out = _load("house_prices_api").main([])
    assert out["mae"] < 8.0
    assert 250 < out["one"]["output"][0] < 420 and len(out["many"]["outputs"]) == 2


@pytest.mark.gpu
def test_quantization_sample():
    out = _load("quantization").main(["--kind", "int4", "--layers", "2", "--dim", "512"])
    assert out["relative_error"] < 0.25 and out["reload_identical"]


def test_spirals_sample_separates_the_classes():
    out = _load("spirals").main(quiet=True)
    assert out["accuracy"] > 0.9 and out["picture"].shape == (24, 24)


def test_override_sample_swaps_a_kernel_in_and_out():
    out = _load("override").main(quiet=True)
    assert out["source_while_registered"] == "plug-in" and out["restored"]
    assert 0.005 < out["largest_difference"] < 0.05
    assert out["conformance"] and all(v == "ok" for v in out["conformance"]), "close enough at the bf16 tolerance"
    assert all(v == "failed" for v in out["conformance_of_relu"])


def test_onnx_import_sample_round_trips_and_trains():
    out = _load("onnx_import").main(quiet=True)
    assert out["largest_difference"] < 1e-5 and out["last_loss"] < 0.5 * out["first_loss"] and out["parameters"] > 2000


def test_reranker_sample_puts_the_right_passage_first():
    out = _load("reranker").main(quiet=True)
    assert out["reranked"][0] == "collective.txt" and len(out["shortlist"]) >= 2


def test_gpt_api_sample_answers_over_v1():
    pytest.importorskip("fastapi")
    out = _load("gpt_api").main(["--quiet"])
    assert out["models"] == ["tiny"] and out["completion"]["usage"]["completion_tokens"] == 8
    assert out["chat"]["choices"][0]["message"]["role"] == "assistant" and out["streamed_chunks"] >= 2
    assert out["refused"] == 400


def test_shape_recognition_sample_learns_the_four_shapes():
    out = _load("shape_recognition").main(epochs=5, quiet=True)
    assert out["accuracy"] > 0.9


def test_sentiment_sample_needs_word_order():
    scores = _load("sentiment").main(epochs=6, quiet=True, only=("bag of words", "lstm", "gru"))
    assert scores["bag of words"] < 0.7 and scores["lstm"] > 0.95 and scores["gru"] > 0.95


def test_ocr_sample_reads_lines_through_ctc():
    out = _load("ocr").main(steps=450, quiet=True, train_lines=1000)
    assert out["final_loss"] < 0.5 and out["characters"] > 0.8


def test_summarizer_sample_beats_the_extractive_baselines():
    out = _load("summarizer").main(steps=200, quiet=True)
    assert out["scores"]["model"] > out["scores"]["best sentence"] + 0.1 and out["final_loss"] < 0.3


def test_text_generation_sample_continues_the_grammar_and_the_paths_agree():
    out = _load("text_generation").main(steps=150, quiet=True, benchmark=True, length=48)
    assert out["final_loss"] < 1.0 and out["benchmark"]["same_text"]
    assert any(w in out["continuations"][0] for w in ("the ", "a ", "road", "key", "rain"))


def test_vision_sample_detects_and_segments_the_shapes():
    out = _load("idrak_vision").main(steps=120, quiet=True)
    assert out["map50"] > 0.8 and out["miou"] > 0.9


def test_whisper_speech_sample_runs_the_whole_pipeline(tmp_path):
    from idrak_b200.audio.flac import write_flac
    mod = _load("whisper_speech")
    out = mod.main(quiet=True)
    assert out["features"] == (1, 80, 3000) and len(out["tokens"]) <= 32
    path = tmp_path / "tone.flac"
    write_flac(str(path), mod.synthetic_recording(1.0, 16000), 16000)
    again = mod.main(audio=str(path), quiet=True)
    assert again["features"] == (1, 80, 3000)


def test_chat_sample_info_chat_and_profile():
    mod = _load("chat")
    described = mod.main("info", quiet=True)
    assert described["layers"] == 2 and described["kv_heads"] == 2 and described["parameters"] > 50_000
    talked = mod.main("chat", message="hello", quiet=True)
    assert len(talked["replies"]) == 1 and talked["messages"][-1]["role"] == "assistant"
    timed = mod.main("profile", quiet=True)
    assert timed["prompt_tokens"] > 50 and timed["decode_tokens_per_s"] > 0


def test_tts_sample_trains_and_writes_a_recording(tmp_path):
    from idrak_b200.audio import read_wav
    mod = _load("tts_vits")
    path = tmp_path / "said.wav"
    out = mod.main(text="bead", out=str(path), steps=12, quiet=True)
    first, last = out["history"][0], out["history"][-1]
    assert last["kl"] + last["duration"] < first["kl"] + first["duration"]
    samples, rate = read_wav(str(path))
    assert rate == 8000 and samples.shape[-1] == out["samples"] and out["samples"] >= 4 * 32
