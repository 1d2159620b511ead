"""Speech to text with a Whisper checkpoint: audio file (WAV or FLAC) -> 16 kHz mono -> log-mel features -> encoder ->
greedy decoding with a key / value cache. With ``--model <folder>`` (a Hugging Face Whisper folder: ``config.json``,
``model.safetensors``, tokenizer files) the words are real; without one a small randomly initialised model of the
same architecture runs the identical pipeline on a synthetic recording, so that every stage can be seen offline
(the token ids it prints mean nothing).

    python samples/whisper_speech.py [--model <folder>] [--audio speech.wav]

Reference: samples/WhisperSpeech.
"""
import argparse
import json
import math
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.audio import decode_audio, resample  # noqa: E402
from idrak_b200.audio.whisper import Whisper, WhisperSpec, features  # noqa: E402


def synthetic_recording(seconds: float = 2.0, rate: int = 22050) -> torch.Tensor:
    t = torch.arange(int(seconds * rate)) / rate
    sweep = torch.sin(2 * math.pi * (200 + 300 * t) * t)
    return 0.4 * sweep * (0.5 + 0.5 * torch.sin(2 * math.pi * 3 * t))


def load(folder):
    from idrak_b200.formats.safetensors import load_file
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    model = Whisper(WhisperSpec.from_hf_config(config))
    missing = model.load_hf(load_file(os.path.join(folder, "model.safetensors")))
    if missing:
        raise SystemExit(f"the checkpoint lacks {len(missing)} tensors, e.g. {missing[:3]}")
    prefix = [config.get("decoder_start_token_id", 50258)]
    for pair in config.get("forced_decoder_ids") or []:
        prefix.append(pair[1])
    tokenizer = None
    try:
        from idrak_b200.text.tokenizer_io import load_tokenizer
        tokenizer = load_tokenizer(folder)
    except Exception:
        pass
    return model, prefix, config.get("eos_token_id", 50257), tokenizer


def main(model_folder=None, audio=None, device="cpu", quiet=False) -> dict:
    if audio:
        with open(audio, "rb") as f:
            samples, rate = decode_audio(f.read())
        samples = samples.mean(0)
    else:
        samples, rate = synthetic_recording(), 22050
    if rate != 16000:
        samples = resample(samples, rate, 16000)
    if model_folder:
        model, prefix, end, tokenizer = load(model_folder)
    else:
        torch.manual_seed(0)
        model = Whisper(WhisperSpec(mels=80, vocabulary=300, dim=64, encoder_layers=2, decoder_layers=2, heads=4, ff_dim=128))
        prefix, end, tokenizer = [1], 2, None
    model = model.to(device).eval()
    t0 = time.perf_counter()
    mel = features(samples, mels=model.spec.mels)[None].to(device)
    t1 = time.perf_counter()
    ids = model.generate(mel, prefix, end, max_tokens=32)[0]
    t2 = time.perf_counter()
    text = tokenizer.decode(ids) if tokenizer is not None else None
    if not quiet:
        print(f"audio {samples.numel() / 16000:.2f} s -> features {tuple(mel.shape)} in {1e3 * (t1 - t0):.0f} ms, "
              f"{len(ids)} tokens in {1e3 * (t2 - t1):.0f} ms")
        print("text  :", text if text is not None else "(no tokenizer: token ids only)")
        print("tokens:", ids)
    return {"features": tuple(mel.shape), "tokens": ids, "text": text}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model")
    ap.add_argument("--audio")
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args()
    main(a.model, a.audio, a.device)
