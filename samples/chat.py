"""Chat with a language model in the Hugging Face layout (Llama, Qwen, Mistral, Gemma, GPT-2 ...), run by this
package's own engine:

    python samples/chat.py info    <folder>     what the loader made of the model (architecture, parameters)
    python samples/chat.py chat    <folder>     chat in the model's own chat template (a line per turn, empty line ends)
    python samples/chat.py profile <folder>     time a prompt pass and decoding

``<folder>`` may also be a ``.gguf`` file or an ``.ikm`` package. Without a folder a tiny randomly initialised
Llama-shaped model is written to a temporary folder in the Hugging Face layout and loaded back from it, so the three
commands can be tried offline (its answers are noise).

Reference: samples/Idrak.Samples.Chat/Program.cs.
"""
import argparse
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.generation.text_generator import TextGenerator  # noqa: E402
from idrak_b200.models import DecoderSpec, build_decoder  # noqa: E402
from idrak_b200.models.pretrained import load_pretrained, save_huggingface  # noqa: E402
from idrak_b200.serve.engine import GenerationOptions  # noqa: E402
from idrak_b200.text import ByteTokenizer  # noqa: E402


def tiny_folder(folder: str) -> str:
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=ByteTokenizer().vocab_size,
                             max_positions=256)
    save_huggingface(build_decoder(spec, seed=0).float(), folder)
    return folder


def tokenizer_for(folder: str):
    try:
        from idrak_b200.text.tokenizer_io import load_tokenizer
        return load_tokenizer(folder)
    except Exception:
        return ByteTokenizer()                          # a folder without tokenizer files: bytes


def info(model) -> dict:
    s = model.spec
    params = sum(p.numel() for p in model.parameters())
    return {"layers": s.layers, "dim": s.dim, "heads": s.heads, "kv_heads": s.kv_heads, "head_dim": s.head_dim,
            "ff_dim": s.ff_dim, "vocabulary": s.vocabulary, "max_positions": s.max_positions, "norm": s.norm,
            "gated": s.gated, "activation": s.activation, "rope": s.rope is not None, "tied": s.tie_embeddings,
            "parameters": params, "megabytes": round(sum(p.numel() * p.element_size() for p in model.parameters()) / 2 ** 20, 1)}


def profile(model, tokenizer, device) -> dict:
    gen = TextGenerator(model, tokenizer).start()
    try:
        prompt = "Tell me about the sea. " * 8
        opts = GenerationOptions(temperature=0.0, max_tokens=1)
        gen.generate(prompt, opts)                       # first pass: lazy set-up
        t0 = time.perf_counter()
        gen.generate(prompt, opts)
        t1 = time.perf_counter()
        r = gen.generate(prompt, GenerationOptions(temperature=0.0, max_tokens=48))
        t2 = time.perf_counter()
        n_prompt = len(gen.encode_prompt(prompt))
        new = max(len(r.token_ids) - 1, 1) if hasattr(r, "token_ids") else 47
        return {"prompt_tokens": n_prompt, "prompt_ms": 1e3 * (t1 - t0), "decode_tokens_per_s": new / max(t2 - t1 - (t1 - t0), 1e-6)}
    finally:
        gen.close()


def main(command: str = "info", folder=None, device: str = "cpu", message=None, quiet: bool = False) -> dict:
    with tempfile.TemporaryDirectory() as tmp:
        path = folder or tiny_folder(tmp)
        model = load_pretrained(path, device=device).eval()
        tokenizer = tokenizer_for(path)
        if command == "info":
            out = info(model)
            if not quiet:
                for k, v in out.items():
                    print(f"{k:14s} {v}")
            return out
        if command == "profile":
            out = profile(model, tokenizer, device)
            if not quiet:
                print(f"prompt of {out['prompt_tokens']} tokens: {out['prompt_ms']:.1f} ms; decoding {out['decode_tokens_per_s']:.1f} tokens/s")
            return out
        gen = TextGenerator(model, tokenizer).start()
        try:
            messages, replies = [], []
            turns = [message] if message else iter(lambda: input("> "), "")
            for line in turns:
                messages.append({"role": "user", "content": line})
                r = gen.chat(messages, GenerationOptions(temperature=0.7, max_tokens=64, seed=1))
                messages.append({"role": "assistant", "content": r.text})
                replies.append(r.text)
                if not quiet:
                    print(r.text)
            return {"replies": replies, "messages": messages}
        finally:
            gen.close()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("command", choices=["info", "chat", "profile"])
    ap.add_argument("folder", nargs="?")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--message")
    a = ap.parse_args()
    main(a.command, a.folder, a.device, a.message)
