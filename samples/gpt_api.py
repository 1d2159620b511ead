"""A model behind the OpenAI-style API: a small decoder is registered with the inference engine, the `/v1` routes are
mounted, and completions, a chat completion, a streamed completion and the model list are requested in process.

    python samples/gpt_api.py            # add --serve to listen on 127.0.0.1:8080 instead

Reference: samples/Idrak.Samples.GptApi/Program.cs.
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.models import DecoderSpec, build_decoder  # noqa: E402
from idrak_b200.serve.api import create_app  # noqa: E402
from idrak_b200.serve.inference_engine import InferenceEngine  # noqa: E402
from idrak_b200.text import ByteTokenizer  # noqa: E402


def main(argv=None) -> dict:
    argv = list(argv or [])
    tok = ByteTokenizer()
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=tok.vocab_size, max_positions=256)
    device = "cuda" if torch.cuda.is_available() else "cpu"

    def load():
        return build_decoder(spec, seed=0).to(device, torch.bfloat16 if device == "cuda" else torch.float32).eval(), tok
    engine = InferenceEngine.create().add_chat("tiny", load, engine_args={"num_blocks": 64, "max_batch": 4}).build()
    app = create_app(engine, default_model="tiny")
    if "--serve" in argv:
        import uvicorn
        uvicorn.run(app, host="127.0.0.1", port=8080)
        return {}
    from fastapi.testclient import TestClient
    out = {}
    with TestClient(app) as client:
        out["models"] = [m["id"] for m in client.get("/v1/models").json()["data"]]
        r = client.post("/v1/completions", json={"model": "tiny", "prompt": "abc", "max_tokens": 8, "temperature": 0})
        out["completion"] = r.json()
        r = client.post("/v1/chat/completions", json={"model": "tiny", "max_tokens": 6, "temperature": 0,
                                                      "messages": [{"role": "user", "content": "hi"}]})
        out["chat"] = r.json()
        chunks = []
        with client.stream("POST", "/v1/completions", json={"model": "tiny", "prompt": "abc", "max_tokens": 5,
                                                            "temperature": 0, "stream": True}) as s:
            for line in s.iter_lines():
                if line.startswith("data: ") and line != "data: [DONE]":
                    chunks.append(json.loads(line[6:]))
        out["streamed_chunks"] = len(chunks)
        out["refused"] = client.post("/v1/completions", json={"model": "tiny", "prompt": "x", "best_of": 3}).status_code
    engine.close()
    if "--quiet" not in argv:
        print(json.dumps({k: v if not isinstance(v, dict) else v.get("usage") for k, v in out.items()}))
    return out


if __name__ == "__main__":
    main(sys.argv[1:])
