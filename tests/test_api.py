"""Inference engine semantics (copies, leases, queue limit, timeout, keep-alive, micro-batching, stats) and the HTTP
API over a tiny byte-level model, all on CPU."""
import json
import threading
import time

import pytest
import torch

from idrak_b200.models.decoder import build_decoder
from idrak_b200.models.spec import DecoderSpec
from idrak_b200.serve.inference_engine import (InferenceEngine, InferenceQueueFull, InferenceTimeout,
                                               register_model_kind)
from idrak_b200.text import ByteTokenizer


def _chat_model():
    tok = ByteTokenizer()
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=128, vocab=tok.vocab_size, max_positions=256)
    m = build_decoder(spec, seed=3).float().eval()
    for p in m.parameters():
        p.data.mul_(3.0)
    return m, tok


class Doubler(torch.nn.Module):
    calls = 0

    def forward(self, x):
        Doubler.calls += 1
        return x * 2


def test_predictor_copies_exclusive_leases_queue_limit_and_timeout():
    gate = threading.Event()

    class Slow:
        def __call__(self, x):
            gate.wait(5)
            return x + 1

    eng = (InferenceEngine.create()
           .add_predictor("slow", Slow, copies=1, exclusive=True, queue_limit=1, timeout=0.2)
           .add_predictor("double", Doubler, copies=2)
           .build())
    assert not eng.model("slow").loaded                       # load on first use
    results = []
    t = threading.Thread(target=lambda: results.append(eng.predict("slow", 1)))
    t.start()
    while eng.model("slow")._active == 0:
        time.sleep(0.01)
    waiter_error = []

    def waiter():
        try:
            eng.predict("slow", 2)
        except InferenceTimeout as e:
            waiter_error.append(e)
    w = threading.Thread(target=waiter)
    w.start()
    while eng.model("slow")._waiting == 0:
        time.sleep(0.01)
    with pytest.raises(InferenceQueueFull, match="queue limit 1"):
        eng.predict("slow", 3)
    w.join()
    assert len(waiter_error) == 1 and "0.2 s" in str(waiter_error[0])
    gate.set()
    t.join()
    assert results == [2]
    st = eng.model("slow").status()
    assert st["rejected"] == 1 and st["timeouts"] == 1 and st["requests"] == 1 and st["failures"] == 0
    assert st["p95_latency"] >= st["average_queue_wait"] >= 0
    # shared copies rotate
    a = [eng.model("double").acquire()[0] for _ in range(4)]
    assert a == [0, 1, 0, 1]
    for i in a:
        eng.model("double").release(i)
    assert float(eng.predict("double", torch.tensor(2.0))) == 4.0
    with pytest.raises(KeyError, match="no model named 'nope'"):
        eng.predict("nope", 1)
    with pytest.raises(TypeError, match="predictor model"):
        eng.generate("double", "x")


def test_keep_alive_unloads_idle_models_and_micro_batcher_batches():
    now = [0.0]
    Doubler.calls = 0
    eng = (InferenceEngine.create().with_clock(lambda: now[0])
           .add_predictor("d", Doubler, keep_alive=10.0, micro_batch=8, micro_batch_wait=0.05).build())
    outs = [None] * 6
    ts = [threading.Thread(target=lambda i=i: outs.__setitem__(i, eng.predict("d", torch.tensor([float(i)]))))
          for i in range(6)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert [float(o) for o in outs] == [0.0, 2.0, 4.0, 6.0, 8.0, 10.0] and Doubler.calls < 6
    assert eng.model("d").loaded and eng.expire_idle() == []
    now[0] = 11.0
    assert eng.expire_idle() == ["d"] and not eng.model("d").loaded
    assert float(eng.predict("d", torch.tensor([3.0]))) == 6.0 and eng.model("d").stats.loads == 2
    register_model_kind("echo", lambda m, req: {"echo": req, "by": m})
    e2 = InferenceEngine.create().add_plugin("echo", "e", lambda: "copy").build()
    assert e2.invoke("e", 5) == {"echo": 5, "by": "copy"}
    eng.close()


@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    from idrak_b200.serve.api import create_app
    eng = (InferenceEngine.create()
           .add_chat("tiny", _chat_model, engine_args={"num_blocks": 64, "max_batch": 4})
           .add_predictor("double", Doubler)
           .build())
    with TestClient(create_app(eng, default_max_tokens=16)) as c:
        yield c
    eng.close()


def test_v1_models_chat_and_completions(client):
    assert [m["id"] for m in client.get("/v1/models").json()["data"]] == ["tiny", "double"]
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "temperature": 0, "max_tokens": 8}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    j = r.json()
    assert j["object"] == "chat.completion" and j["choices"][0]["message"]["role"] == "assistant"
    assert j["usage"]["completion_tokens"] <= 8 and j["usage"]["total_tokens"] == j["usage"]["prompt_tokens"] + j["usage"]["completion_tokens"]
    assert j["choices"][0]["finish_reason"] in ("stop", "length")
    # the same request streamed gives the same text, then usage, then [DONE]
    r = client.post("/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}})
    events = [l[6:] for l in r.text.split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert text == j["choices"][0]["message"]["content"] and chunks[-1]["usage"] == j["usage"]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    r = client.post("/v1/completions", json={"model": "tiny", "prompt": "abc", "temperature": 0, "max_tokens": 5})
    assert r.status_code == 200 and r.json()["object"] == "text_completion" and r.json()["usage"]["prompt_tokens"] == 3
    r = client.post("/v1/embeddings", json={"model": "tiny", "input": ["hello", "world!"]})
    data = r.json()["data"]
    assert len(data) == 2 and len(data[0]["embedding"]) == 64 and r.json()["usage"]["prompt_tokens"] == 11
    assert abs(sum(v * v for v in data[0]["embedding"]) - 1.0) < 1e-4


def test_v1_refuses_unimplemented_fields_by_name(client):
    base = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}]}
    for extra, word in (({"n": 2}, "'n'"), ({"logprobs": True}, "'logprobs'"), ({"logit_bias": {"5": 1}}, "'logit_bias'"),
                        ({"response_format": {"type": "json_object"}}, "'response_format'"),
                        ({"tool_choice": "required"}, "'tool_choice'"), ({"temperature": "hot"}, "'temperature'"),
                        ({"stop": 5}, "'stop'")):
        r = client.post("/v1/chat/completions", json={**base, **extra})
        assert r.status_code == 400 and word in r.json()["error"]["message"], r.text
        assert r.json()["error"]["type"] == "invalid_request_error"
    for extra, word in (({"echo": True}, "'echo'"), ({"best_of": 3}, "'best_of'"), ({"suffix": "x"}, "'suffix'")):
        r = client.post("/v1/completions", json={"model": "tiny", "prompt": "a", **extra})
        assert r.status_code == 400 and word in r.json()["error"]["message"]
    r = client.post("/v1/chat/completions", json={**base, "model": "missing"})
    assert r.status_code == 404 and r.json()["error"]["code"] == "model_not_found"
    r = client.post("/v1/chat/completions", json={**base, "model": "double"})
    assert r.status_code == 400 and "predictor" in r.json()["error"]["message"]
    r = client.post("/v1/chat/completions", content=b"{nope", headers={"content-type": "application/json"})
    assert r.status_code == 400 and "JSON" in r.json()["error"]["message"]
    r = client.post("/v1/chat/completions", json={**base, "messages": [{"role": "user", "content": [
        {"type": "image_url", "image_url": {"url": "data:"}}]}]})
    assert r.status_code == 400 and "image_url" in r.json()["error"]["message"]


def test_api_routes_predict_and_status(client):
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "stream": False,
            "options": {"temperature": 0, "num_predict": 6}}
    j = client.post("/api/chat", json=body).json()
    assert j["done"] and j["message"]["role"] == "assistant" and j["eval_count"] <= 6
    lines = [json.loads(l) for l in client.post("/api/chat", json={**body, "stream": True}).text.splitlines()]
    assert lines[-1]["done"] and "".join(l["message"]["content"] for l in lines) == j["message"]["content"]
    assert client.post("/api/chat", json={**body, "options": {"mirostat": 2}}).status_code == 400
    assert client.post("/api/generate", json={"model": "tiny", "prompt": "ab", "options": {"num_predict": 3}}).json()["done"]
    tags = client.get("/api/tags").json()["models"]
    assert tags[0]["name"] == "tiny" and tags[0]["details"]["context_length"] == 256
    assert client.get("/api/ps").json()["models"][0]["name"] == "tiny"
    assert "version" in client.get("/api/version").json()
    assert client.post("/predict/double", json={"input": [1, 2]}).json() == {"output": [2.0, 4.0]}
    assert client.post("/predict/double/batch", json={"inputs": [[1], [3]]}).json() == {"outputs": [[2.0], [6.0]]}
    assert client.post("/predict/none", json={"input": 1}).status_code == 404
    st = client.get("/status").json()
    assert {m["name"] for m in st["models"]} == {"tiny", "double"} and st["models"][0]["requests"] > 0
