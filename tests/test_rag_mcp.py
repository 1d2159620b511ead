"""Retrieval index / prompt assembly and the MCP stdio server (host only)."""
import io
import json

import pytest
import torch

from idrak_b200.rag import VectorIndex, augment, chunks_of
from idrak_b200.serve.inference_engine import InferenceEngine
from idrak_b200.serve.mcp import McpServer


def _embed(texts):
    """Bag of letters: enough structure for nearest-neighbour checks."""
    out = []
    for t in texts:
        v = torch.zeros(26)
        for ch in t.lower():
            if "a" <= ch <= "z":
                v[ord(ch) - 97] += 1
        out.append(v.tolist())
    return out


def test_chunking_index_search_and_prompt(tmp_path):
    doc = ("Zebras live in Africa. They have stripes. " * 6) + "\n\n" + ("Quartz is a mineral. It is very hard. " * 6)
    chunks = chunks_of([("zoo.txt", doc)], size=120, overlap=20)
    assert len(chunks) > 3 and all(len(c.text) <= 240 for c in chunks) and chunks[0].source == "zoo.txt"
    assert chunks[1].text[:10] in doc and chunks[1].start > 0
    index = VectorIndex.build(chunks, _embed, batch=4)
    hits = index.search(_embed(["quartz mineral hard"])[0], k=2)
    assert len(hits) == 2 and "Quartz" in hits[0].chunk.text and hits[0].score >= hits[1].score
    index.save(str(tmp_path / "idx"))
    again = VectorIndex.load(str(tmp_path / "idx"))
    assert len(again) == len(index) and "Zebras" in again.search(_embed(["zebras stripes africa"])[0], k=1)[0].chunk.text
    msgs = augment("What is quartz?", hits)
    assert msgs[0]["role"] == "system" and "[1] (zoo.txt)" in msgs[1]["content"] and msgs[1]["content"].endswith("What is quartz?")
    assert "(no passages found)" in augment("x", [])[1]["content"]
    with pytest.raises(ValueError):
        chunks_of(["a"], size=10, overlap=10)


def test_mcp_server_lists_and_calls_tools():
    server = McpServer(InferenceEngine.create().build())
    server.register("add", "adds", {"type": "object", "properties": {"a": {"type": "number"}, "b": {"type": "number"}}},
                    lambda args: args["a"] + args["b"])
    server.register("boom", "fails", {"type": "object"}, lambda args: 1 / 0)
    lines = [{"jsonrpc": "2.0", "id": 1, "method": "initialize", "params": {"protocolVersion": "2024-11-05"}},
             {"jsonrpc": "2.0", "method": "notifications/initialized"},
             {"jsonrpc": "2.0", "id": 2, "method": "tools/list"},
             {"jsonrpc": "2.0", "id": 3, "method": "tools/call", "params": {"name": "add", "arguments": {"a": 2, "b": 3}}},
             {"jsonrpc": "2.0", "id": 4, "method": "tools/call", "params": {"name": "boom", "arguments": {}}},
             {"jsonrpc": "2.0", "id": 5, "method": "tools/call", "params": {"name": "nope"}},
             {"jsonrpc": "2.0", "id": 6, "method": "resources/list"}]
    reader = io.StringIO("\n".join(json.dumps(l) for l in lines) + "\nnot json\n")
    writer = io.StringIO()
    server.serve(reader, writer)
    out = [json.loads(l) for l in writer.getvalue().splitlines()]
    by_id = {o["id"]: o for o in out}
    assert by_id[1]["result"]["serverInfo"]["name"] == "idrak-b200" and by_id[1]["result"]["capabilities"]["tools"] is not None
    assert [t["name"] for t in by_id[2]["result"]["tools"]] == ["add", "boom"]
    assert by_id[3]["result"]["content"][0]["text"] == "5" and by_id[3]["result"]["isError"] is False
    assert by_id[4]["result"]["isError"] is True and "ZeroDivisionError" in by_id[4]["result"]["content"][0]["text"]
    assert by_id[5]["error"]["code"] == -32602 and by_id[6]["error"]["code"] == -32601
    assert by_id[None]["error"]["code"] == -32700 and len(out) == 7
