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


def test_mcp_client_over_http_stdio_and_in_process(tmp_path):
    import sys
    from idrak_b200.serve.mcp import McpClient, McpError, McpServer, serve_http
    server = McpServer(None, name="tools")
    server.register("add", "Add two numbers.", {"type": "object", "properties": {"a": {"type": "number"}, "b": {"type": "number"}},
                                               "required": ["a", "b"]}, lambda args: str(args["a"] + args["b"]))
    server.register("fail", "Always fails.", {"type": "object"}, lambda args: 1 / 0)
    local = McpClient.local(server)
    assert local.server_info["name"] == "tools" and local.ping()
    assert [t["name"] for t in local.list_tools()] == ["add", "fail"] and local.call("add", a=2, b=3) == "5"
    with pytest.raises(McpError, match="ZeroDivisionError"):
        local.call("fail")
    with pytest.raises(McpError, match="unknown tool"):
        local.call("nope")
    tools = local.as_tool_functions()
    assert tools["add"](a=1, b=1) == "2" and tools["add"].__doc__ == "Add two numbers." and "a" in tools["add"].schema["properties"]
    httpd = serve_http(server, token="secret")
    url = f"http://127.0.0.1:{httpd.server_address[1]}/mcp"
    try:
        remote = McpClient.http(url, token="secret")
        assert remote.call("add", a=10, b=-4) == "6" and len(remote.list_tools()) == 2
        import urllib.error
        with pytest.raises(urllib.error.HTTPError):
            McpClient.http(url, token="wrong")
    finally:
        httpd.shutdown()
    script = tmp_path / "srv.py"
    script.write_text(
        "import sys\n"
        f"sys.path.insert(0, {str(__import__('os').path.dirname(__import__('os').path.dirname(__import__('os').path.abspath(__file__))))!r})\n"
        "from idrak_b200.serve.mcp import McpServer\n"
        "s = McpServer(None)\n"
        "s.register('echo', 'Echo.', {'type': 'object'}, lambda a: a.get('text', ''))\n"
        "s.serve(sys.stdin, sys.stdout)\n")
    child = McpClient.stdio([sys.executable, str(script)])
    try:
        assert child.call("echo", text="hello") == "hello"
    finally:
        child.close()
