"""Model Context Protocol: a server (stdio or HTTP) that offers the inference engine's models as tools, and a client
that calls the tools of any MCP server (stdio child process, HTTP endpoint or an in-process server).

Speaks JSON-RPC 2.0, one message per line: ``initialize``, ``ping``, ``tools/list``, ``tools/call``. Every text /
chat model becomes a ``generate_<name>`` tool (prompt or messages in, text out); every model that can embed a
``embed_<name>`` tool; extra tools can be registered as plain Python callables with a JSON schema.

    McpServer(engine).serve(sys.stdin, sys.stdout)

Reference: the MCP server of the reference (src/Idrak.Mcp: tools over the engine, stdio transport).
"""
from __future__ import annotations

import json
from typing import Any, Callable, Dict, IO, List, Optional

from .engine import GenerationOptions
from .inference_engine import InferenceEngine

PROTOCOL = "2024-11-05"


class McpError(Exception):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code, self.message = code, message


class McpServer:
    def __init__(self, engine: Optional[InferenceEngine] = None, name: str = "idrak-b200", version: str = "0.1.0"):
        self.engine, self.name, self.version = engine, name, version
        self.tools: Dict[str, dict] = {}
        self.initialized = False
        if engine is not None:
            for model in engine.names():
                kind = engine.model(model).settings.kind
                if kind in ("text", "chat"):
                    self._add_generate(model, kind)
                if kind in ("text", "chat", "embed"):
                    self._add_embed(model)

    # ------------------------------------------------------------------ tools
    def register(self, name: str, description: str, schema: dict, fn: Callable[[dict], Any]) -> None:
        self.tools[name] = {"description": description, "inputSchema": schema, "fn": fn}

    def _add_generate(self, model: str, kind: str) -> None:
        schema = {"type": "object", "properties": {
            "prompt": {"type": "string"}, "messages": {"type": "array", "items": {"type": "object"}},
            "max_tokens": {"type": "integer", "minimum": 1}, "temperature": {"type": "number", "minimum": 0}}}

        def call(args: dict):
            o = GenerationOptions(max_tokens=int(args.get("max_tokens", 256)))
            if "temperature" in args:
                o.temperature = float(args["temperature"])
            if args.get("messages"):
                if kind != "chat":
                    raise McpError(-32602, f"model '{model}' is a text model: pass 'prompt', not 'messages'")
                return self.engine.chat(model, args["messages"], o).text
            if not isinstance(args.get("prompt"), str) or not args["prompt"]:
                raise McpError(-32602, "pass a non-empty 'prompt' or 'messages'")
            return self.engine.generate(model, args["prompt"], o).text
        self.register(f"generate_{model}", f"Generate text with the model '{model}'.", schema, call)

    def _add_embed(self, model: str) -> None:
        schema = {"type": "object", "properties": {"texts": {"type": "array", "items": {"type": "string"}}},
                  "required": ["texts"]}
        self.register(f"embed_{model}", f"Sentence vectors from the model '{model}'.", schema,
                      lambda args: json.dumps(self.engine.embed(model, list(args["texts"]))))

    # ------------------------------------------------------------------ protocol
    def handle(self, message: dict) -> Optional[dict]:
        """One request -> its response (None for notifications)."""
        mid = message.get("id")
        method = message.get("method")
        try:
            if message.get("jsonrpc") != "2.0" or not isinstance(method, str):
                raise McpError(-32600, "not a JSON-RPC 2.0 request")
            if method == "initialize":
                self.initialized = True
                result = {"protocolVersion": PROTOCOL, "capabilities": {"tools": {"listChanged": False}},
                          "serverInfo": {"name": self.name, "version": self.version}}
            elif method in ("notifications/initialized", "notifications/cancelled"):
                return None
            elif method == "ping":
                result = {}
            elif method == "tools/list":
                result = {"tools": [{"name": n, "description": t["description"], "inputSchema": t["inputSchema"]}
                                    for n, t in sorted(self.tools.items())]}
            elif method == "tools/call":
                params = message.get("params") or {}
                tool = self.tools.get(params.get("name"))
                if tool is None:
                    raise McpError(-32602, f"unknown tool '{params.get('name')}'")
                try:
                    value = tool["fn"](params.get("arguments") or {})
                    text = value if isinstance(value, str) else json.dumps(value)
                    result = {"content": [{"type": "text", "text": text}], "isError": False}
                except McpError:
                    raise
                except Exception as e:            # a failing tool is a result, not a protocol error
                    result = {"content": [{"type": "text", "text": f"{type(e).__name__}: {e}"}], "isError": True}
            else:
                raise McpError(-32601, f"method '{method}' is not supported")
        except McpError as e:
            if mid is None:
                return None
            return {"jsonrpc": "2.0", "id": mid, "error": {"code": e.code, "message": e.message}}
        if mid is None:
            return None
        return {"jsonrpc": "2.0", "id": mid, "result": result}

    def serve(self, reader: IO[str], writer: IO[str]) -> None:
        for line in reader:
            line = line.strip()
            if not line:
                continue
            try:
                message = json.loads(line)
            except ValueError:
                response = {"jsonrpc": "2.0", "id": None, "error": {"code": -32700, "message": "parse error"}}
            else:
                response = self.handle(message)
            if response is not None:
                writer.write(json.dumps(response, ensure_ascii=False) + "\n")
                writer.flush()


# --------------------------------------------------------------------------- HTTP transport for the server
def serve_http(server: McpServer, host: str = "127.0.0.1", port: int = 0, token: Optional[str] = None):
    """The same server over HTTP: ``POST /mcp`` carries one JSON-RPC message (or a batch) and gets the response(s) as
    ``application/json``; notifications get ``202``. ``token`` asks for ``Authorization: Bearer <token>``. Returns the
    running ``ThreadingHTTPServer`` (``.server_address`` holds the bound port; ``.shutdown()`` stops it).

    Reference: the MCP server's http mode (src/Idrak.Mcp)."""
    import threading
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *args):          # quiet
            pass

        def _send(self, code: int, body: Optional[bytes] = None):
            self.send_response(code)
            if body is not None:
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            if body is not None:
                self.wfile.write(body)

        def do_POST(self):
            if self.path.rstrip("/") != "/mcp":
                return self._send(404)
            if token is not None and self.headers.get("Authorization") != f"Bearer {token}":
                return self._send(401, b'{"error": "missing or wrong bearer token"}')
            try:
                n = int(self.headers.get("Content-Length", "0"))
                message = json.loads(self.rfile.read(n) or b"null")
            except ValueError:
                return self._send(400, json.dumps({"jsonrpc": "2.0", "id": None,
                                                   "error": {"code": -32700, "message": "parse error"}}).encode())
            if isinstance(message, list):
                out = [r for r in (server.handle(m) for m in message) if r is not None]
                return self._send(200, json.dumps(out).encode()) if out else self._send(202)
            response = server.handle(message) if isinstance(message, dict) else {
                "jsonrpc": "2.0", "id": None, "error": {"code": -32600, "message": "not a JSON-RPC 2.0 request"}}
            if response is None:
                return self._send(202)
            self._send(200, json.dumps(response, ensure_ascii=False).encode())

    httpd = ThreadingHTTPServer((host, port), Handler)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    return httpd


# --------------------------------------------------------------------------- client
class McpClient:
    """Talks to an MCP server - a child process over stdio (``McpClient.stdio([...command...])``), an HTTP endpoint
    (``McpClient.http(url)``) or an in-process ``McpServer`` (``McpClient.local(server)``) - and exposes its tools:
    ``list_tools()``, ``call(name, **arguments)`` and ``as_tool_functions()`` (plain callables with the tool's name and
    description, the shape the agent loop of ``text.tool_calls`` takes).

    Reference: the MCP client tools of src/Idrak.Mcp."""

    def __init__(self, send: Callable[[dict], Optional[dict]], close: Optional[Callable[[], None]] = None):
        self._send, self._close = send, close
        self._next = 0
        self.server_info: dict = {}
        self._tools: Optional[List[dict]] = None

    # ------------------------------------------------------------------ transports
    @classmethod
    def local(cls, server: McpServer) -> "McpClient":
        return cls(server.handle).initialize()

    @classmethod
    def http(cls, url: str, token: Optional[str] = None, timeout: float = 60.0) -> "McpClient":
        import urllib.request

        def send(message: dict) -> Optional[dict]:
            req = urllib.request.Request(url, data=json.dumps(message).encode(), method="POST",
                                         headers={"Content-Type": "application/json"})
            if token is not None:
                req.add_header("Authorization", f"Bearer {token}")
            with urllib.request.urlopen(req, timeout=timeout) as r:
                body = r.read()
                return json.loads(body) if r.status == 200 and body else None
        return cls(send).initialize()

    @classmethod
    def stdio(cls, command: List[str], timeout: float = 60.0) -> "McpClient":
        import subprocess
        proc = subprocess.Popen(command, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)

        def send(message: dict) -> Optional[dict]:
            proc.stdin.write(json.dumps(message) + "\n")
            proc.stdin.flush()
            if "id" not in message:
                return None
            line = proc.stdout.readline()
            if not line:
                raise McpError(-32000, "the server closed its output")
            return json.loads(line)

        def close():
            try:
                proc.stdin.close()
                proc.wait(timeout=5)
            except Exception:
                proc.kill()
        return cls(send, close).initialize()

    # ------------------------------------------------------------------ protocol
    def _request(self, method: str, params: Optional[dict] = None) -> dict:
        self._next += 1
        message = {"jsonrpc": "2.0", "id": self._next, "method": method}
        if params is not None:
            message["params"] = params
        response = self._send(message)
        if response is None or response.get("id") != self._next:
            raise McpError(-32000, f"no response to '{method}'")
        if "error" in response:
            raise McpError(int(response["error"].get("code", -32000)), str(response["error"].get("message", "")))
        return response["result"]

    def initialize(self) -> "McpClient":
        result = self._request("initialize", {"protocolVersion": PROTOCOL, "capabilities": {},
                                              "clientInfo": {"name": "idrak-b200", "version": "0.1.0"}})
        self.server_info = result.get("serverInfo", {})
        self._send({"jsonrpc": "2.0", "method": "notifications/initialized"})
        return self

    def ping(self) -> bool:
        return self._request("ping") == {}

    def list_tools(self, refresh: bool = False) -> List[dict]:
        if self._tools is None or refresh:
            self._tools = list(self._request("tools/list").get("tools", []))
        return self._tools

    def call(self, name: str, **arguments) -> str:
        """The text of the tool's result; a tool that failed raises ``McpError`` with its message."""
        result = self._request("tools/call", {"name": name, "arguments": arguments})
        text = "".join(c.get("text", "") for c in result.get("content", []) if c.get("type") == "text")
        if result.get("isError"):
            raise McpError(-32001, text)
        return text

    def as_tool_functions(self) -> Dict[str, Callable[..., str]]:
        out: Dict[str, Callable[..., str]] = {}
        for t in self.list_tools():
            def fn(_name=t["name"], **arguments):
                return self.call(_name, **arguments)
            fn.__name__, fn.__doc__ = t["name"], t.get("description", "")
            fn.schema = t.get("inputSchema", {})
            out[t["name"]] = fn
        return out

    def close(self) -> None:
        if self._close is not None:
            self._close()
            self._close = None
