"""A Model Context Protocol server over stdio: the inference engine's models as tools an MCP client can call.

Speaks JSON-RPC 2.0, one message per line: ``initialize``, ``ping``, ``tools/list``, ``tools/call``. Every text /
chat model becomes a ``generate_<name>`` tool (prompt or messages in, text out); every model that can embed a
``embed_<name>`` tool; extra tools can be registered as plain Python callables with a JSON schema.

    McpServer(engine).serve(sys.stdin, sys.stdout)

Reference: the MCP server of the reference (src/Idrak.Mcp: tools over the engine, stdio transport).
"""
from __future__ import annotations

import json
from typing import Any, Callable, Dict, IO, Optional

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
