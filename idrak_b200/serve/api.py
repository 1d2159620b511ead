"""HTTP face of the inference engine (FastAPI): the ``/v1`` completions API, the ``/api`` chat routes, predictor
routes and a status page.

``/v1``: ``GET /models``, ``POST /chat/completions``, ``POST /completions``, ``POST /embeddings`` with
server-sent-event streaming. Sampling fields taken: temperature, top_p, top_k, min_p, repeat_penalty,
presence_penalty, frequency_penalty, seed, max_tokens | max_completion_tokens, stop; ``tool_choice`` only "auto" or
"none". A field this server does not implement is refused with a message that names it rather than ignored.
Errors have the shape ``{"error": {"message", "type", "code"}}``; a full queue answers 429, a queue timeout 504.

Reference: src/Idrak.AspNetCore/CompletionsApi.cs:90-94 (routes), :754-840 (accepted and refused fields), :654 (error
body); src/Idrak.AspNetCore/IdrakEndpoints.cs:110-262 (predict, chat, tags, ps, version, status).
"""
from __future__ import annotations

import json
import time
import uuid
from typing import Any, Dict, Iterator, List, Optional

from starlette.concurrency import run_in_threadpool
from starlette.requests import Request

from .engine import GenerationOptions
from .inference_engine import InferenceEngine, InferenceQueueFull, InferenceTimeout

VERSION = "0.1.0"


class ApiError(Exception):
    def __init__(self, status: int, message: str, code: Optional[str] = None):
        super().__init__(message)
        self.status, self.message, self.code = status, message, code

    def body(self) -> dict:
        kind = ("server_error" if self.status >= 500 else "not_found_error" if self.status == 404
                else "request_too_large" if self.status == 413 else "invalid_request_error")
        return {"error": {"message": self.message, "type": kind, "code": self.code}}


_REFUSED_CHAT = {
    "n": lambda v: v not in (None, 1), "logprobs": lambda v: bool(v), "top_logprobs": lambda v: bool(v),
    "logit_bias": lambda v: bool(v), "response_format": lambda v: isinstance(v, dict) and v.get("type", "text") != "text",
    "json_schema": lambda v: v is not None, "audio": lambda v: v is not None,
    "modalities": lambda v: isinstance(v, list) and any(m != "text" for m in v),
    "parallel_tool_calls": lambda v: False, "functions": lambda v: bool(v), "function_call": lambda v: v is not None,
}
_REFUSED_COMPLETION = {
    "n": lambda v: v not in (None, 1), "best_of": lambda v: v not in (None, 1), "echo": lambda v: bool(v),
    "suffix": lambda v: v not in (None, ""), "logprobs": lambda v: v not in (None, 0, False),
    "logit_bias": lambda v: bool(v),
}


def _refuse(body: dict, table: dict) -> None:
    for key, bad in table.items():
        if key in body and bad(body[key]):
            raise ApiError(400, f"'{key}' is not supported by this server (got {json.dumps(body[key])[:80]})",
                           "unsupported_parameter")


def _number(body, key, kind=float, low=None, high=None):
    if key not in body or body[key] is None:
        return None
    v = body[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ApiError(400, f"'{key}' must be a number")
    if (low is not None and v < low) or (high is not None and v > high):
        raise ApiError(400, f"'{key}' must be between {low} and {high}")
    return kind(v)


def options_from_body(body: dict, default_max_tokens: int = 512) -> GenerationOptions:
    """The request's sampling fields over neutral defaults (no repetition penalty unless asked)."""
    o = GenerationOptions(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, max_tokens=default_max_tokens)
    for key, field, kind, low, high in (
            ("temperature", "temperature", float, 0.0, 2.0), ("top_p", "top_p", float, 0.0, 1.0),
            ("top_k", "top_k", int, 0, None), ("min_p", "min_p", float, 0.0, 1.0),
            ("repeat_penalty", "repeat_penalty", float, 0.0, None), ("presence_penalty", "presence_penalty", float, -2.0, 2.0),
            ("frequency_penalty", "frequency_penalty", float, -2.0, 2.0), ("seed", "seed", int, None, None)):
        v = _number(body, key, kind, low, high)
        if v is not None:
            setattr(o, field, v)
    mt = _number(body, "max_completion_tokens", int, 1, None) or _number(body, "max_tokens", int, 1, None)
    if mt is not None:
        o.max_tokens = mt
    stop = body.get("stop")
    if isinstance(stop, str):
        o.stop = (stop,)
    elif isinstance(stop, list):
        if not all(isinstance(s, str) for s in stop):
            raise ApiError(400, "'stop' must be a string or an array of strings")
        o.stop = tuple(stop)
    elif stop is not None:
        raise ApiError(400, "'stop' must be a string or an array of strings")
    return o


def _usage(res) -> dict:
    return {"prompt_tokens": res.prompt_tokens, "completion_tokens": res.completion_tokens,
            "total_tokens": res.prompt_tokens + res.completion_tokens}


def _finish(reason: Optional[str]) -> str:
    return {"stop": "stop", "tool_calls": "tool_calls", "length": "length", "repeat": "stop"}.get(reason or "stop", "stop")


def _sse(obj) -> str:
    return "data: " + (obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)) + "\n\n"


def _guard(call):
    """Run an engine call, turning engine conditions into API errors."""
    try:
        return call()
    except InferenceQueueFull as e:
        raise ApiError(429, str(e), "queue_full")
    except InferenceTimeout as e:
        raise ApiError(504, str(e), "timeout")
    except KeyError as e:
        raise ApiError(404, str(e.args[0]) if e.args else "not found", "model_not_found")
    except (ValueError, TypeError) as e:
        raise ApiError(400, str(e))


def create_app(engine: InferenceEngine, default_model: Optional[str] = None, default_max_tokens: int = 512):
    from fastapi import FastAPI
    from fastapi.responses import JSONResponse, StreamingResponse

    app = FastAPI(title="idrak-b200", version=VERSION)
    created = int(time.time())

    @app.exception_handler(ApiError)
    async def _api_error(_request, exc: ApiError):
        return JSONResponse(exc.body(), status_code=exc.status)

    async def _json(request: Request) -> dict:
        try:
            body = await request.json()
        except Exception:
            raise ApiError(400, "the request body is not valid JSON")
        if not isinstance(body, dict):
            raise ApiError(400, "the request body must be a JSON object")
        return body

    def _model_name(body: dict, kinds) -> str:
        name = body.get("model") or default_model
        if not name:
            names = engine.names()
            if len(names) == 1:
                return names[0]
            raise ApiError(400, "'model' is required")
        if name not in engine.names():
            raise ApiError(404, f"The model '{name}' does not exist", "model_not_found")
        if engine.model(name).settings.kind not in kinds:
            raise ApiError(400, f"The model '{name}' cannot serve this route (it is a "
                                f"{engine.model(name).settings.kind} model)")
        return name

    # ------------------------------------------------------------------ /v1
    @app.get("/v1/models")
    def models():
        return {"object": "list", "data": [{"id": n, "object": "model", "created": created, "owned_by": "idrak"}
                                           for n in engine.names()]}

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        body = await _json(request)
        _refuse(body, _REFUSED_CHAT)
        name = _model_name(body, ("chat",))
        messages = body.get("messages")
        if not isinstance(messages, list) or not messages:
            raise ApiError(400, "'messages' must be a non-empty array")
        for m in messages:
            if not isinstance(m, dict) or "role" not in m:
                raise ApiError(400, "every message needs a 'role'")
        tools = body.get("tools") or None
        choice = body.get("tool_choice", "auto")
        if choice not in ("auto", "none", None):
            raise ApiError(400, "'tool_choice' supports only \"auto\" and \"none\"", "unsupported_parameter")
        if choice == "none":
            tools = None
        opts = options_from_body(body, default_max_tokens)
        rid = "chatcmpl-" + uuid.uuid4().hex[:24]
        if not body.get("stream"):
            res = await run_in_threadpool(_guard, lambda: engine.chat(name, messages, opts, tools))
            msg: Dict[str, Any] = {"role": "assistant", "content": res.text or (None if res.tool_calls else "")}
            if res.tool_calls:
                msg["tool_calls"] = [c.to_openai() for c in res.tool_calls]
            return {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": name,
                    "choices": [{"index": 0, "message": msg, "finish_reason": _finish(res.finish_reason)}],
                    "usage": _usage(res)}
        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
        from ..generation.text_generator import GenerationResult
        res = GenerationResult()
        pieces = await run_in_threadpool(_guard, lambda: engine.stream(name, messages, opts, tools, res))
        parser = engine.model(name).run(lambda g: g.template.parser(tools)) if tools else None

        def chunk(delta, finish=None):
            return {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()), "model": name,
                    "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}

        def events() -> Iterator[str]:
            yield _sse(chunk({"role": "assistant", "content": ""}))
            n_calls = 0
            try:
                for piece in pieces:
                    d = parser.feed(piece) if parser else None
                    text = d.content if d else piece
                    if text:
                        yield _sse(chunk({"content": text}))
                    for c in (d.tool_calls if d else []):
                        yield _sse(chunk({"tool_calls": [c.to_openai(n_calls)]}))
                        n_calls += 1
                if parser:
                    d = parser.finish()
                    if d.content:
                        yield _sse(chunk({"content": d.content}))
                    for c in d.tool_calls:
                        yield _sse(chunk({"tool_calls": [c.to_openai(n_calls)]}))
                        n_calls += 1
            except Exception as e:            # the stream is already open: report in-band and stop
                yield _sse({"error": {"message": str(e), "type": "server_error", "code": None}})
                yield _sse("[DONE]")
                return
            reason = "tool_calls" if n_calls and res.finish_reason == "stop" else _finish(res.finish_reason)
            yield _sse(chunk({}, reason))
            if include_usage:
                last = chunk({}, None)
                last["choices"], last["usage"] = [], _usage(res)
                yield _sse(last)
            yield _sse("[DONE]")

        return StreamingResponse(events(), media_type="text/event-stream")

    @app.post("/v1/completions")
    async def completions(request: Request):
        body = await _json(request)
        _refuse(body, _REFUSED_COMPLETION)
        name = _model_name(body, ("text", "chat"))
        prompt = body.get("prompt")
        if isinstance(prompt, list) and len(prompt) == 1 and isinstance(prompt[0], str):
            prompt = prompt[0]
        if isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
            pass                                   # a token array
        elif not isinstance(prompt, str) or prompt == "":
            raise ApiError(400, "'prompt' must be a non-empty string or an array of token ids")
        opts = options_from_body(body, default_max_tokens)
        rid = "cmpl-" + uuid.uuid4().hex[:24]
        if not body.get("stream"):
            res = await run_in_threadpool(_guard, lambda: engine.generate(name, prompt, opts))
            return {"id": rid, "object": "text_completion", "created": int(time.time()), "model": name,
                    "choices": [{"index": 0, "text": res.text, "finish_reason": _finish(res.finish_reason),
                                 "logprobs": None}], "usage": _usage(res)}
        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
        from ..generation.text_generator import GenerationResult
        res = GenerationResult()
        pieces = await run_in_threadpool(_guard, lambda: engine.stream(name, prompt, opts, None, res))

        def events():
            base = {"id": rid, "object": "text_completion", "created": int(time.time()), "model": name}
            for piece in pieces:
                yield _sse({**base, "choices": [{"index": 0, "text": piece, "finish_reason": None}]})
            yield _sse({**base, "choices": [{"index": 0, "text": "", "finish_reason": _finish(res.finish_reason)}]})
            if include_usage:
                yield _sse({**base, "choices": [], "usage": _usage(res)})
            yield _sse("[DONE]")

        return StreamingResponse(events(), media_type="text/event-stream")

    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        body = await _json(request)
        if body.get("encoding_format", "float") != "float":
            raise ApiError(400, "'encoding_format' supports only \"float\"", "unsupported_parameter")
        if body.get("dimensions") is not None:
            raise ApiError(400, "'dimensions' is not supported by this server", "unsupported_parameter")
        name = _model_name(body, ("embed", "text", "chat"))
        texts = body.get("input")
        if isinstance(texts, str):
            texts = [texts]
        if not isinstance(texts, list) or not texts or not all(isinstance(t, str) and t for t in texts):
            raise ApiError(400, "'input' must be a non-empty string or an array of non-empty strings")
        vectors = await run_in_threadpool(_guard, lambda: engine.embed(name, texts))
        tokens = sum(engine.count_tokens(name, t) for t in texts)
        return {"object": "list", "model": name,
                "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vectors)],
                "usage": {"prompt_tokens": tokens, "total_tokens": tokens}}

    _add_native_routes(app, engine, default_model, default_max_tokens, _json, _model_name)
    return app


def _ollama_options(body: dict, default_max_tokens: int) -> GenerationOptions:
    """``options`` of the /api routes: the reference's GenerationOptions names (snake case), its defaults."""
    src = body.get("options") or {}
    o = GenerationOptions(max_tokens=default_max_tokens)
    names = {"temperature": float, "top_k": int, "top_p": float, "min_p": float, "repeat_penalty": float,
             "repeat_last_n": int, "presence_penalty": float, "frequency_penalty": float, "seed": int}
    for k, v in src.items():
        if k in names:
            setattr(o, k, names[k](v))
        elif k == "num_predict":
            o.max_tokens = int(v) if int(v) > 0 else 0
        elif k == "stop":
            o.stop = tuple(v if isinstance(v, list) else [v])
        elif k == "num_ctx":
            pass                                   # the context is fixed by the loaded model
        else:
            raise ApiError(400, f"option '{k}' is not supported by this server", "unsupported_parameter")
    return o


def _add_native_routes(app, engine: InferenceEngine, default_model, default_max_tokens, _json, _model_name):
    from fastapi.responses import StreamingResponse

    def now():
        return time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())

    def describe(name: str) -> dict:
        h = engine.model(name)
        size = params = ctx = 0
        if h.loaded and h.settings.kind in ("text", "chat", "embed"):
            g = h._copies[0]
            params = sum(p.numel() for p in g.engine.runner.model.parameters())
            size = sum(p.numel() * p.element_size() for p in g.engine.runner.model.parameters())
            ctx = g.engine.spec.max_positions
        return {"name": name, "model": name, "modified_at": now(), "size": size,
                "details": {"format": "idrak", "family": h.settings.kind, "parameter_size": _count(params),
                            "context_length": ctx}}

    @app.post("/api/chat")
    async def api_chat(request: Request):
        body = await _json(request)
        name = _model_name(body, ("chat",))
        messages = body.get("messages")
        if not isinstance(messages, list) or not messages:
            raise ApiError(400, "'messages' must be a non-empty array")
        if body.get("format") not in (None, ""):
            raise ApiError(400, "'format' is not supported by this server", "unsupported_parameter")
        opts = _ollama_options(body, default_max_tokens)
        tools = body.get("tools") or None
        t0 = time.perf_counter()
        if body.get("stream", True) is False:
            res = await run_in_threadpool(_guard, lambda: engine.chat(name, messages, opts, tools))
            msg = {"role": "assistant", "content": res.text}
            if res.tool_calls:
                msg["tool_calls"] = [{"function": {"name": c.name, "arguments": json.loads(c.arguments)}}
                                     for c in res.tool_calls]
            return {"model": name, "created_at": now(), "message": msg, "done": True,
                    "done_reason": res.finish_reason or "stop", "total_duration": int((time.perf_counter() - t0) * 1e9),
                    "prompt_eval_count": res.prompt_tokens, "eval_count": res.completion_tokens}
        from ..generation.text_generator import GenerationResult
        res = GenerationResult()
        pieces = await run_in_threadpool(_guard, lambda: engine.stream(name, messages, opts, None, res))

        def lines():
            for piece in pieces:
                yield json.dumps({"model": name, "created_at": now(), "message": {"role": "assistant", "content": piece},
                                  "done": False}) + "\n"
            yield json.dumps({"model": name, "created_at": now(), "message": {"role": "assistant", "content": ""},
                              "done": True, "done_reason": res.finish_reason or "stop",
                              "total_duration": int((time.perf_counter() - t0) * 1e9),
                              "prompt_eval_count": res.prompt_tokens, "eval_count": res.completion_tokens}) + "\n"
        return StreamingResponse(lines(), media_type="application/x-ndjson")

    @app.post("/api/generate")
    async def api_generate(request: Request):
        body = await _json(request)
        name = _model_name(body, ("text", "chat"))
        prompt = body.get("prompt")
        if not isinstance(prompt, str) or not prompt:
            raise ApiError(400, "'prompt' must be a non-empty string")
        opts = _ollama_options(body, default_max_tokens)
        res = await run_in_threadpool(_guard, lambda: engine.generate(name, prompt, opts))
        return {"model": name, "created_at": now(), "response": res.text, "done": True,
                "done_reason": res.finish_reason or "stop", "prompt_eval_count": res.prompt_tokens,
                "eval_count": res.completion_tokens}

    @app.get("/api/tags")
    def api_tags():
        return {"models": [describe(n) for n in engine.names() if engine.model(n).settings.kind != "predictor"]}

    @app.get("/api/ps")
    def api_ps():
        out = []
        for n in engine.names():
            h = engine.model(n)
            if h.loaded and h.settings.kind != "predictor":
                d = describe(n)
                st = h.status()
                d["expires_in"] = st["expires_in"]
                d["size_vram"] = d["size"]
                out.append(d)
        return {"models": out}

    @app.get("/api/version")
    def api_version():
        return {"version": VERSION}

    @app.post("/predict/{name}")
    async def predict(name: str, request: Request):
        import torch
        body = await _json(request)
        if name not in engine.names("predictor"):
            raise ApiError(404, f"no predictor named '{name}'", "model_not_found")
        if "input" not in body:
            raise ApiError(400, "'input' is required")
        y = await run_in_threadpool(_guard, lambda: engine.predict(name, torch.tensor(body["input"], dtype=torch.float32)))
        return {"output": y.tolist() if hasattr(y, "tolist") else y}

    @app.post("/predict/{name}/batch")
    async def predict_batch(name: str, request: Request):
        import torch
        body = await _json(request)
        if name not in engine.names("predictor"):
            raise ApiError(404, f"no predictor named '{name}'", "model_not_found")
        inputs = body.get("inputs")
        if not isinstance(inputs, list) or not inputs:
            raise ApiError(400, "'inputs' must be a non-empty array")
        ys = [await run_in_threadpool(_guard, lambda x=x: engine.predict(name, torch.tensor(x, dtype=torch.float32))) for x in inputs]
        return {"outputs": [y.tolist() if hasattr(y, "tolist") else y for y in ys]}

    @app.get("/status")
    def status():
        import torch
        devices = []
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                free, total = torch.cuda.mem_get_info(i)
                devices.append({"device": f"cuda:{i}", "name": torch.cuda.get_device_name(i),
                                "memory_in_use": total - free, "memory_cached": torch.cuda.memory_reserved(i),
                                "memory_limit": total})
        return {"models": engine.statuses(), "devices": devices}


def _count(n: int) -> str:
    for unit, size in (("B", 1e9), ("M", 1e6), ("K", 1e3)):
        if n >= size:
            return f"{n / size:.1f}{unit}"
    return str(n)


def serve(engine: InferenceEngine, host: str = "127.0.0.1", port: int = 8000, **kw) -> None:
    """Run the API under uvicorn until interrupted."""
    import uvicorn
    uvicorn.run(create_app(engine, **kw), host=host, port=port, log_level="info")
