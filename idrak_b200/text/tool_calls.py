"""Finding tool calls in a model's reply while it streams.

A parser is fed text pieces and returns, for each, the answer text that is safe to show and the calls completed so
far. Text that may still turn out to be the start of a marker is held back until it can be decided; a call body
that does not parse stays answer text. Formats are registered by name; a chat template's format is detected from
its text.

Built-in formats:
  json      ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` (also a bare JSON object / list as the
            whole answer when it names one of the request's tools)
  llama3    bare JSON with ``"parameters"``, optionally after ``<|python_tag|>``, calls separated by ``;``
  mistral   ``[TOOL_CALLS][{"name": ..., "arguments": {...}}, ...]`` running to the end of the turn
  pythonic  ``[get_weather(city="Paris"), other()]`` as the whole answer

Reference: MarkedToolCallParser and the json / pythonic parsers (src/Idrak.Abstraction/Generation/ToolCallParsers.cs:19,207,252),
the format registry and detection (src/Idrak.Abstraction/Generation/ToolCallFormats.cs:99).
"""
from __future__ import annotations

import ast
import json
import uuid
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

PYTHON_TAG = "<|python_tag|>"


@dataclass
class ToolCall:
    name: str
    arguments: str                       # a JSON object, as text
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_openai(self, index: Optional[int] = None) -> dict:
        d = {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}
        if index is not None:
            d["index"] = index
        return d


@dataclass
class ChatDelta:
    content: str = ""
    tool_calls: List[ToolCall] = field(default_factory=list)


def _held_suffix(text: str, marker: str) -> int:
    """Length of the longest proper prefix of ``marker`` that ends ``text`` (it may still become the marker)."""
    for n in range(min(len(marker) - 1, len(text)), 0, -1):
        if text.endswith(marker[:n]):
            return n
    return 0


class MarkedToolCallParser:
    """Answer text, then calls between ``open`` and ``close`` (``close`` may be empty or missing: the calls run to
    the end of the turn). With ``whole_answer`` the reply itself may be a call, decided from how it starts."""

    open: str = ""
    close: str = ""
    whole_answer: bool = False

    def __init__(self, tools: Sequence[dict] = ()):
        self.tools = list(tools)
        self.tool_names = {(t.get("function") or t).get("name") for t in self.tools}
        self._pending = ""
        self._mode = "text"              # text | call | whole
        self._decided = not self.whole_answer
        self._seen_text = False

    # ---- to override
    def parse(self, body: str) -> Optional[List[ToolCall]]:
        raise NotImplementedError

    def decide(self, start: str) -> int:
        """From the answer's first characters (no leading whitespace): 1 a call, 0 not, -1 need more text."""
        return 0

    # ---- streaming
    def feed(self, text: str) -> ChatDelta:
        self._pending += text
        return self._drain(False)

    def finish(self) -> ChatDelta:
        return self._drain(True)

    def _drain(self, final: bool) -> ChatDelta:
        out = ChatDelta()
        while True:
            if self._mode == "whole":
                if not final:
                    return out
                calls = self.parse(self._pending)
                if calls is None:
                    out.content += self._pending
                else:
                    out.tool_calls += calls
                self._pending = ""
                return out
            if self._mode == "text":
                if not self._decided:
                    start = self._pending.lstrip()
                    verdict = self.decide(start) if start else -1
                    if verdict == -1 and not final:
                        return out
                    self._decided = True
                    if verdict == 1:
                        self._mode = "whole"
                        continue
                if self.open:
                    at = self._pending.find(self.open)
                    if at >= 0:
                        out.content += self._pending[:at]
                        self._pending = self._pending[at + len(self.open):]
                        self._mode = "call"
                        continue
                    hold = 0 if final else _held_suffix(self._pending, self.open)
                else:
                    hold = 0
                cut = len(self._pending) - hold
                out.content += self._pending[:cut]
                self._pending = self._pending[cut:]
                return out
            # call mode
            at = self._pending.find(self.close) if self.close else -1
            if at < 0 and not final:
                return out
            body = self._pending if at < 0 else self._pending[:at]
            rest = "" if at < 0 else self._pending[at + len(self.close):]
            calls = self.parse(body)
            if calls is None:
                out.content += self.open + body + (self.close if at >= 0 else "")
            else:
                out.tool_calls += calls
            self._pending, self._mode = rest, "text"
            if final and not rest:
                return out


def _call_from_json(obj, arguments_keys=("arguments", "parameters")) -> Optional[ToolCall]:
    if not isinstance(obj, dict):
        return None
    if isinstance(obj.get("function"), dict):
        obj = obj["function"]
    name = obj.get("name")
    if not isinstance(name, str) or not name:
        return None
    args = None
    for k in arguments_keys:
        if k in obj:
            args = obj[k]
            break
    if args is None:
        args = {}
    if isinstance(args, str):
        try:
            json.loads(args)
            text = args
        except ValueError:
            return None
    else:
        text = json.dumps(args, ensure_ascii=False)
    return ToolCall(name, text)


def _calls_from_json_text(body: str) -> Optional[List[ToolCall]]:
    body = body.strip()
    if body.startswith(PYTHON_TAG):
        body = body[len(PYTHON_TAG):].strip()
    if not body:
        return None
    try:
        parsed = [json.loads(body)]
    except ValueError:
        try:                                 # several objects separated by ';' or new lines
            parts = [p for p in body.replace("\n", ";").split(";") if p.strip()]
            parsed = [json.loads(p) for p in parts]
        except ValueError:
            return None
    flat = []
    for p in parsed:
        flat += p if isinstance(p, list) else [p]
    calls = [_call_from_json(p) for p in flat]
    if not calls or any(c is None for c in calls):
        return None
    return calls


class JsonToolCallParser(MarkedToolCallParser):
    open, close, whole_answer = "<tool_call>", "</tool_call>", True

    def parse(self, body):
        calls = _calls_from_json_text(body)
        if calls is not None and self._mode == "whole" and self.tool_names:
            if any(c.name not in self.tool_names for c in calls):
                return None              # a JSON answer that is not a call of this request's tools stays text
        return calls

    def decide(self, start):
        if start.startswith(PYTHON_TAG):
            return 1
        if len(start) < len(PYTHON_TAG) and PYTHON_TAG.startswith(start):
            return -1
        if not self.tools:
            return 0
        return 1 if start[0] in "{[" else 0


class Llama3ToolCallParser(JsonToolCallParser):
    open, close = "", ""


class MistralToolCallParser(MarkedToolCallParser):
    open, close = "[TOOL_CALLS]", ""

    def parse(self, body):
        return _calls_from_json_text(body)


def _python_value(node):
    return ast.literal_eval(node)


class PythonicToolCallParser(MarkedToolCallParser):
    open, close, whole_answer = "", "", True

    def decide(self, start):
        if start.startswith(PYTHON_TAG):
            return 1
        if start[0] != "[":
            return 0
        rest = start[1:].lstrip()
        if not rest:
            return -1
        return 1 if (rest[0].isalpha() or rest[0] == "_") else 0

    def parse(self, body):
        body = body.strip()
        if body.startswith(PYTHON_TAG):
            body = body[len(PYTHON_TAG):].strip()
        try:
            tree = ast.parse(body, mode="eval").body
        except SyntaxError:
            return None
        nodes = tree.elts if isinstance(tree, (ast.List, ast.Tuple)) else [tree]
        calls = []
        for n in nodes:
            if not isinstance(n, ast.Call) or n.args:
                return None
            parts, f = [], n.func
            while isinstance(f, ast.Attribute):
                parts.append(f.attr)
                f = f.value
            if not isinstance(f, ast.Name):
                return None
            name = ".".join([f.id] + parts[::-1])
            try:
                args = {k.arg: _python_value(k.value) for k in n.keywords if k.arg}
            except (ValueError, SyntaxError):
                return None
            if self.tool_names and name not in self.tool_names:
                return None
            calls.append(ToolCall(name, json.dumps(args, ensure_ascii=False)))
        return calls or None


_FORMATS: Dict[str, Callable[[Sequence[dict]], MarkedToolCallParser]] = {
    "json": JsonToolCallParser, "llama3": Llama3ToolCallParser, "mistral": MistralToolCallParser,
    "pythonic": PythonicToolCallParser,
}
_DETECTORS: List = [
    ("mistral", lambda t: "[TOOL_CALLS]" in t),
    ("pythonic", lambda t: "[func_name1(" in t or "pythonic" in t.lower()),
    ("llama3", lambda t: PYTHON_TAG in t or '"parameters"' in t),
    ("json", lambda t: True),
]


def register_tool_call_format(name: str, factory, detector=None) -> None:
    """Add (or replace) a format; ``detector(template_text) -> bool`` lets templates select it."""
    _FORMATS[name] = factory
    if detector is not None:
        _DETECTORS.insert(0, (name, detector))


def detect_format(template_text: Optional[str]) -> str:
    text = template_text or ""
    for name, hit in _DETECTORS:
        if hit(text):
            return name
    return "json"


def create_parser(name: str, tools: Sequence[dict] = ()) -> MarkedToolCallParser:
    if name not in _FORMATS:
        raise KeyError(f"Tool-call format '{name}' is not registered: add it with register_tool_call_format. "
                       f"Known: {', '.join(sorted(_FORMATS))}")
    return _FORMATS[name](tools)
