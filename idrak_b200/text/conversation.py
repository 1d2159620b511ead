"""Multi-turn conversations with server-side tool rounds: the history lives here, each ``say`` renders it through the
model's chat template, and when the model answers with tool calls that name registered tools, those are run and their
results appended as ``tool`` messages before the model is asked again - until it answers in text or the round limit is
reached.

    chat = Conversation(generator, system="You are terse.")
    chat.add_tool("add", "Add two numbers.", {"type": "object", "properties": {"a": {"type": "number"}, "b": {"type": "number"}}},
                  lambda a, b: a + b)
    reply = chat.say("What is 2 + 3?")          # GenerationResult of the final text answer
    chat.messages                                 # the whole exchange, tool rounds included

``generator`` is anything with ``chat(messages, options, tools) -> result`` whose result has ``text``, ``tool_calls``
(objects with ``name`` and ``arguments``) and ``finish_reason`` - the ``TextGenerator`` of this package, or the
inference engine's chat models.

Reference: ChatGenerator's server-side tool rounds and Conversation (src/Idrak.Text/Generation/ChatGenerator.cs:127,
Conversation.cs).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional


@dataclass
class Tool:
    name: str
    description: str
    parameters: dict
    fn: Callable[..., Any]

    def schema(self) -> dict:
        return {"type": "function", "function": {"name": self.name, "description": self.description, "parameters": self.parameters}}


@dataclass
class ToolRound:
    name: str
    arguments: dict
    result: str
    failed: bool = False


class Conversation:
    def __init__(self, generator, system: Optional[str] = None, options=None, max_tool_rounds: int = 4):
        self.generator, self.options, self.max_tool_rounds = generator, options, max_tool_rounds
        self.system = system
        self.messages: List[Dict[str, Any]] = []
        self.tools: Dict[str, Tool] = {}
        self.rounds: List[ToolRound] = []
        self.reset()

    def reset(self) -> None:
        self.messages = [{"role": "system", "content": self.system}] if self.system else []
        self.rounds = []

    def add_tool(self, name: str, description: str, parameters: dict, fn: Callable[..., Any]) -> None:
        self.tools[name] = Tool(name, description, parameters, fn)

    def _run_tool(self, name: str, arguments) -> ToolRound:
        args = arguments
        if isinstance(args, str):
            try:
                args = json.loads(args) if args.strip() else {}
            except ValueError:
                return ToolRound(name, {}, f"error: the arguments are not JSON: {arguments[:200]}", True)
        tool = self.tools.get(name)
        if tool is None:
            return ToolRound(name, args, f"error: there is no tool '{name}'; tools: {', '.join(sorted(self.tools)) or 'none'}", True)
        try:
            value = tool.fn(**args) if isinstance(args, dict) else tool.fn(args)
        except Exception as e:                    # the model sees the failure and can try again
            return ToolRound(name, args, f"error: {type(e).__name__}: {e}", True)
        return ToolRound(name, args, value if isinstance(value, str) else json.dumps(value, ensure_ascii=False))

    def say(self, text: str, options=None):
        """Add a user message and return the model's final answer (after any tool rounds)."""
        self.messages.append({"role": "user", "content": text})
        schemas = [t.schema() for t in self.tools.values()] or None
        result = None
        for round_index in range(self.max_tool_rounds + 1):
            result = self.generator.chat(self.messages, options or self.options, schemas)
            calls = list(getattr(result, "tool_calls", None) or [])
            if not calls or not self.tools or round_index == self.max_tool_rounds:
                self.messages.append({"role": "assistant", "content": result.text})
                return result
            ids = [getattr(c, "id", None) or f"call_{len(self.rounds) + i}" for i, c in enumerate(calls)]
            self.messages.append({"role": "assistant", "content": result.text or "", "tool_calls": [
                {"id": ids[i], "type": "function",
                 "function": {"name": c.name, "arguments": c.arguments if isinstance(c.arguments, str) else json.dumps(c.arguments)}}
                for i, c in enumerate(calls)]})
            for i, c in enumerate(calls):
                done = self._run_tool(c.name, c.arguments)
                self.rounds.append(done)
                self.messages.append({"role": "tool", "name": c.name, "content": done.result, "tool_call_id": ids[i]})
        return result

    def transcript(self) -> str:
        lines = []
        for m in self.messages:
            if m.get("tool_calls"):
                for c in m["tool_calls"]:
                    lines.append(f"assistant -> {c['function']['name']}({c['function']['arguments']})")
                if m.get("content"):
                    lines.append(f"assistant: {m['content']}")
            else:
                lines.append(f"{m['role']}: {m['content']}")
        return "\n".join(lines)
