"""Chat messages -> prompt text through the model's own Jinja template (or a built-in one).

Templates run in a sandboxed Jinja2 environment with the helpers Hugging Face templates expect
(``raise_exception``, ``strftime_now``, ``tojson``). Messages are plain dicts: ``role``, ``content`` (a string or
a list of parts ``{"type": "text" | "image_url" | "input_audio", ...}``), optional ``tool_calls`` /
``tool_call_id`` / ``name``.

Reference: chat contracts and built-in templates (src/Idrak.Abstraction/Generation/Chat.cs:95-168), Jinja template
evaluation (src/Idrak/Generation/ChatTemplates).
"""
from __future__ import annotations

import datetime
import json
from typing import Any, Dict, List, Optional, Sequence

CHATML = (
    "{% for message in messages %}"
    "{{ '<|im_start|>' + message['role'] + '\n' + (message['content'] or '') + '<|im_end|>\n' }}"
    "{% endfor %}"
    "{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}"
)

PLAIN = (
    "{% for message in messages %}{{ message['role'] }}: {{ message['content'] }}\n{% endfor %}"
    "{% if add_generation_prompt %}assistant: {% endif %}"
)

BUILT_IN = {"chatml": CHATML, "plain": PLAIN}

_ENV = None


def _environment():
    global _ENV
    if _ENV is None:
        from jinja2.ext import loopcontrols
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(message):
            raise ValueError(message)

        def strftime_now(fmt):
            return datetime.datetime.now().strftime(fmt)

        def tojson(value, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
            return json.dumps(value, ensure_ascii=ensure_ascii, indent=indent, separators=separators,
                              sort_keys=sort_keys)

        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=[loopcontrols])
        env.globals["raise_exception"] = raise_exception
        env.globals["strftime_now"] = strftime_now
        env.filters["tojson"] = tojson
        _ENV = env
    return _ENV


def flatten_content(content: Any) -> str:
    """The text of a message's content; non-text parts are refused by type so nothing is dropped silently."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    out = []
    for part in content:
        kind = part.get("type")
        if kind == "text":
            out.append(part.get("text", ""))
        elif kind in ("image_url", "input_audio"):
            raise ValueError(f"this model takes text only: a '{kind}' content part cannot be used")
        else:
            raise ValueError(f"unknown content part type {kind!r}")
    return "".join(out)


def render_chat(messages: Sequence[Dict[str, Any]], template: Optional[str] = None, tools: Optional[List[dict]] = None,
                add_generation_prompt: bool = True, bos_token: str = "", eos_token: str = "", **extra) -> str:
    """Render the prompt for ``messages``. ``template`` is Jinja text, the name of a built-in one, or None (ChatML)."""
    text = BUILT_IN.get(template or "chatml", template)
    msgs = []
    for m in messages:
        m = dict(m)
        if not isinstance(m.get("content"), str):
            m["content"] = flatten_content(m.get("content"))
        msgs.append(m)
    tpl = _environment().from_string(text)
    return tpl.render(messages=msgs, tools=tools or None, add_generation_prompt=add_generation_prompt,
                      bos_token=bos_token, eos_token=eos_token, **extra)


class ChatTemplate:
    """A model's template with its special tokens bound, and the tool-call format its replies are parsed in."""

    def __init__(self, template: Optional[str] = None, bos_token: str = "", eos_token: str = "",
                 tool_call_format: Optional[str] = None):
        self.template, self.bos_token, self.eos_token = template, bos_token, eos_token
        from .tool_calls import detect_format
        self.tool_call_format = tool_call_format or detect_format(BUILT_IN.get(template or "chatml", template))

    @classmethod
    def for_tokenizer(cls, tokenizer) -> "ChatTemplate":
        def text(i):
            return tokenizer.decode([i], skip_special_tokens=False) if i is not None else ""
        eos = tokenizer.eos_token_ids[-1] if tokenizer.eos_token_ids else None
        return cls(tokenizer.chat_template, text(tokenizer.bos_token_id), text(eos))

    def render(self, messages, tools=None, add_generation_prompt=True, **extra) -> str:
        return render_chat(messages, self.template, tools, add_generation_prompt, self.bos_token, self.eos_token, **extra)

    def parser(self, tools: Optional[List[dict]] = None):
        from .tool_calls import create_parser
        return create_parser(self.tool_call_format, tools or [])
