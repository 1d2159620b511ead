"""A coding agent: a chat model that reads, searches, edits and writes files and runs allow-listed commands inside one
workspace folder, as tool rounds of a ``Conversation``.

``Workspace`` is the sandbox. Every path a tool receives is resolved against the workspace root and refused when it
leaves it (``..``, absolute paths, symbolic links that point outside); commands run without a shell, only when their
program is on the allow-list, in the workspace, with a time limit, a scrubbed environment and their output cut to a
size the model can read. Nothing here trusts the model: a refusal comes back to it as the tool's result, so it can try
something else.

``CodingAgent`` wires the workspace's tools into a conversation and reports what happened (answer, tool rounds, files
changed, commands run).

Reference: the coding agent sample and its sandboxes (samples/Idrak.Samples.CodingAgent/Program.cs,
src/Idrak.Reinforcement.Plugins/Coding).
"""
from __future__ import annotations

import fnmatch
import os
import re
import shlex
import subprocess
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

from .conversation import Conversation, ToolRound


class SandboxRefusal(Exception):
    """A tool call the workspace does not allow; its text goes back to the model."""


class Workspace:
    def __init__(self, root, allowed_commands: Sequence[str] = ("python", "python3", "pytest"), read_only: bool = False,
                 max_file_bytes: int = 256 * 1024, max_output_chars: int = 6000, command_timeout: float = 60.0):
        self.root = Path(root).resolve()
        if not self.root.is_dir():
            raise ValueError(f"workspace folder '{root}' does not exist")
        self.allowed_commands = tuple(allowed_commands)
        self.read_only = read_only
        self.max_file_bytes, self.max_output_chars, self.command_timeout = max_file_bytes, max_output_chars, command_timeout
        self.changed: List[str] = []
        self.commands: List[str] = []

    # ------------------------------------------------------------------ paths
    def resolve(self, path: str) -> Path:
        """The file inside the workspace that ``path`` names; refuses anything that would end up outside."""
        if not isinstance(path, str) or not path or "\x00" in path:
            raise SandboxRefusal("a path must be a non-empty string")
        p = Path(path)
        if p.is_absolute():
            raise SandboxRefusal(f"'{path}' is an absolute path; paths are relative to the workspace")
        full = (self.root / p).resolve()
        if full != self.root and self.root not in full.parents:
            raise SandboxRefusal(f"'{path}' leaves the workspace")
        return full

    def _relative(self, full: Path) -> str:
        return str(full.relative_to(self.root)).replace(os.sep, "/")

    def _files(self, pattern: str = "*"):
        for base, dirs, files in os.walk(self.root):
            dirs[:] = sorted(d for d in dirs if not d.startswith(".") and d != "__pycache__")
            for name in sorted(files):
                full = Path(base) / name
                rel = self._relative(full)
                if fnmatch.fnmatch(rel, pattern) or fnmatch.fnmatch(name, pattern):
                    yield full, rel

    # ------------------------------------------------------------------ tools
    def list_files(self, pattern: str = "*") -> str:
        rows = [f"{rel} ({full.stat().st_size} bytes)" for full, rel in self._files(pattern)]
        return "\n".join(rows[:400]) if rows else "no files match"

    def read_file(self, path: str, first_line: int = 1, last_line: int = 0) -> str:
        full = self.resolve(path)
        if not full.is_file():
            raise SandboxRefusal(f"there is no file '{path}'")
        if full.stat().st_size > self.max_file_bytes:
            raise SandboxRefusal(f"'{path}' is larger than {self.max_file_bytes} bytes; read a range of lines")
        lines = full.read_text(errors="replace").splitlines()
        lo = max(1, int(first_line))
        hi = len(lines) if not last_line else min(len(lines), int(last_line))
        body = "\n".join(f"{i:5d}  {lines[i - 1]}" for i in range(lo, hi + 1))
        return self._cut(body) if body else "(empty)"

    def search(self, text: str, pattern: str = "*", regex: bool = False) -> str:
        try:
            needle = re.compile(text if regex else re.escape(text))
        except re.error as e:
            raise SandboxRefusal(f"not a regular expression: {e}")
        hits = []
        for full, rel in self._files(pattern):
            if full.stat().st_size > self.max_file_bytes:
                continue
            try:
                for n, line in enumerate(full.read_text(errors="replace").splitlines(), 1):
                    if needle.search(line):
                        hits.append(f"{rel}:{n}: {line.strip()[:200]}")
                        if len(hits) >= 200:
                            return "\n".join(hits) + "\n(more matches not shown)"
            except OSError:
                continue
        return "\n".join(hits) if hits else "no matches"

    def _writable(self, path: str) -> Path:
        if self.read_only:
            raise SandboxRefusal("the workspace is read-only")
        full = self.resolve(path)
        if full == self.root or full.is_dir():
            raise SandboxRefusal(f"'{path}' is a folder")
        return full

    def write_file(self, path: str, content: str) -> str:
        full = self._writable(path)
        if len(content.encode()) > self.max_file_bytes:
            raise SandboxRefusal(f"the content is larger than {self.max_file_bytes} bytes")
        full.parent.mkdir(parents=True, exist_ok=True)
        full.write_text(content)
        self._note_change(full)
        return f"wrote {len(content)} characters to {self._relative(full)}"

    def edit_file(self, path: str, old: str, new: str) -> str:
        """Replace ``old`` by ``new``; ``old`` must occur exactly once, so that an edit cannot land in the wrong place."""
        full = self._writable(path)
        if not full.is_file():
            raise SandboxRefusal(f"there is no file '{path}'")
        text = full.read_text()
        count = text.count(old) if old else 0
        if count != 1:
            raise SandboxRefusal(f"the text to replace occurs {count} times in '{path}'; it must occur exactly once")
        full.write_text(text.replace(old, new, 1))
        self._note_change(full)
        return f"edited {self._relative(full)}"

    def _note_change(self, full: Path) -> None:
        rel = self._relative(full)
        if rel not in self.changed:
            self.changed.append(rel)

    def run(self, command: str) -> str:
        """Run one allow-listed program (no shell: no pipes, redirections or substitutions) in the workspace."""
        try:
            argv = shlex.split(command)
        except ValueError as e:
            raise SandboxRefusal(f"cannot split the command: {e}")
        if not argv:
            raise SandboxRefusal("empty command")
        program = argv[0]
        if os.path.basename(program) != program or program not in self.allowed_commands:
            raise SandboxRefusal(f"'{program}' is not an allowed command; allowed: {', '.join(self.allowed_commands)}")
        for a in argv[1:]:
            if a.startswith("/") or ".." in Path(a).parts:
                raise SandboxRefusal(f"argument '{a}' points outside the workspace")
        env = {"PATH": os.environ.get("PATH", ""), "HOME": str(self.root), "LANG": "C.UTF-8", "PYTHONDONTWRITEBYTECODE": "1"}
        self.commands.append(command)
        try:
            r = subprocess.run(argv, cwd=self.root, env=env, capture_output=True, text=True, timeout=self.command_timeout,
                               stdin=subprocess.DEVNULL)
        except subprocess.TimeoutExpired:
            return f"the command did not finish within {self.command_timeout:.0f} s and was stopped"
        except FileNotFoundError:
            raise SandboxRefusal(f"'{program}' is not installed")
        out = (r.stdout or "") + (("\n[stderr]\n" + r.stderr) if r.stderr else "")
        return f"exit code {r.returncode}\n{self._cut(out.strip())}"

    def _cut(self, text: str) -> str:
        if len(text) <= self.max_output_chars:
            return text
        half = self.max_output_chars // 2
        return text[:half] + f"\n... ({len(text) - 2 * half} characters left out) ...\n" + text[-half:]

    # ------------------------------------------------------------------ as tools of a conversation
    def tool_table(self) -> Dict[str, tuple]:
        s = lambda **props: {"type": "object", "properties": props, "required": [k for k, v in props.items() if v.pop("required", True)]}  # noqa: E731
        string, integer, boolean = {"type": "string"}, {"type": "integer", "required": False}, {"type": "boolean", "required": False}
        table = {
            "list_files": ("List files of the workspace (optional glob pattern).", s(pattern={**string, "required": False}), self.list_files),
            "read_file": ("Read a file with line numbers (optionally a range of lines).",
                          s(path=dict(string), first_line=dict(integer), last_line=dict(integer)), self.read_file),
            "search": ("Find lines that contain a text (or match a regular expression) in the workspace.",
                       s(text=dict(string), pattern={**string, "required": False}, regex=dict(boolean)), self.search),
        }
        if not self.read_only:
            table["write_file"] = ("Create or overwrite a file.", s(path=dict(string), content=dict(string)), self.write_file)
            table["edit_file"] = ("Replace a text that occurs exactly once in a file.",
                                  s(path=dict(string), old=dict(string), new=dict(string)), self.edit_file)
        if self.allowed_commands:
            table["run"] = (f"Run a command in the workspace (allowed programs: {', '.join(self.allowed_commands)}; no shell).",
                            s(command=dict(string)), self.run)
        return table


@dataclass
class AgentReport:
    answer: str
    rounds: List[ToolRound] = field(default_factory=list)
    files_changed: List[str] = field(default_factory=list)
    commands: List[str] = field(default_factory=list)
    refusals: int = 0


SYSTEM = ("You are a coding agent working in one folder. Look before you change: list and read files, search for what you "
          "need, make small exact edits, run the tests, and finish with a short account of what you did.")


class CodingAgent:
    def __init__(self, generator, workspace: Workspace, system: str = SYSTEM, options=None, max_tool_rounds: int = 16):
        self.workspace = workspace
        self.chat = Conversation(generator, system=system, options=options, max_tool_rounds=max_tool_rounds)
        for name, (description, parameters, fn) in workspace.tool_table().items():
            self.chat.add_tool(name, description, parameters, self._guarded(fn))

    @staticmethod
    def _guarded(fn):
        def call(**arguments):
            try:
                return fn(**arguments)
            except SandboxRefusal as e:
                return f"refused: {e}"
            except TypeError as e:                    # wrong or missing argument names
                return f"refused: {e}"
        return call

    def solve(self, task: str) -> AgentReport:
        before = len(self.chat.rounds)
        result = self.chat.say(task)
        rounds = self.chat.rounds[before:]
        return AgentReport(answer=result.text, rounds=rounds, files_changed=list(self.workspace.changed),
                           commands=list(self.workspace.commands),
                           refusals=sum(1 for r in rounds if r.result.startswith("refused:")))
