"""A coding agent in a sandboxed workspace: the model lists, reads, searches and edits files and runs allow-listed
commands as tool rounds until the task is done. With ``--model <folder>`` a chat model in the Hugging Face layout
drives it; without one a scripted stand-in plays the same tool calls a model would make, so the sandbox, the tool
rounds and the report can be seen end to end offline.

    python samples/coding_agent.py [--model <folder>] [--task "..."]

Reference: samples/Idrak.Samples.CodingAgent/Program.cs.
"""
import argparse
import os
import sys
import tempfile
from types import SimpleNamespace

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.text.agents import CodingAgent, Workspace  # noqa: E402

BUGGY = '''def mean(values):
    """Arithmetic mean of a non-empty list."""
    return sum(values) / (len(values) - 1)
'''
TEST = '''from stats import mean

assert mean([2, 4, 6]) == 4, mean([2, 4, 6])
assert mean([5]) == 5
print("all tests pass")
'''


def make_workspace(folder: str) -> Workspace:
    with open(os.path.join(folder, "stats.py"), "w") as f:
        f.write(BUGGY)
    with open(os.path.join(folder, "check_stats.py"), "w") as f:
        f.write(TEST)
    return Workspace(folder, allowed_commands=("python", "python3"))


class ScriptedModel:
    """Plays a fixed sequence of tool calls, then answers: what a model that solves the task would emit."""

    def __init__(self, script):
        self.script, self.turn = list(script), 0

    def chat(self, messages, options=None, tools=None):
        step = self.script[min(self.turn, len(self.script) - 1)]
        self.turn += 1
        if isinstance(step, str):
            return SimpleNamespace(text=step, tool_calls=[], finish_reason="stop")
        name, arguments = step
        return SimpleNamespace(text="", tool_calls=[SimpleNamespace(name=name, arguments=arguments, id=None)],
                               finish_reason="tool_calls")


SCRIPT = [
    ("list_files", {}),
    ("run", {"command": "python check_stats.py"}),
    ("read_file", {"path": "stats.py"}),
    ("read_file", {"path": "../outside.txt"}),                         # refused: leaves the workspace
    ("edit_file", {"path": "stats.py", "old": "(len(values) - 1)", "new": "len(values)"}),
    ("run", {"command": "rm -rf ."}),                                   # refused: not an allowed program
    ("run", {"command": "python check_stats.py"}),
    "The mean divided by one less than the number of values; I fixed the divisor and the checks pass.",
]


def main(model_folder=None, task=None, quiet=False) -> dict:
    task = task or "check_stats.py fails. Find the bug in stats.py, fix it, and run the checks again."
    with tempfile.TemporaryDirectory() as folder:
        workspace = make_workspace(folder)
        if model_folder:
            from idrak_b200.generation.text_generator import TextGenerator
            from idrak_b200.models.pretrained import load_pretrained
            model, tokenizer = load_pretrained(model_folder)
            generator = TextGenerator(model, tokenizer).start()
        else:
            generator = ScriptedModel(SCRIPT)
        report = CodingAgent(generator, workspace).solve(task)
        fixed = open(os.path.join(folder, "stats.py")).read()
    if not quiet:
        for r in report.rounds:
            print(f"-> {r.name}({r.arguments})\n   {r.result.splitlines()[0][:110] if r.result else ''}")
        print("answer:", report.answer)
        print(f"files changed: {report.files_changed}; commands: {report.commands}; refusals: {report.refusals}")
    return {"report": report, "fixed_source": fixed}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model")
    ap.add_argument("--task")
    a = ap.parse_args()
    main(a.model, a.task)
