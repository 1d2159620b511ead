from dataclasses import dataclass, field
from typing import List

from idrak_b200.text.conversation import Conversation


@dataclass
class Call:
    name: str
    arguments: object


@dataclass
class Result:
    text: str = ""
    tool_calls: List[Call] = field(default_factory=list)
    finish_reason: str = "stop"


class Scripted:
    """A stand-in generator: answers from a script and records what it was shown."""

    def __init__(self, script):
        self.script, self.seen = list(script), []

    def chat(self, messages, options, tools):
        self.seen.append(([dict(m) for m in messages], tools))
        return self.script.pop(0)


def test_tool_rounds_run_on_the_server_and_history_is_kept():
    gen = Scripted([Result(tool_calls=[Call("add", '{"a": 2, "b": 3}')], finish_reason="tool_calls"),
                    Result(tool_calls=[Call("add", {"a": 5, "b": 10}), Call("nope", "{}")]),
                    Result("The answers are 5 and 15."),
                    Result("You are welcome.")])
    chat = Conversation(gen, system="Be terse.")
    chat.add_tool("add", "Add two numbers.", {"type": "object", "properties": {"a": {"type": "number"}, "b": {"type": "number"}}},
                  lambda a, b: a + b)
    reply = chat.say("add things")
    assert reply.text == "The answers are 5 and 15."
    roles = [m["role"] for m in chat.messages]
    assert roles == ["system", "user", "assistant", "tool", "assistant", "tool", "tool", "assistant"]
    assert chat.messages[3]["content"] == "5" and chat.messages[5]["content"] == "15"
    assert chat.messages[6]["content"].startswith("error: there is no tool 'nope'; tools: add")
    assert chat.messages[3]["tool_call_id"] == chat.messages[2]["tool_calls"][0]["id"]
    assert [r.failed for r in chat.rounds] == [False, False, True]
    # the model was shown the tool schemas and, on the second round, the first tool result
    assert gen.seen[0][1][0]["function"]["name"] == "add" and gen.seen[1][0][-1]["role"] == "tool"
    chat.say("thanks")
    assert chat.messages[-1] == {"role": "assistant", "content": "You are welcome."} and len(gen.seen) == 4
    assert "assistant -> add(" in chat.transcript() and "tool: 5" in chat.transcript()
    chat.reset()
    assert chat.messages == [{"role": "system", "content": "Be terse."}] and chat.rounds == []


def test_round_limit_bad_arguments_and_failing_tools():
    loop = [Result(tool_calls=[Call("boom", "{}")]) for _ in range(3)] + [Result("gave up", [Call("boom", "{}")])]
    gen = Scripted(loop)
    chat = Conversation(gen, max_tool_rounds=3)
    chat.add_tool("boom", "Always fails.", {"type": "object"}, lambda: 1 / 0)
    reply = chat.say("go")
    assert reply.text == "gave up" and len(chat.rounds) == 3 and all(r.failed for r in chat.rounds)
    assert "ZeroDivisionError" in chat.rounds[0].result
    gen2 = Scripted([Result(tool_calls=[Call("boom", "{not json")]), Result("ok")])
    chat2 = Conversation(gen2)
    chat2.add_tool("boom", "x", {"type": "object"}, lambda: 1)
    assert chat2.say("go").text == "ok" and "not JSON" in chat2.rounds[0].result
    # without registered tools a tool call is simply the answer
    gen3 = Scripted([Result("text", [Call("add", "{}")])])
    assert Conversation(gen3).say("hi").text == "text" and gen3.seen[0][1] is None
