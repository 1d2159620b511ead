"""Replacing one operation's kernel from outside the library: a plug-in registers its own `gelu` for the CPU device,
the dispatcher runs it instead of the built-in one, the conformance replay judges it, and removing the registration
brings the built-in kernel back.

    python samples/override.py

Reference: samples/Idrak.Samples.Override/Program.cs (a user kernel shadowing a library kernel).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200 import core, testing  # noqa: E402


def sigmoid_gelu(x: torch.Tensor) -> torch.Tensor:
    """The cheap x * sigmoid(1.702 x) form: close to GELU, not equal to it."""
    return x * torch.sigmoid(1.702 * x)


def main(quiet: bool = False) -> dict:
    x = torch.linspace(-3, 3, 13)
    built_in = core.run("gelu", x)
    with core.register_kernel("gelu", "cpu", sigmoid_gelu):
        replaced = core.run("gelu", x)
        source = [r["source"] for r in core.operation_report(core.backend_for("cpu")) if r["operation"] == "gelu"][0]
        # would the replacement pass for the library's own kernel? the conformance replay of the recorded gelu calls says
        calls = [c for c in testing.record_scenarios(["feed_forward"]) if c.op == "gelu"]
        verdicts = [testing.replay(c, "cpu", implementation=sigmoid_gelu).status for c in calls]
        wrong = [testing.replay(c, "cpu", implementation=torch.relu).status for c in calls]      # not a GELU at all
    after = core.run("gelu", x)
    out = {"largest_difference": float((replaced - built_in).abs().max()), "source_while_registered": source,
           "conformance": verdicts, "conformance_of_relu": wrong, "restored": bool(torch.equal(after, built_in))}
    if not quiet:
        print(out)
    return out


if __name__ == "__main__":
    main()
