"""Failing calls kept as files and replayed later.

``save_case`` writes one recorded call (operation, arguments, host result) with ``torch.save``; ``replay_folder`` runs
every saved call on a device through the conformance replay and reports what still fails.

Reference: Regression.Replay (src/Idrak.Abstraction.Testing/Regression.cs:27) over tests/Idrak.Tests/data/regressions.
"""
from __future__ import annotations

from pathlib import Path
from typing import List

import torch

from .conformance import CallOutcome, RecordedCall, replay

FORMAT = "idrak-regression/1"


def save_case(call: RecordedCall, folder, note: str = "") -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    n = len(list(folder.glob(f"{call.op}-*.pt")))
    path = folder / f"{call.op}-{n:03d}.pt"
    torch.save({"format": FORMAT, "op": call.op, "args": call.args, "kwargs": call.kwargs, "result": call.result,
                "differentiable": call.differentiable, "scenario": call.scenario, "note": note}, path)
    return path


def load_case(path) -> RecordedCall:
    d = torch.load(path, weights_only=False)
    if d.get("format") != FORMAT:
        raise ValueError(f"{path}: not a saved regression case (format {d.get('format')!r})")
    return RecordedCall(d["op"], d["args"], d["kwargs"], d["result"], d["differentiable"], d.get("scenario", ""))


def replay_folder(folder, device="cuda") -> List[CallOutcome]:
    return [replay(load_case(p), device) for p in sorted(Path(folder).glob("*.pt"))]
