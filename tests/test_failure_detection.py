"""Failure detection without touching a GPU: a rank leaves between steps (with or without saying so) and the others
find out on the host before their next collective; without the heartbeat the process group's short timeout ends the
collective with an error."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = [29760]


def _run(mode, out, nproc=3):
    _PORT[0] += 1
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(_PORT[0]), os.path.join(HERE, "failure_worker.py"), mode, str(out)]
    subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    return [json.loads((out / f"rank{r}.json").read_text()) for r in range(nproc) if (out / f"rank{r}.json").exists()]


def test_rank_that_says_bye_is_named_at_once(tmp_path):
    reports = _run("bye", tmp_path)
    assert len(reports) == 3 and reports[2]["error"] == "left" and reports[2]["steps"] == 2
    for r in reports[:2]:
        assert r["steps"] == 2 and r["error"].startswith("RankLeft: rank 2 left the run: test says so")


def test_silent_rank_is_found_by_its_stale_heartbeat(tmp_path):
    reports = _run("silent", tmp_path)
    assert len(reports) == 3
    for r in reports[:2]:
        assert "no heartbeat from rank 2 within 1 s" in (r["error"] or "") or "RuntimeError" in (r["error"] or ""), r


def test_short_process_group_timeout_ends_the_collective(tmp_path):
    reports = _run("pgtimeout", tmp_path)
    survivors = [r for r in reports if r["rank"] != 2]
    assert survivors and all(r["steps"] == 2 and (r["error"] or "").startswith("RuntimeError") for r in survivors)
