"""The coding agent's sandbox (path confinement, allow-listed commands, exact edits) and its tool rounds."""
import importlib.util
import os

import pytest

from idrak_b200.text.agents import SandboxRefusal, Workspace


def _ws(tmp_path, **kw):
    (tmp_path / "pkg").mkdir()
    (tmp_path / "pkg" / "a.py").write_text("x = 1\ny = 2\nx = 1\n")
    (tmp_path / "notes.txt").write_text("alpha\nbeta\n")
    return Workspace(tmp_path, **kw)


def test_paths_stay_inside_the_workspace(tmp_path):
    ws = _ws(tmp_path)
    outside = tmp_path.parent / "secret.txt"
    outside.write_text("no")
    for bad in ("../secret.txt", str(outside), "pkg/../../secret.txt", ""):
        with pytest.raises(SandboxRefusal):
            ws.read_file(bad)
    os.symlink(outside, tmp_path / "link.txt")
    with pytest.raises(SandboxRefusal, match="leaves the workspace"):
        ws.read_file("link.txt")
    with pytest.raises(SandboxRefusal):
        ws.write_file("../escape.txt", "x")
    assert "pkg/a.py" in ws.list_files("*.py") and "notes.txt" not in ws.list_files("*.py")
    assert ws.read_file("notes.txt", 2, 2).split() == ["2", "beta"]
    assert "pkg/a.py:2:" in ws.search("y = ")
    assert ws.search("^x", regex=True).count("pkg/a.py") == 2
    with pytest.raises(SandboxRefusal, match="regular expression"):
        ws.search("(", regex=True)


def test_edits_must_be_exact_and_commands_allow_listed(tmp_path):
    ws = _ws(tmp_path, allowed_commands=("python",))
    with pytest.raises(SandboxRefusal, match="occurs 2 times"):
        ws.edit_file("pkg/a.py", "x = 1", "x = 3")
    with pytest.raises(SandboxRefusal, match="occurs 0 times"):
        ws.edit_file("pkg/a.py", "z = 9", "z = 1")
    assert ws.edit_file("pkg/a.py", "y = 2", "y = 5") == "edited pkg/a.py"
    assert (tmp_path / "pkg" / "a.py").read_text().splitlines()[1] == "y = 5"
    ws.write_file("new/b.txt", "hello")
    assert ws.changed == ["pkg/a.py", "new/b.txt"]
    out = ws.run("python -c \"print(6 * 7)\"")
    assert out.startswith("exit code 0") and "42" in out
    for bad in ("rm -rf .", "/usr/bin/python -V", "python ../x.py", "python /etc/passwd", "bash -c ls"):
        with pytest.raises(SandboxRefusal):
            ws.run(bad)
    slow = Workspace(tmp_path, allowed_commands=("python",), command_timeout=0.5)
    assert "did not finish" in slow.run("python -c \"import time; time.sleep(5)\"")
    ro = Workspace(tmp_path, read_only=True)
    with pytest.raises(SandboxRefusal, match="read-only"):
        ro.write_file("c.txt", "x")
    assert "write_file" not in ro.tool_table() and "read_file" in ro.tool_table()


def test_agent_fixes_the_bug_through_tool_rounds():
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "samples", "coding_agent.py")
    spec = importlib.util.spec_from_file_location("sample_coding_agent", root)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = mod.main(quiet=True)
    report = out["report"]
    assert "/ len(values)" in out["fixed_source"]
    assert report.files_changed == ["stats.py"] and report.refusals == 2
    assert report.commands == ["python check_stats.py", "python check_stats.py"]       # the refused command never ran
    results = [r.result for r in report.rounds if r.name == "run"]
    assert "exit code 1" in results[0] and "all tests pass" in results[-1]
    assert report.answer.startswith("The mean divided")
