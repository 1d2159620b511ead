"""Cluster simulator (virtual time, failure models, replay), step header / stop agreement / control file, topology
files and the settings advisor. All on the host."""
import json

import numpy as np
import pytest

from idrak_b200.cluster import (ClusterReplay, ClusterRunStopped, ControlFileSteering, EventLog, Fault, FaultInjector,
                                HeaderMismatch, InProcessCluster, LinkModel, RankDropped, RankTimeout, StepHeader,
                                StopAgreement, advise, parse_topology)


def _sum_step(ctx, step):
    ctx.compute(0.010)
    return float(ctx.all_reduce([float(ctx.rank + step)])[0])


def test_collectives_virtual_time_and_bytes():
    link = LinkModel(latency=1e-3, bandwidth=1e6)
    res = InProcessCluster(4, link).run(_sum_step, steps=3)
    assert not res.errors and set(res.returns.values()) == {0 + 1 + 2 + 3 + 4 * 2}
    # three steps of 10 ms compute + gather and broadcast hops of ~1 ms each; far below any wall-clock timeout
    assert 0.03 < res.virtual_seconds < 0.06 and res.bytes_sent == 3 * 6 * 8
    a = InProcessCluster(4, LinkModel(jitter=0.5), seed=7).run(_sum_step, steps=3).virtual_seconds
    b = InProcessCluster(4, LinkModel(jitter=0.5), seed=7).run(_sum_step, steps=3).virtual_seconds
    assert a == b                                                    # seeded: runs repeat


def test_slow_worker_is_logged_and_replayed(tmp_path):
    inj = FaultInjector(seed=3, model="slow-worker", rate=0.9, slow_seconds=2.0)
    run = InProcessCluster(3, failures=inj).run(_sum_step, steps=4)
    faults = run.log.of("fault")
    assert faults and all(f["fault"] == "slow" and f["key"].startswith("slow@step") for f in faults)
    assert not run.errors and run.virtual_seconds > 2.0
    path = tmp_path / "run.ikev"
    run.log.save(str(path))
    again = InProcessCluster(3, failures=ClusterReplay(EventLog.load(str(path)))).run(_sum_step, steps=4)
    assert again.virtual_seconds == run.virtual_seconds and again.log.of("fault") == faults
    with pytest.raises(KeyError, match="not registered"):
        FaultInjector(model="meteor")


def test_dropped_worker_times_out_by_name_and_late_joiner_sits_out():
    drop = FaultInjector(model="scripted", scripted=[Fault(step=1, rank=2, kind="drop")])
    run = InProcessCluster(3, failures=drop, timeout=120.0).run(_sum_step, steps=3)
    assert isinstance(run.errors[2], RankDropped)
    e = run.errors[0]
    assert isinstance(e, RankTimeout) and e.on == 2 and "rank 2 within 120 s" in str(e)
    assert run.virtual_seconds >= 120.0                              # the timeout passed on the virtual clock only
    late = FaultInjector(model="scripted", scripted=[Fault(step=1, rank=1, kind="late", amount=2)])
    run = InProcessCluster(3, failures=late).run(lambda ctx, s: float(ctx.all_reduce([1.0])[0]), steps=4)
    assert not run.errors and [e["step"] for e in run.log.of("sat-out")] == [1, 2]
    assert run.returns == {0: 3.0, 1: 3.0, 2: 3.0}                   # everyone is back for the last step
    cut = FaultInjector(model="scripted", scripted=[Fault(step=0, rank=1, kind="partition", peer=0)])
    run = InProcessCluster(2, failures=cut, timeout=30.0).run(_sum_step, steps=1)
    assert isinstance(run.errors[0], RankTimeout) and run.errors[0].on == 1


def test_header_and_stop_agreement_over_the_simulator(tmp_path):
    stop_file = tmp_path / "stop"

    def rank_main(ctx, step):
        h = StepHeader(model_hash=77, ctx=ctx)
        agree = StopAgreement(h, stop_file=str(stop_file) if ctx.rank == 2 else None)
        if step == 2 and ctx.rank == 2:
            stop_file.write_text("now")
        red = agree.at_boundary(step, tokens=100.0 * (ctx.rank + 1), loss=float(ctx.rank))
        return (red.tokens, round(red.mean_loss, 6), red.ranks)

    run = InProcessCluster(3).run(rank_main, steps=4)
    assert all(isinstance(e, ClusterRunStopped) and "step 2" in str(e) for e in run.errors.values()) and len(run.errors) == 3
    stop_file.unlink()
    ok = InProcessCluster(3).run(rank_main, steps=2)
    assert ok.returns[0] == ok.returns[2] == (600.0, round((0 * 100 + 1 * 200 + 2 * 300) / 600, 6), 3)

    def mismatch(ctx, step):
        return StepHeader(model_hash=1 + (ctx.rank == 1), ctx=ctx).exchange(step, 1.0, 0.0)
    bad = InProcessCluster(2).run(mismatch, steps=1)
    assert all(isinstance(e, HeaderMismatch) and "different parameter shapes" in str(e) for e in bad.errors.values())


def test_control_file_pause_resume_stop(tmp_path):
    path = tmp_path / "control.json"
    naps = []

    def sleeper(seconds):
        naps.append(seconds)
        if len(naps) == 3:
            path.write_text(json.dumps({"command": "resume"}))
    s = ControlFileSteering(str(path), rank=0, sleep=sleeper)
    s.at_boundary(0)                                                 # no file: run on
    path.write_text(json.dumps({"command": "pause"}))
    s.at_boundary(1)
    assert len(naps) == 3 and s.pauses == 3
    path.write_text(json.dumps({"command": "stop"}))
    with pytest.raises(ClusterRunStopped, match="stop command"):
        s.at_boundary(2)
    path.write_text(json.dumps({"command": "explode"}))
    with pytest.raises(ValueError, match="unknown command 'explode'"):
        s.at_boundary(3)


TOPOLOGY = """
{ // two nodes
  "format": "idrak-topology/1",
  "nodes": [
    { "name": "a", "address": "10.0.0.1", "gpus": [ { "device": 0, "memory": "180GiB" }, { "device": 1, "memory": "180GiB" }, ] },
    { "name": "b", "address": "10.0.0.2", "gpus": [ { "device": 0, "memory": "96 GiB" } ] },
  ],
  "links": { "intra-node": "nvlink", "inter-node": "tcp", /* one fast pair */
             "overrides": [ { "between": ["a", "b"], "type": "rdma", "address": "10.1.0.1" } ] },
  "simulation": { "seed": 4, "failures": "slow-worker" },
}
"""


def test_topology_file_and_advisor():
    t = parse_topology(TOPOLOGY)
    assert t.world == 3 and t.nodes[0].gpus[1].memory == 180 << 30 and t.link_type("a", "b") == "rdma"
    assert t.link_type("a", "a") == "nvlink" and t.ranks()[2] == {"rank": 2, "node": "b", "address": "10.0.0.2",
                                                                   "device": 0, "memory": 96 << 30}
    with pytest.raises(ValueError, match="unknown key 'colour'"):
        parse_topology(TOPOLOGY.replace('"address": "10.0.0.2"', '"address": "10.0.0.2", "colour": 1'))
    with pytest.raises(ValueError, match="needs a unit|expected a number and a unit"):
        parse_topology(TOPOLOGY.replace('"96 GiB"', '"96000"'))
    with pytest.raises(ValueError, match="format"):
        parse_topology(TOPOLOGY.replace("idrak-topology/1", "idrak-topology/9"))
    quiet = advise(1.0, 0.01, 500 << 20, 400e9)
    assert len(quiet) == 1 and quiet[0].setting == "none"
    loud = advise(1.0, 0.5, 500 << 20, 10e9, world=16, same_switch=False)
    names = [a.setting for a in loud]
    assert "compression" in names and "gradient_sync" in names and "collectives" in names and "accumulation" in names


def test_dashboard_rows_summary_pages_and_local_launch(tmp_path):
    import json
    import time
    import urllib.request
    from idrak_b200.cluster import dashboard
    from idrak_b200.cluster.topology import load_topology
    folder = str(tmp_path / "status")
    w0, w1, w2 = (dashboard.StatusWriter(folder, r, 4, "run") for r in range(3))
    w0.update(step=12, loss=2.5, tokens_per_s=1000.0, memory_bytes=3 << 30,
              network={"bytes_sent": 5 << 20, "bytes_read": 1 << 20})
    w1.update(step=12, loss=2.6, tokens_per_s=900.0)
    w2.update(step=11)
    w2.finish("stopped")
    now = time.time()
    rows = dashboard.read_status(folder, stale_after=5.0, now=now + 1)
    assert [r["rank"] for r in rows] == [0, 1, 2] and [r["state"] for r in rows] == ["running", "running", "stopped"]
    late = dashboard.read_status(folder, stale_after=5.0, now=now + 60)
    assert [r["state"] for r in late] == ["silent", "silent", "stopped"]          # what a rank wrote itself stays
    s = dashboard.summary(rows)
    assert s["running"] == 2 and s["tokens_per_s"] == 1900.0 and (s["step_min"], s["step_max"]) == (11, 12)
    text = dashboard.render_text(rows)
    assert "3.0 GiB" in text and "5.0 MiB" in text and "2 of 4 ranks running" in text and "1 never reported" in text
    assert "silent: [0, 1]" in dashboard.render_text(late)
    page = dashboard.render_html(late)
    assert "<tr class='silent'>" in page and "http-equiv='refresh'" in page
    (tmp_path / "status" / "rank-0009.json").write_text("{half a file")            # mid-replace: skipped, not fatal
    assert len(dashboard.read_status(folder)) == 3
    httpd = dashboard.serve(folder)
    try:
        base = f"http://127.0.0.1:{httpd.server_address[1]}"
        got = json.loads(urllib.request.urlopen(base + "/status.json").read())
        assert got["summary"]["ranks"] == 3 and got["ranks"][0]["loss"] == 2.5
        assert b"<table>" in urllib.request.urlopen(base + "/").read()
    finally:
        httpd.shutdown()
    topo_path = tmp_path / "topo.json"
    topo_path.write_text(json.dumps({"format": "idrak-topology/1", "links": {"intra-node": "nvlink", "inter-node": "tcp"},
                                     "nodes": [{"name": "a", "address": "10.0.0.1", "gpus": [{"device": 0, "memory": "80GiB"}, {"device": 1, "memory": "80GiB"}]},
                                               {"name": "b", "address": "10.0.0.2", "gpus": [{"device": 0, "memory": "80GiB"}]}]}))
    jobs = dashboard.local_rank_commands(load_topology(str(topo_path)), "b", ["python", "train.py"], 29511)
    assert len(jobs) == 1 and jobs[0]["env"] == {"RANK": "2", "LOCAL_RANK": "0", "WORLD_SIZE": "3", "LOCAL_WORLD_SIZE": "1",
                                                  "MASTER_ADDR": "10.0.0.1", "MASTER_PORT": "29511"}
    import pytest as _pytest
    with _pytest.raises(KeyError, match="known: a, b"):
        dashboard.local_rank_commands(load_topology(str(topo_path)), "c", ["x"])
    from idrak_b200.cli.__main__ import main
    assert main(["cluster", "ui", folder, "--once"]) == 0
    assert main(["cluster", "start", str(topo_path), "--node", "a", "--dry-run"]) == 0
