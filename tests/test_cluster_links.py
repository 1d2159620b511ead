"""Link calibration, all-reduce prediction, token bucket / throttled transport, capped fake devices, topology builder."""
import json

import pytest
import torch

from idrak_b200.cluster.links import (BUILT_IN_LINKS, ClusterCache, DeviceMemoryExceeded, LinkCalibration, ThrottledTransport,
                                      TokenBucket, TopologyBuilder, carve, fastest, predict_all_reduce)
from idrak_b200.cluster.sim import InProcessCluster
from idrak_b200.cluster.topology import parse_topology
from idrak_b200.parallel.host_collectives import SimRankTransport, create


def test_calibration_recovers_latency_and_bandwidth(tmp_path):
    samples = [(n, 20e-6 + n / 12e9) for n in (1 << 10, 1 << 16, 1 << 20, 1 << 24)]
    cal = LinkCalibration.fit(samples)
    assert cal.link.latency == pytest.approx(20e-6, rel=1e-3) and cal.link.bandwidth == pytest.approx(12e9, rel=1e-6)
    assert cal.r2 > 0.999999 and cal.samples == 4
    with pytest.raises(ValueError, match="two or more"):
        LinkCalibration.fit([(1024, 1e-5), (1024, 1.1e-5)])
    cache = ClusterCache(str(tmp_path / "c" / "cluster.json"))
    assert cache.load() == {}
    cache.store("tcp", cal)
    assert cache.load()["tcp"].bandwidth == pytest.approx(12e9, rel=1e-6)


def test_prediction_follows_the_algorithms():
    b = TopologyBuilder()
    one = parse_topology(json.dumps(b.build({"nodes": 1, "gpus": 8})))
    two = parse_topology(json.dumps(b.build({"nodes": 2, "gpus": 8, "inter_node": "tcp"})))
    n = 64 << 20
    nv, tcp = BUILT_IN_LINKS["nvlink"], BUILT_IN_LINKS["tcp"]
    assert predict_all_reduce(one, n, "ring") == pytest.approx(14 * nv.transfer_time(n / 8))
    assert predict_all_reduce(one, n, "naive") > predict_all_reduce(one, n, "ring")
    ring, hier = predict_all_reduce(two, n, "ring"), predict_all_reduce(two, n, "hierarchical")
    assert ring == pytest.approx(30 * tcp.transfer_time(n / 16))
    assert hier == pytest.approx(14 * nv.transfer_time(n / 8) + 2 * tcp.transfer_time(n / 16))
    assert hier < ring / 5                                     # only 1/8 of the values cross the slow link per column
    faster = predict_all_reduce(two, n, "hierarchical", {"tcp": LinkCalibration.fit([(0, 1e-5), (1e9, 1e-5 + 1 / 40.0)]).link})
    assert faster < hier
    assert fastest(["tcp", "nvlink", "shared-memory"]) == "nvlink"
    with pytest.raises(KeyError, match="not registered"):
        predict_all_reduce(one, n, "tree")


def test_token_bucket_and_throttled_transport():
    now = [0.0]
    bucket = TokenBucket(rate=1000.0, burst=500.0, clock=lambda: now[0])
    assert bucket.take(400) == 0.0
    assert bucket.take(300) == pytest.approx(0.2)              # 200 bytes of debt at 1000 B/s
    now[0] += 1.0
    assert bucket.take(100) == 0.0                             # refilled up to the burst

    slept = []

    def fn(ctx):
        t = ThrottledTransport(SimRankTransport(ctx), TokenBucket(1e6, 1024.0, clock=lambda: 0.0), latency=1e-3,
                               sleep=slept.append if ctx.rank == 0 else (lambda s: None))
        out = create("ring", t).all_reduce(torch.full((1024,), float(ctx.rank + 1)))
        return out, t.waited
    res = InProcessCluster(2).run(lambda ctx, step: fn(ctx), steps=1)
    assert not res.errors
    assert torch.equal(res.returns[0][0], torch.full((1024,), 3.0))
    assert res.returns[0][1] == pytest.approx(sum(slept)) and res.returns[0][1] > 2e-3


def test_carved_devices_enforce_their_caps():
    devs = carve(16 << 30, 4)
    assert len(devs) == 4 and devs[0].capacity == int((16 << 30) * 0.95) // 4
    devs[0].allocate(3 << 30)
    with pytest.raises(DeviceMemoryExceeded, match="sim:0"):
        devs[0].allocate(1 << 30)
    devs[0].release(2 << 30)
    devs[0].allocate(1 << 30)
    assert devs[0].peak == 3 << 30 and devs[1].used == 0


def test_topology_builder_questions_are_data():
    b = TopologyBuilder()
    assert [q["key"] for q in b.questions()] == ["nodes", "gpus", "memory"]
    assert [q["key"] for q in b.questions({"nodes": 3})] == ["nodes", "gpus", "memory", "addresses", "inter_node"]
    doc = b.build({"nodes": 2, "gpus": 2, "addresses": "10.1.0.1, 10.1.0.2", "inter_node": "rdma"})
    topo = parse_topology(json.dumps(doc))
    assert topo.world == 4 and topo.link_type("node0", "node1") == "rdma" and topo.nodes[1].address == "10.1.0.2"
    with pytest.raises(ValueError, match="addresses"):
        b.build({"nodes": 2, "addresses": "10.0.0.1"})
