"""Host collectives (naive / ring / hierarchical) on the in-process cluster and on gloo ranks: the sums agree with a
plain sum, every rank ends with identical bits, traffic follows the algorithm, uneven pieces and all-to-all work."""
import os
import subprocess
import sys

import pytest
import torch

from idrak_b200.cluster.sim import InProcessCluster
from idrak_b200.parallel.host_collectives import COLLECTIVES, SimRankTransport, create, even_counts

HERE = os.path.dirname(os.path.abspath(__file__))


def _values(rank, n):
    return torch.randn(n, generator=torch.Generator().manual_seed(100 + rank))


def _run(world, fn):
    res = InProcessCluster(world).run(lambda ctx, step: fn(ctx), steps=1)
    assert not res.errors, res.errors
    return [res.returns[r] for r in range(world)]


@pytest.mark.parametrize("name,world,nodes", [("naive", 4, None), ("ring", 1, None), ("ring", 3, None), ("ring", 5, None),
                                              ("hierarchical", 4, [[0, 1], [2, 3]]), ("hierarchical", 5, [[0, 1, 2], [3, 4]]),
                                              ("hierarchical", 6, [[0], [1, 2, 3], [4, 5]])])
def test_all_reduce_matches_the_sum_with_identical_bits(name, world, nodes):
    n = 1003

    def fn(ctx):
        kw = {"nodes": nodes} if nodes else {}
        return create(name, SimRankTransport(ctx), chunk=256, **kw).all_reduce(_values(ctx.rank, n))
    out = _run(world, fn)
    want = torch.stack([_values(r, n) for r in range(world)]).double().sum(0).float()
    for o in out:
        assert torch.equal(o, out[0])
        assert torch.allclose(o, want, atol=1e-5)


def test_ring_traffic_is_two_w_minus_one_over_w():
    world, n = 4, 4096

    def fn(ctx):
        ring, naive = create("ring", SimRankTransport(ctx)), create("naive", SimRankTransport(ctx))
        ring.all_reduce(_values(ctx.rank, n))
        naive.all_reduce(_values(ctx.rank, n))
        return ring.bytes_sent, naive.bytes_sent
    out = _run(world, fn)
    for ring_bytes, _ in out:
        assert ring_bytes == 2 * (world - 1) * (n // world) * 4
    assert out[0][1] == (world - 1) * n * 4 and out[1][1] == n * 4          # the first rank sends everything back


def test_bfloat16_wire_halves_the_bytes_and_keeps_ranks_identical():
    def fn(ctx):
        c = create("hierarchical", SimRankTransport(ctx), nodes=[[0, 1, 2], [3, 4]], wire="bfloat16")
        return c.all_reduce(_values(ctx.rank, 512)), c.bytes_sent
    out = _run(5, fn)
    want = torch.stack([_values(r, 512) for r in range(5)]).sum(0)
    for o, _ in out:
        assert torch.equal(o, out[0][0])
        assert torch.allclose(o, want, atol=0.08, rtol=0.02)
        assert torch.equal(o, o.bfloat16().float())                                # what travelled was bfloat16


def test_uneven_reduce_scatter_all_gather_broadcast_and_all_to_all():
    world, counts = 3, [5, 0, 12]

    def fn(ctx):
        c = create("ring", SimRankTransport(ctx))
        mine = c.reduce_scatter(_values(ctx.rank, 17), counts)
        whole = c.all_gather(mine, counts)
        b = c.broadcast(_values(ctx.rank, 7), root=1)
        got = c.all_to_all([torch.full((ctx.rank + j + 1,), float(10 * ctx.rank + j)) for j in range(world)])
        c.barrier()
        return mine, whole, b, got
    out = _run(world, fn)
    want = torch.stack([_values(r, 17) for r in range(world)]).sum(0)
    offs = [0, 5, 5, 17]
    for r, (mine, whole, b, got) in enumerate(out):
        assert mine.numel() == counts[r] and torch.allclose(mine, want[offs[r]:offs[r + 1]], atol=1e-5)
        assert torch.allclose(whole, want, atol=1e-5) and torch.equal(whole, out[0][1])
        assert torch.equal(b, _values(1, 7))
        for src in range(world):
            assert torch.equal(got[src], torch.full((src + r + 1,), float(10 * src + r)))


def test_registry_and_argument_checks():
    assert sorted(COLLECTIVES) == ["hierarchical", "naive", "ring"]
    assert even_counts(10, 4) == [3, 3, 2, 2]

    def fn(ctx):
        with pytest.raises(KeyError, match="not registered"):
            create("tree", SimRankTransport(ctx))
        with pytest.raises(ValueError, match="every rank exactly once"):
            create("hierarchical", SimRankTransport(ctx), nodes=[[0], [0, 1]])
        return True
    assert _run(2, fn) == [True, True]


def test_on_gloo_ranks(tmp_path):
    out = tmp_path / "out.pt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29833", os.path.join(HERE, "host_collectives_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    got = torch.load(out)
    want = torch.stack([_values(r, 5000) for r in range(3)]).sum(0)
    for name in ("naive", "ring", "hierarchical"):
        assert torch.allclose(got[name], want, atol=1e-5), name
    assert got["identical"]
