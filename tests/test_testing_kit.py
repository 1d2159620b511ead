"""The shipped testing kit: conformance record / replay, contract suites with broken twins, stress, regression files,
and the transports that share one contract."""
import threading
import uuid

import pytest
import torch

from idrak_b200 import testing
from idrak_b200.testing import conformance, contracts


def test_recorder_keeps_outermost_calls_with_their_arguments():
    calls = testing.record_scenarios(["feed_forward"])
    names = {c.op for c in calls}
    assert {"mlp_gelu", "mlp_gated", "gated_activation", "gelu"} <= names
    assert "gemm" not in names and "linear" not in names          # inner calls of a recorded operation are not kept
    c = next(c for c in calls if c.op == "mlp_gelu")
    assert len(c.args) == 6 and torch.is_tensor(c.result) and c.differentiable and c.scenario == "feed_forward"
    from idrak_b200 import ops
    assert not hasattr(ops.gelu, "__wrapped__")                    # the recorder put the functions back


def test_conformance_replay_on_the_host_passes_and_a_wrong_kernel_is_caught():
    rep = testing.check("cpu", scenarios=["rows", "losses", "attention"])
    assert rep.ok and rep.counts().get("ok", 0) > 30, rep.to_json()

    def wrong_gelu(x):                    # exact erf form instead of the tanh form: off by up to ~5e-4... use relu to be plain
        return torch.relu(x)
    bad = testing.check("cpu", scenarios=["feed_forward"], implementations={"gelu": wrong_gelu})
    assert not bad.ok and {o.op for o in bad.outcomes if o.status == "failed"} == {"gelu"}

    def refuses(*a, **k):
        raise NotImplementedError("no kernel for this on the device")
    skipped = testing.check("cpu", scenarios=["feed_forward"], implementations={"gelu": refuses})
    assert skipped.ok and "gelu" in skipped.to_json() and skipped.counts()["skipped"] >= 1


def test_gradients_are_compared_too():
    calls = [c for c in testing.record_scenarios(["rows"]) if c.op == "rms_norm"]

    class Detached(torch.autograd.Function):      # right values, wrong gradient
        @staticmethod
        def forward(ctx, x, w, eps):
            from idrak_b200 import ops
            return ops.rms_norm(x.detach(), w.detach(), eps)

        @staticmethod
        def backward(ctx, g):
            return g, None, None
    out = testing.replay(calls[0], "cpu", implementation=lambda x, w, eps: Detached.apply(x, w, eps))
    assert out.status == "failed" and "gradient" in out.detail


@pytest.mark.parametrize("name", sorted(contracts.SUITES))
def test_every_suite_accepts_its_reference_and_rejects_its_broken_twin(name):
    assert contracts.SUITES[name]().self_test() == []


def test_library_pieces_conform():
    from idrak_b200.ops.decode import sample_rows_reference
    assert contracts.SamplerContract().run(
        lambda l, t, k, p, m, u: sample_rows_reference(l, l.shape[1], t, k, p, m, u)) == []
    from idrak_b200.parallel.host_collectives import create
    from idrak_b200.parallel.transport import MemoryTransport
    for kind in ("naive", "ring"):
        def all_reduce(parts, kind=kind):
            return MemoryTransport.hub(len(parts)).run(lambda r, t: create(kind, t.as_exchange()).all_reduce(parts[r]))
        assert contracts.CollectiveContract().run({"all_reduce": all_reduce}, random_cases=4) == []


def test_tcp_and_shared_memory_transports_meet_the_transport_contract():
    from idrak_b200.parallel.transport import FramedTcpTransport, Rendezvous, SharedMemoryTransport
    ports = iter(range(29910, 29990))

    def tcp(world):
        port = next(ports)
        return lambda r: FramedTcpTransport(r, world, Rendezvous("127.0.0.1", port, world, b"shared secret", 20.0),
                                            credits=2, timeout=20.0)

    def shm(world):
        session = "idrk" + uuid.uuid4().hex[:10]
        return lambda r: SharedMemoryTransport(r, world, session, capacity=1 << 12, timeout=20.0)
    suite = contracts.TransportContract()
    assert suite.run(tcp, random_cases=2) == []
    assert suite.run(shm, random_cases=2) == []


def test_rendezvous_turns_away_a_wrong_secret():
    from idrak_b200.parallel.transport import Rendezvous
    good = Rendezvous("127.0.0.1", 29995, 1, b"right", 5.0)
    good.serve()
    with pytest.raises(PermissionError):
        Rendezvous("127.0.0.1", 29995, 1, b"wrong", 5.0).join(0, "127.0.0.1:1")
    assert good.join(0, "127.0.0.1:7") == {0: "127.0.0.1:7"}      # the stranger did not take the seat


def test_stress_notices_memory_that_grows_and_accepts_memory_that_does_not():
    kept = []
    leaky = testing.run_stress(lambda i: kept.append(torch.zeros(1000)), steps=10, warmup=2, device="cpu")
    assert not leaky.ok and leaky.growth >= 9 * 4000 and "grew" in leaky.errors[0]
    steady = testing.run_stress(lambda i: torch.zeros(1000 + i).sum(), steps=10, warmup=2, device="cpu")
    assert steady.ok and steady.growth == 0
    broken = testing.run_stress(lambda i: (_ for _ in ()).throw(ValueError("odd shape")) if i == 4 else None,
                                steps=10, warmup=2, device="cpu")
    assert not broken.ok and "step 4" in broken.errors[0]
    stop = threading.Event()
    stop.set()
    assert testing.run_stress(lambda i: None, steps=5, device="cpu", should_stop=stop.is_set).stopped_early


def test_default_workload_holds_memory_level_on_the_host():
    from idrak_b200.testing.stress import default_workload
    rep = testing.run_stress(default_workload("cpu"), steps=8, warmup=8, device="cpu", allowed_growth=1 << 16)
    assert rep.ok, rep.errors


def test_regression_cases_round_trip(tmp_path):
    call = next(c for c in testing.record_scenarios(["rows"]) if c.op == "layer_norm")
    p = testing.save_case(call, tmp_path, note="kept after a wrong variance on 129 rows")
    assert p.name == "layer_norm-000.pt"
    out = testing.replay_folder(tmp_path, "cpu")
    assert len(out) == 1 and out[0].status == "ok" and out[0].op == "layer_norm"
    (tmp_path / "junk.pt").write_bytes(b"nothing")
    with pytest.raises(Exception):
        testing.replay_folder(tmp_path, "cpu")


@pytest.mark.gpu
def test_conformance_on_the_gpu():
    rep = testing.check("cuda")
    assert rep.ok, rep.to_json()
    assert rep.counts().get("ok", 0) > 80


@pytest.mark.gpu
def test_stress_on_the_gpu_keeps_device_memory_level():
    from idrak_b200.testing.stress import default_workload
    rep = testing.run_stress(default_workload("cuda"), steps=28, warmup=14, device="cuda")
    assert rep.ok, rep.errors
    # two threads, each with its own stream: the caching allocator keeps one pool per stream, so the level may rise by
    # what the second stream's pool holds - bounded, and it must not keep rising with more steps
    two = testing.run_stress(default_workload("cuda", seed=1), steps=16, warmup=14, device="cuda", threads=2,
                             allowed_growth=8 << 20)
    more = testing.run_stress(default_workload("cuda", seed=1), steps=48, warmup=14, device="cuda", threads=2,
                              allowed_growth=8 << 20)
    assert two.ok and more.ok, (two.errors, more.errors)
