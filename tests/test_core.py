import pytest
import torch

from idrak_b200 import core


def test_gradient_ready_fires_in_backward_order_and_detaches():
    a = torch.nn.Linear(4, 4)
    b = torch.nn.Linear(4, 2)
    seen = []
    with core.on_gradient_ready(list(a.parameters()) + list(b.parameters()), lambda p: seen.append(id(p))):
        b(torch.relu(a(torch.randn(3, 4)))).sum().backward()
        assert set(seen) == {id(p) for p in list(a.parameters()) + list(b.parameters())}
        first_a = min(seen.index(id(p)) for p in a.parameters())
        last_b = max(seen.index(id(p)) for p in b.parameters())
        assert last_b < first_a                  # the later layer's gradients are ready first
    seen.clear()
    b(a(torch.randn(3, 4))).sum().backward()
    assert not seen
    assert core.gradient_norm(a.parameters()).item() > 0


def test_user_function_and_no_grad():
    class Square(core.Function):
        @staticmethod
        def forward(ctx, x):
            ctx.save_for_backward(x)
            return x * x

        @staticmethod
        def backward(ctx, g):
            (x,) = ctx.saved_tensors
            return 2 * x * g

    x = torch.tensor([3.0], requires_grad=True)
    core.backward(Square.apply(x).sum())
    assert x.grad.item() == 6.0
    with core.no_grad():
        assert not (x * 2).requires_grad


def test_scopes():
    assert core.product_precision() in ("float32", "bfloat16", "float16", "float8")
    lin = torch.nn.Linear(8, 8)
    with core.mixed_precision("bfloat16"):
        assert core.product_precision() == "bfloat16"
        assert lin(torch.randn(2, 8)).dtype == torch.bfloat16
        with core.mixed_precision("float32"):
            assert lin(torch.randn(2, 8)).dtype == torch.float32
    assert lin(torch.randn(2, 8)).dtype == torch.float32
    with pytest.raises(ValueError):
        with core.mixed_precision("int3"):
            pass
    from idrak_b200.models import DecoderSpec, build_decoder
    m = build_decoder(DecoderSpec.llama(layers=2, dim=32, heads=2, kv_heads=2, ff_dim=64, vocab=64, max_positions=32), seed=0)
    assert m.checkpoint_blocks is False
    ids = torch.randint(0, 64, (2, 16))
    with core.activation_memory(m, "checkpoint_blocks"):
        assert m.checkpoint_blocks is True
        l1 = m.loss(ids, ids)
        l1.backward()
    g1 = [p.grad.clone() for p in m.parameters()]
    m.zero_grad()
    assert m.checkpoint_blocks is False
    l2 = m.loss(ids, ids)
    l2.backward()
    assert torch.allclose(l1, l2)
    for a, p in zip(g1, m.parameters()):
        assert torch.allclose(a, p.grad, atol=1e-6)
    with core.TensorScope(trim=True):
        torch.zeros(4)


def test_slot_table_policies():
    ensured = []
    t = core.SlotTable("things", defaults=lambda tab: (ensured.append(1), tab.register("a", "default-a", "fallback")))
    assert t["a"] == "default-a" and ensured == [1]
    s = t.register("a", "plugin-a")
    assert t["a"] == "plugin-a"
    t.register("a", "late-default", "fallback")
    assert t["a"] == "plugin-a"
    with t.register("a", "scoped"):
        assert t["a"] == "scoped"
    assert t["a"] == "plugin-a"
    s.remove()
    assert t["a"] == "default-a"
    assert "b" not in t and t.get("b", 5) == 5
    with pytest.raises(KeyError, match="known: a"):
        t["b"]
    with pytest.raises(ValueError):
        t.register("c", 1, "replace")


@pytest.mark.gpu
def test_compute_graph_capture_and_replay():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    w = torch.randn(64, 64, device="cuda")
    g = core.ComputeGraph.capture(lambda a, b: torch.relu(a @ w) + b, torch.zeros(8, 64, device="cuda"),
                                  torch.zeros(8, 64, device="cuda"))
    for _ in range(3):
        a, b = torch.randn(8, 64, device="cuda"), torch.randn(8, 64, device="cuda")
        assert torch.allclose(g.replay(a, b), torch.relu(a @ w) + b, atol=1e-5)
    assert g.replays == 3
    with pytest.raises(ValueError):
        g.replay(torch.zeros(4, 64, device="cuda"), torch.zeros(8, 64, device="cuda"))
