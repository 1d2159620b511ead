"""Routed experts on the device: routing kernels, the permutation plan, grouped products and the whole layer against
the loop over experts in fp32."""
import pytest
import torch

from idrak_b200.ops import moe

pytestmark = pytest.mark.gpu


def _rand(shape, scale, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("T,E,k,normalize", [(1, 8, 2, True), (1000, 8, 2, True), (513, 64, 6, False), (77, 16, 1, True)])
def test_route_choose_matches_the_sorted_softmax_with_ties_to_the_lowest_id(T, E, k, normalize):
    g = torch.Generator(device="cuda").manual_seed(T)
    logits = torch.randn(T, E, generator=g, device="cuda")
    logits[::3] = logits[::3].round()                # plenty of exact ties
    if T > 4:
        logits[4] = 0.0                              # every expert equal: picks 0 .. k-1
    ids, w, probs = moe.route_choose(logits, k, normalize)
    ids_r, w_r, probs_r = moe.route_reference(logits, k, normalize)
    assert torch.equal(ids, ids_r)
    torch.testing.assert_close(w, w_r, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(probs, probs_r, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (700, 8, 2), (5000, 16, 4), (300, 64, 8)])
def test_plan_sorts_assignments_by_expert_in_token_order_with_padded_segments(T, E, k):
    g = torch.Generator(device="cuda").manual_seed(3)
    top_i = torch.stack([torch.randperm(E, generator=g, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    if E > 8:
        top_i[top_i == 5] = 6                        # an expert nobody picks (duplicates inside a token are fine here)
    plan = moe.RoutePlan(top_i, E)
    again = moe.RoutePlan(top_i, E)
    torch.cuda.synchronize()
    flat = top_i.reshape(-1).cpu()
    start, count = plan.seg_start.cpu(), plan.seg_count.cpu()
    row_of, dst_of, tile_group, meta = plan.row_of.cpu(), plan.dst_of.cpu(), plan.tile_group.cpu(), plan.meta.cpu()
    at = 0
    for e in range(E):
        mine = torch.nonzero(flat == e).reshape(-1)
        assert int(start[e]) == at and int(count[e]) == mine.numel()
        assert torch.equal(row_of[at:at + mine.numel()].long(), mine), "token order is kept inside an expert"
        padded = (mine.numel() + 127) // 128 * 128
        assert (row_of[at + mine.numel():at + padded] == -1).all()
        assert (tile_group[at // 128:(at + padded) // 128] == e).all()
        at += padded
    assert int(meta[0]) == at // 128 and int(meta[1]) == at and at <= plan.cap
    assert (tile_group[at // 128:] == -1).all()
    assert torch.equal(row_of[dst_of.long()].long(), torch.arange(T * k))
    assert torch.equal(plan.group_kb.cpu()[:-1], (start // 64).to(torch.int32)) and int(plan.group_kb[-1]) == at // 64
    assert torch.equal(again.row_of.cpu()[:at], row_of[:at]) and torch.equal(again.dst_of.cpu(), dst_of)


def test_gather_and_combine_are_inverse_views_of_the_plan():
    T, E, k, C = 300, 8, 2, 256
    x = _rand((T, C), 1.0, 1)
    logits = torch.randn(T, E, device="cuda")
    ids, w, _ = moe.route_choose(logits, k, True)
    plan = moe.RoutePlan(ids, E)
    xp = plan.gather(x)
    rows = int(plan.meta[1])
    src = plan.row_of[:rows].long()
    want = torch.where((src >= 0)[:, None], x[(src.clamp(min=0) // k)], torch.zeros_like(x[:1]))
    assert torch.equal(xp[:rows], want)
    out, dw = plan.combine(xp, w, residual=x, grad=x)
    ref = x.float() * w.sum(-1, keepdim=True) + x.float()
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(dw, (x.float() ** 2).sum(-1, keepdim=True).expand(T, k), atol=0.5, rtol=1e-2)


@pytest.mark.parametrize("T,E,k,dim,ff,gated,kind", [
    (1000, 8, 2, 256, 512, True, "silu"),          # Mixtral-shaped, scaled down
    (40, 8, 2, 128, 256, True, "gelu"),            # fewer tokens than experts x tile: empty and tiny segments
    (2048, 16, 4, 256, 384, True, "silu"),
    (600, 8, 1, 128, 128, False, "gelu"),
])
def test_routed_layer_matches_the_loop_over_experts(T, E, k, dim, ff, gated, kind):
    x = _rand((T, dim), 1.0, 1).requires_grad_()
    router = _rand((E, dim), 0.2, 2).requires_grad_()
    up = _rand((E, (2 if gated else 1) * ff, dim), dim ** -0.5, 3).requires_grad_()
    down = _rand((E, dim, ff), ff ** -0.5, 4).requires_grad_()
    res = _rand((T, dim), 1.0, 5)
    assert moe.supported(x, up, down, gated, kind)
    y = moe.routed_experts(x, router, up, down, k, True, gated, kind, res)
    dy = _rand((T, dim), 1.0, 6)
    y.backward(dy)
    ref_in = [t.detach().float().requires_grad_() for t in (x, router, up, down)]
    yr = moe.routed_experts_reference(ref_in[0], ref_in[1], ref_in[2], ref_in[3], k, True, gated, kind, res.float())
    yr.backward(dy.float())

    def close(a, b, tol):
        scale = max(1.0, b.abs().max().item())
        err = (a.float() - b).abs().max().item()
        assert err <= tol * scale, f"{err} > {tol * scale}"
    close(y, yr, 2e-2)
    close(x.grad, ref_in[0].grad, 3e-2)
    close(up.grad, ref_in[2].grad, 3e-2)
    close(down.grad, ref_in[3].grad, 3e-2)
    close(router.grad, ref_in[1].grad, 5e-2)


def test_routed_layer_records_into_a_cuda_graph_and_replays_bit_for_bit():
    T, E, k, dim, ff = 512, 8, 2, 128, 256
    x = _rand((T, dim), 1.0, 1).requires_grad_()
    router, up, down = (_rand((E, dim), 0.2, 2).requires_grad_(), _rand((E, 2 * ff, dim), 0.1, 3).requires_grad_(),
                        _rand((E, dim, ff), 0.1, 4).requires_grad_())
    dy = _rand((T, dim), 1.0, 6)

    def step():
        # fresh leaves every time: a leaf remembers the stream it was first used on, and the capture runs on its own
        xx, uu = x.detach().requires_grad_(), up.detach().requires_grad_()
        y = moe.routed_experts(xx, router.detach(), uu, down.detach(), k)
        gx, gu = torch.autograd.grad(y, [xx, uu], dy)
        return y, gx, gu
    eager = [t.clone() for t in step()]
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):                    # any host read of device data in here would raise
        captured = step()
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, captured):
        assert torch.equal(a, b)


def test_decoder_with_experts_uses_the_device_path_and_matches_the_loop():
    from idrak_b200.models import DecoderSpec, build_decoder
    spec = DecoderSpec.llama(layers=2, dim=128, heads=2, kv_heads=2, ff_dim=256, vocab=512, max_positions=256)
    spec.head_dim = 64
    spec.experts, spec.experts_per_token, spec.expert_ff_dim = 8, 2, 128
    model = build_decoder(spec, seed=2).to("cuda", torch.bfloat16)
    block = model.blocks[0].mlp
    assert block._stacked_now() is not None
    x = _rand((3, 50, 128), 1.0, 1)
    from idrak_b200 import _native
    before = _native.lib().idrak_launch_count()
    fast = block(x, x)
    used = _native.lib().idrak_launch_count() - before
    slow = block._forward_loop(x, x)
    assert used >= 8, "the routed path launches this library's kernels"
    assert (fast.float() - slow.float()).abs().max().item() <= 3e-2 * max(1.0, slow.float().abs().max().item())
    ids = torch.randint(0, 512, (2, 64), device="cuda", dtype=torch.int32)
    loss = model.loss(ids, ids)
    loss.backward()
    g = block.experts[3].up_weight.grad
    assert g is not None and torch.isfinite(g).all() and block.router.grad is not None
    torch.cuda.synchronize()
    _native.check_status("moe decoder")
