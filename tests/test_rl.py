import math

import numpy as np
import torch

from idrak_b200 import rl
from idrak_b200.nn import Network


def test_gae_matches_the_definition():
    torch.manual_seed(0)
    T, gamma, lam = 7, 0.9, 0.8
    r, v = torch.randn(T), torch.randn(T)
    dones = torch.tensor([0, 0, 1, 0, 0, 0, 0], dtype=torch.bool)
    last = torch.tensor(0.7)
    adv, ret = rl.gae(r, v, dones, last, gamma, lam)
    # direct sums of discounted residuals, stopping at episode ends
    vals = torch.cat([v, last[None]])
    for t in range(T):
        a, w = 0.0, 1.0
        for k in range(t, T):
            alive = 0.0 if dones[k] else 1.0
            a += w * (r[k] + gamma * vals[k + 1] * alive - v[k])
            if dones[k]:
                break
            w *= gamma * lam
        assert abs(adv[t].item() - float(a)) < 1e-5
    assert torch.allclose(ret, adv + v)
    # lam = 1 gives discounted returns minus values
    adv1, ret1 = rl.gae(r, v, torch.zeros(T, dtype=torch.bool), torch.tensor(0.0), gamma, 1.0)
    assert torch.allclose(ret1, rl.discounted_returns(r, torch.zeros(T, dtype=torch.bool), gamma), atol=1e-5)


def test_group_advantages_and_losses():
    a = rl.group_advantages(torch.tensor([1.0, 0.0, 0.0, 1.0, 5.0, 5.0, 5.0, 5.0]), 4)
    assert torch.allclose(a[:4], torch.tensor([1.0, -1.0, -1.0, 1.0]), atol=1e-4) and a[4:].abs().max() < 1e-3
    lp_old = torch.log(torch.tensor([0.5, 0.5, 0.5]))
    adv = torch.tensor([1.0, 1.0, -1.0])
    lp = torch.log(torch.tensor([0.5, 0.9, 0.9])).requires_grad_()
    loss, stats = rl.clipped_policy_loss(lp, lp_old, adv, 0.2)
    # ratios 1, 1.8 (clipped to 1.2 for a positive advantage), 1.8 (not clipped for a negative one)
    assert abs(loss.item() + (1.0 + 1.2 - 1.8) / 3) < 1e-6 and abs(stats["clip_fraction"] - 2 / 3) < 1e-6
    loss.backward()
    assert lp.grad[1].item() == 0.0 and lp.grad[2].item() != 0.0
    mask = torch.tensor([[1, 1, 0], [1, 0, 0]])
    lp2 = torch.zeros(2, 3)
    g, s = rl.grpo_loss(lp2, lp2, lp2 - 0.1, torch.tensor([1.0, -1.0]), mask, kl_weight=0.5)
    kl = math.exp(-0.1) + 0.1 - 1
    assert abs(g.item() - (-(1 + 1 - 1) / 3 + 0.5 * kl)) < 1e-6 and abs(s["reference_kl"] - kl) < 1e-6
    assert rl.value_loss(torch.tensor([1.0]), torch.tensor([3.0])).item() == 2.0
    assert rl.value_loss(torch.tensor([2.0]), torch.tensor([3.0]), torch.tensor([0.0]), 0.5).item() == 0.5 * 2.5 ** 2
    assert abs(rl.categorical_entropy(torch.zeros(4)).item() - math.log(4)) < 1e-6


def test_replay_buffer_and_environments():
    buf = rl.ReplayBuffer(5, seed=1)
    for i in range(8):
        buf.add(obs=np.full(3, i, np.float32), action=i, reward=float(i))
    assert len(buf) == 5
    s = buf.sample(64)
    assert s["obs"].shape == (64, 3) and set(s["action"].tolist()) <= {3, 4, 5, 6, 7} and len(set(s["action"].tolist())) > 2
    env = rl.CartPole(seed=0)
    o = env.reset()
    steps, done = 0, False
    while not done:
        o, r, done = env.step(0)            # always pushing left tips the pole quickly
        steps += 1
    assert 5 < steps < 20 and o.shape == (4,)
    p = rl.Pendulum(seed=0)
    o = p.reset()
    total = sum(p.step(0.0)[1] for _ in range(200))
    assert o.shape == (3,) and total < 0 and p.step(0.0)[2]
    b = rl.Bandit([0.1, 0.9], seed=0)
    assert np.mean([b.step(1)[1] for _ in range(500)]) > 0.8 and b.step(0)[2]


def test_ppo_learns_cartpole():
    torch.manual_seed(0)
    env = rl.CartPole(seed=0, limit=200)
    policy = Network.input(4).linear(32).tanh().linear(2).build()
    value = Network.input(4).linear(32).tanh().linear(1).build()
    trainer = rl.OnPolicyTrainer(env, policy, value, steps_per_update=1024, epochs=6, minibatch=256, learning_rate=5e-3, seed=0)
    history = trainer.train(12)
    first, best = history[0]["mean_return"], max(h["mean_return"] for h in history)
    assert best > 2.5 * first and best > 80, (first, best)


def test_rollouts_are_exchanged_across_ranks(tmp_path):
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    from rollout_worker import episodes_of
    out = tmp_path / "r.pt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29771", os.path.join(here, "rollout_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    got = torch.load(out)
    want = [e for rank in range(3) for e in episodes_of(rank)]
    assert len(got["all"]) == len(want) == 6 and all(torch.equal(a, b) for a, b in zip(got["all"], want))
    assert [e.tolist() for e in got["empty"]] == [[1.5, 2.5], [1.5, 2.5]]
    solo = rl.exchange_rollouts([torch.tensor([1, 2, 3])])
    assert solo[0].tolist() == [1, 2, 3]
