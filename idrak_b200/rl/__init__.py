"""Reinforcement learning: advantages (GAE, group-relative), clipped policy losses (PPO, GRPO-style), value and entropy
terms, a replay buffer, small environments (CartPole, Pendulum, a bandit) and an on-policy trainer that ties them
together. Language-model policies use the same losses over token log-probabilities.

    env = CartPole(seed=0)
    policy = Network.input(4).linear(64).tanh().linear(2).build()
    value = Network.input(4).linear(64).tanh().linear(1).build()
    trainer = OnPolicyTrainer(env, policy, value, steps_per_update=1024)
    history = trainer.train(updates=30)

Reference: src/Idrak.Reinforcement (Advantages.cs: GAE / group advantages; PolicyLosses.cs: clipped surrogate, KL
penalty; ReplayBuffer.cs; OnPolicyTrainer / OffPolicyTrainer) and its plug-in environments (CartPole, Pendulum, bandit).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------------------------------
# advantages
# ---------------------------------------------------------------------------------------------------------------------
def gae(rewards: torch.Tensor, values: torch.Tensor, dones: torch.Tensor, last_value: torch.Tensor,
        gamma: float = 0.99, lam: float = 0.95) -> Tuple[torch.Tensor, torch.Tensor]:
    """Generalised advantage estimation over ``[T, ...]`` rollouts. ``dones[t]`` marks that step ``t`` ended an episode
    (no bootstrap across it). Returns (advantages, returns = advantages + values)."""
    T = rewards.shape[0]
    adv = torch.zeros_like(rewards)
    running = torch.zeros_like(last_value)
    nxt = last_value
    for t in range(T - 1, -1, -1):
        alive = 1.0 - dones[t].float()
        delta = rewards[t] + gamma * nxt * alive - values[t]
        running = delta + gamma * lam * alive * running
        adv[t] = running
        nxt = values[t]
    return adv, adv + values


def discounted_returns(rewards: torch.Tensor, dones: torch.Tensor, gamma: float = 0.99) -> torch.Tensor:
    out = torch.zeros_like(rewards)
    running = torch.zeros_like(rewards[0])
    for t in range(rewards.shape[0] - 1, -1, -1):
        running = rewards[t] + gamma * running * (1.0 - dones[t].float())
        out[t] = running
    return out


def group_advantages(rewards: torch.Tensor, group_size: int, epsilon: float = 1e-6, scale: bool = True) -> torch.Tensor:
    """Group-relative advantages: rewards ``[groups * group_size]`` of several samples per prompt, each centred on
    its group's mean (and divided by the group's standard deviation)."""
    r = rewards.float().view(-1, group_size)
    a = r - r.mean(1, keepdim=True)
    if scale:
        a = a / (r.std(1, keepdim=True, unbiased=False) + epsilon)
    return a.view(-1)


def normalise(advantages: torch.Tensor, epsilon: float = 1e-8) -> torch.Tensor:
    return (advantages - advantages.mean()) / (advantages.std(unbiased=False) + epsilon)


# ---------------------------------------------------------------------------------------------------------------------
# losses
# ---------------------------------------------------------------------------------------------------------------------
def clipped_policy_loss(log_probs: torch.Tensor, old_log_probs: torch.Tensor, advantages: torch.Tensor, clip: float = 0.2,
                        mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Dict[str, float]]:
    """PPO's clipped surrogate (to minimise). ``mask`` selects the entries that count (generated tokens)."""
    ratio = (log_probs - old_log_probs).exp()
    surrogate = torch.minimum(ratio * advantages, ratio.clamp(1 - clip, 1 + clip) * advantages)
    m = torch.ones_like(surrogate) if mask is None else mask.float()
    n = m.sum().clamp_min(1.0)
    loss = -(surrogate * m).sum() / n
    with torch.no_grad():
        stats = {"clip_fraction": float((((ratio - 1).abs() > clip).float() * m).sum() / n),
                 "approx_kl": float((((ratio - 1) - (log_probs - old_log_probs)) * m).sum() / n)}
    return loss, stats


def grpo_loss(log_probs: torch.Tensor, old_log_probs: torch.Tensor, reference_log_probs: Optional[torch.Tensor],
              advantages: torch.Tensor, mask: torch.Tensor, clip: float = 0.2, kl_weight: float = 0.04) -> Tuple[torch.Tensor, Dict[str, float]]:
    """Token-level clipped surrogate with one advantage per sequence (``advantages`` [N] broadcast over ``[N, T]``) plus
    a penalty towards a reference policy: the unbiased estimator ``exp(ref - lp) - (ref - lp) - 1``."""
    loss, stats = clipped_policy_loss(log_probs, old_log_probs, advantages[:, None].expand_as(log_probs), clip, mask)
    if reference_log_probs is not None and kl_weight:
        d = reference_log_probs - log_probs
        kl = d.exp() - d - 1.0
        m = mask.float()
        kl_mean = (kl * m).sum() / m.sum().clamp_min(1.0)
        loss = loss + kl_weight * kl_mean
        stats["reference_kl"] = float(kl_mean)
    return loss, stats


def value_loss(values: torch.Tensor, returns: torch.Tensor, old_values: Optional[torch.Tensor] = None, clip: Optional[float] = None):
    if clip is None or old_values is None:
        return 0.5 * (values - returns).pow(2).mean()
    clipped = old_values + (values - old_values).clamp(-clip, clip)
    return 0.5 * torch.maximum((values - returns).pow(2), (clipped - returns).pow(2)).mean()


def categorical_entropy(logits: torch.Tensor) -> torch.Tensor:
    lp = F.log_softmax(logits, -1)
    return -(lp.exp() * lp).sum(-1)


# ---------------------------------------------------------------------------------------------------------------------
# replay buffer
# ---------------------------------------------------------------------------------------------------------------------
class ReplayBuffer:
    """Fixed-capacity ring of transitions stored as tensors; uniform sampling with a seeded generator."""

    def __init__(self, capacity: int, seed: int = 0):
        self.capacity, self.size, self.at = capacity, 0, 0
        self.fields: Dict[str, torch.Tensor] = {}
        self.rng = np.random.default_rng(seed)

    def add(self, **transition) -> None:
        for k, v in transition.items():
            t = torch.as_tensor(v)
            if k not in self.fields:
                self.fields[k] = torch.zeros((self.capacity,) + tuple(t.shape), dtype=t.dtype)
            self.fields[k][self.at] = t
        self.at = (self.at + 1) % self.capacity
        self.size = min(self.size + 1, self.capacity)

    def sample(self, batch: int) -> Dict[str, torch.Tensor]:
        if self.size == 0:
            raise ValueError("the buffer is empty")
        idx = torch.from_numpy(self.rng.integers(0, self.size, batch))
        return {k: v[idx] for k, v in self.fields.items()}

    def __len__(self) -> int:
        return self.size


# ---------------------------------------------------------------------------------------------------------------------
# environments
# ---------------------------------------------------------------------------------------------------------------------
class Environment:
    observation_size: int
    actions: int                     # number of discrete actions, or 0 for a continuous action

    def reset(self) -> np.ndarray:
        raise NotImplementedError

    def step(self, action) -> Tuple[np.ndarray, float, bool]:
        raise NotImplementedError


class CartPole(Environment):
    """The classic pole balancing task (Barto, Sutton and Anderson's dynamics, Euler steps of 20 ms): reward 1 per
    step, the episode ends when the pole passes 12 degrees, the cart leaves +-2.4 or after ``limit`` steps."""
    observation_size, actions = 4, 2

    def __init__(self, seed: int = 0, limit: int = 500):
        self.rng, self.limit = np.random.default_rng(seed), limit
        self.state = np.zeros(4)
        self.t = 0

    def reset(self):
        self.state = self.rng.uniform(-0.05, 0.05, 4)
        self.t = 0
        return self.state.astype(np.float32)

    def step(self, action):
        x, xd, th, thd = self.state
        force = 10.0 if int(action) == 1 else -10.0
        g, mc, mp, length, tau = 9.8, 1.0, 0.1, 0.5, 0.02
        total, pml = mc + mp, mp * length
        cos, sin = math.cos(th), math.sin(th)
        temp = (force + pml * thd * thd * sin) / total
        thacc = (g * sin - cos * temp) / (length * (4.0 / 3.0 - mp * cos * cos / total))
        xacc = temp - pml * thacc * cos / total
        self.state = np.array([x + tau * xd, xd + tau * xacc, th + tau * thd, thd + tau * thacc])
        self.t += 1
        done = abs(self.state[0]) > 2.4 or abs(self.state[2]) > 12 * math.pi / 180 or self.t >= self.limit
        return self.state.astype(np.float32), 1.0, bool(done)


class Pendulum(Environment):
    """Swing-up with a continuous torque in [-2, 2]; observation (cos, sin, angular velocity); 200-step episodes."""
    observation_size, actions = 3, 0

    def __init__(self, seed: int = 0, limit: int = 200):
        self.rng, self.limit = np.random.default_rng(seed), limit
        self.th = self.thd = 0.0
        self.t = 0

    def _obs(self):
        return np.array([math.cos(self.th), math.sin(self.th), self.thd], np.float32)

    def reset(self):
        self.th, self.thd, self.t = float(self.rng.uniform(-math.pi, math.pi)), float(self.rng.uniform(-1, 1)), 0
        return self._obs()

    def step(self, action):
        u = float(np.clip(action, -2.0, 2.0))
        norm = ((self.th + math.pi) % (2 * math.pi)) - math.pi
        cost = norm * norm + 0.1 * self.thd * self.thd + 0.001 * u * u
        self.thd = float(np.clip(self.thd + (3 * 10.0 / 2 * math.sin(self.th) + 3.0 * u) * 0.05, -8, 8))
        self.th += self.thd * 0.05
        self.t += 1
        return self._obs(), -cost, self.t >= self.limit


class Bandit(Environment):
    """``arms`` Bernoulli arms with fixed success rates; one-step episodes; observation is a constant 1."""
    observation_size = 1

    def __init__(self, probabilities: Sequence[float], seed: int = 0):
        self.p, self.actions = np.asarray(probabilities, np.float64), len(probabilities)
        self.rng = np.random.default_rng(seed)

    def reset(self):
        return np.ones(1, np.float32)

    def step(self, action):
        return np.ones(1, np.float32), float(self.rng.random() < self.p[int(action)]), True


# ---------------------------------------------------------------------------------------------------------------------
# rollouts across ranks
# ---------------------------------------------------------------------------------------------------------------------
def exchange_rollouts(episodes: Sequence[torch.Tensor], group=None) -> List[torch.Tensor]:
    """All ranks' episodes on every rank. Each episode is a 1-D tensor (token ids, or flattened transitions) of any
    length; ranks may hold different numbers of episodes. Two collectives: the counts and longest length, then the
    episodes padded to that length. The result is ordered by rank, then by the rank's own order."""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [e.clone() for e in episodes]
    world = dist.get_world_size(group)
    dtype = episodes[0].dtype if episodes else torch.int64
    device = episodes[0].device if episodes else torch.device("cpu")
    mine = torch.tensor([len(episodes), max((len(e) for e in episodes), default=0),
                         int(bool(episodes) and dtype.is_floating_point)], dtype=torch.int64, device=device)
    counts = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(counts, mine, group=group)
    most, longest = max(int(c[0]) for c in counts), max(int(c[1]) for c in counts)
    floating = any(int(c[2]) for c in counts)             # a rank without episodes does not know the type: agree on it
    if not episodes:
        dtype = torch.float32 if floating else torch.int64
    block = torch.zeros(most, longest + 1, dtype=torch.float64 if floating else torch.int64, device=device)
    for i, e in enumerate(episodes):
        block[i, 0] = len(e)
        block[i, 1: 1 + len(e)] = e.to(block.dtype)
    blocks = [torch.zeros_like(block) for _ in range(world)]
    dist.all_gather(blocks, block, group=group)
    out = []
    for r in range(world):
        for i in range(int(counts[r][0])):
            n = int(blocks[r][i, 0])
            out.append(blocks[r][i, 1: 1 + n].to(dtype))
    return out


# ---------------------------------------------------------------------------------------------------------------------
# on-policy trainer (PPO with a separate value network; discrete actions)
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class OnPolicyOptions:
    steps_per_update: int = 1024
    epochs: int = 4
    minibatch: int = 256
    gamma: float = 0.99
    lam: float = 0.95
    clip: float = 0.2
    entropy_weight: float = 0.01
    value_weight: float = 0.5
    learning_rate: float = 3e-3
    max_grad_norm: float = 0.5
    seed: int = 0


class OnPolicyTrainer:
    def __init__(self, env: Environment, policy: torch.nn.Module, value: torch.nn.Module,
                 options: Optional[OnPolicyOptions] = None, **overrides):
        if env.actions <= 0:
            raise ValueError("this trainer handles discrete actions")
        self.env, self.policy, self.value = env, policy, value
        self.o = options or OnPolicyOptions()
        for k, v in overrides.items():
            setattr(self.o, k, v)
        self.opt = torch.optim.Adam(list(policy.parameters()) + list(value.parameters()), lr=self.o.learning_rate)
        self.gen = torch.Generator().manual_seed(self.o.seed)
        self.obs = torch.from_numpy(env.reset())
        self.episode_return, self.finished = 0.0, []

    @torch.no_grad()
    def collect(self) -> Dict[str, torch.Tensor]:
        o = self.o
        obs, act, lp, rew, done, val = [], [], [], [], [], []
        for _ in range(o.steps_per_update):
            logits = self.policy(self.obs[None])[0]
            a = int(torch.multinomial(logits.softmax(-1), 1, generator=self.gen))
            obs.append(self.obs)
            act.append(a)
            lp.append(F.log_softmax(logits, -1)[a])
            val.append(self.value(self.obs[None])[0, 0])
            nxt, r, d = self.env.step(a)
            self.episode_return += r
            rew.append(r)
            done.append(d)
            if d:
                self.finished.append(self.episode_return)
                self.episode_return = 0.0
                nxt = self.env.reset()
            self.obs = torch.from_numpy(nxt)
        last = self.value(self.obs[None])[0, 0]
        rewards, dones, values = torch.tensor(rew), torch.tensor(done), torch.stack(val)
        adv, ret = gae(rewards, values, dones, last, o.gamma, o.lam)
        return {"obs": torch.stack(obs), "actions": torch.tensor(act), "log_probs": torch.stack(lp), "advantages": adv,
                "returns": ret, "values": values}

    def update(self, batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
        o = self.o
        n = batch["obs"].shape[0]
        adv = normalise(batch["advantages"])
        stats: Dict[str, float] = {}
        for _ in range(o.epochs):
            order = torch.randperm(n, generator=self.gen)
            for i in range(0, n, o.minibatch):
                idx = order[i: i + o.minibatch]
                logits = self.policy(batch["obs"][idx])
                lp = F.log_softmax(logits, -1).gather(1, batch["actions"][idx, None])[:, 0]
                pl, stats = clipped_policy_loss(lp, batch["log_probs"][idx], adv[idx], o.clip)
                vl = value_loss(self.value(batch["obs"][idx])[:, 0], batch["returns"][idx])
                ent = categorical_entropy(logits).mean()
                loss = pl + o.value_weight * vl - o.entropy_weight * ent
                self.opt.zero_grad()
                loss.backward()
                torch.nn.utils.clip_grad_norm_(list(self.policy.parameters()) + list(self.value.parameters()), o.max_grad_norm)
                self.opt.step()
                stats.update(policy_loss=float(pl.detach()), value_loss=float(vl.detach()), entropy=float(ent.detach()))
        return stats

    def train(self, updates: int, on_update: Optional[Callable[[int, Dict[str, float]], None]] = None) -> List[Dict[str, float]]:
        history = []
        for u in range(updates):
            seen = len(self.finished)
            stats = self.update(self.collect())
            recent = self.finished[seen:] or self.finished[-1:]
            stats["mean_return"] = float(np.mean(recent)) if recent else 0.0
            history.append(stats)
            if on_update:
                on_update(u, stats)
        return history
