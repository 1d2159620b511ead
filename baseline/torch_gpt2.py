"""The comparison arm of ``bench.py --impl torch``: the same GPT-2 training step written the usual PyTorch way -
library kernels only (cuBLAS matmuls, the library's fused attention, fused AdamW) and NCCL through
``DistributedDataParallel``. Nothing of this package runs on this path; it is the "what you get without the
hand-written kernels" number measured on the same GPU, with the same model, batch, optimizer settings and timing
as the main arm.

Numerics match the main arm: bf16 parameters and activations, fp32 master weights and moments in the optimizer,
gradient clipping at 1.0, AdamW (0.9, 0.95), weight decay 0.1 on matrices only; on one GPU the step is replayed from
a CUDA graph like the main arm's.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn


class Block(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.ln1 = nn.LayerNorm(dim)
        self.qkv = nn.Linear(dim, 3 * dim)
        self.proj = nn.Linear(dim, dim)
        self.ln2 = nn.LayerNorm(dim)
        self.up = nn.Linear(dim, 4 * dim)
        self.down = nn.Linear(4 * dim, dim)

    def forward(self, x):
        B, T, C = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, C))
        return x + self.down(F.gelu(self.up(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, layers: int, dim: int, heads: int, vocab: int, max_positions: int):
        super().__init__()
        self.wte = nn.Embedding(vocab, dim)
        self.wpe = nn.Embedding(max_positions, dim)
        self.blocks = nn.ModuleList([Block(dim, heads) for _ in range(layers)])
        self.ln_f = nn.LayerNorm(dim)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)
        for b in self.blocks:
            nn.init.normal_(b.proj.weight, std=0.02 / math.sqrt(2 * layers))
            nn.init.normal_(b.down.weight, std=0.02 / math.sqrt(2 * layers))

    def forward(self, ids, targets):
        T = ids.shape[1]
        x = self.wte(ids) + self.wpe(torch.arange(T, device=ids.device))
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)            # tied output head
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))


class TorchStep:
    """forward + backward + clip + AdamW the way a tuned PyTorch script does it: bf16 parameters and activations,
    fp32 master weights and moments stepped by the fused (capturable) AdamW, and - on one GPU - the whole step
    captured in a CUDA graph so the host's launch cost is off the clock. Under more than one rank the model runs
    in DistributedDataParallel (NCCL all-reduce overlapped with backward) without the graph."""

    def __init__(self, layers, dim, heads, vocab, seq, device, world, use_graph: bool = True):
        torch.manual_seed(1234)
        self.device = device
        self.model = GPT2(layers, dim, heads, vocab, seq).to(device).to(torch.bfloat16)
        self.params = [p for p in self.model.parameters()]
        self.master = [p.detach().float().clone() for p in self.params]
        for m in self.master:
            m.grad = torch.zeros_like(m)
        decay = [m for m, p in zip(self.master, self.params) if p.dim() >= 2]
        plain = [m for m, p in zip(self.master, self.params) if p.dim() < 2]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": plain, "weight_decay": 0.0}],
                                     lr=6e-4, betas=(0.9, 0.95), fused=True, capturable=True)
        self.net = self.model
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel
            self.net = DistributedDataParallel(self.model, device_ids=[device.index], gradient_as_bucket_view=True)
        self.graph = None
        self.use_graph = use_graph and world == 1
        self.static_ids = self.static_tgt = self.static_loss = None

    def _body(self, ids, targets):
        loss = self.net(ids.long(), targets.long())
        loss.backward()
        with torch.no_grad():
            torch._foreach_copy_([m.grad for m in self.master], [p.grad for p in self.params])
            torch.nn.utils.clip_grad_norm_(self.master, 1.0, foreach=True)
            self.opt.step()
            torch._foreach_copy_(self.params, self.master)
            torch._foreach_zero_([p.grad for p in self.params])
        return loss.detach()

    def _capture(self, ids, targets):
        self.static_ids, self.static_tgt = ids.clone(), targets.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):                       # warm-up outside the graph: allocations, optimizer state
                self._body(self.static_ids, self.static_tgt)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.static_loss = self._body(self.static_ids, self.static_tgt)
        self.graph = g

    def __call__(self, ids, targets):
        if not self.use_graph:
            return self._body(ids, targets)
        if self.graph is None:
            try:
                self._capture(ids, targets)
            except Exception:                        # a PyTorch build that cannot capture this step: run it eagerly
                self.use_graph = False
                torch.cuda.synchronize()
                return self._body(ids, targets)
        self.static_ids.copy_(ids, non_blocking=True)
        self.static_tgt.copy_(targets, non_blocking=True)
        self.graph.replay()
        return self.static_loss

    def step_from_host(self, host_ids, host_targets):
        ids = host_ids.to(self.device, non_blocking=True)
        tgt = host_targets.to(self.device, non_blocking=True)
        return float(self(ids, tgt).item())
