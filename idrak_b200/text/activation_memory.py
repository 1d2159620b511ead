"""How much activation memory a decoder training step holds, and the ladder of policies that trade it for
recomputation: ``held`` (keep everything) -> ``checkpoint_blocks`` (keep block inputs, re-run each block in backward).
The fine-tuner estimates before its first step, starts on the first rung that fits the free memory, and steps down
when a step still runs out of memory.

The estimate counts, per token and layer, what the autograd graph of this package's decoder saves in bf16 (2 bytes):
the two norm inputs, the packed q / k / v, the attention output, the gate / up projection, the activated product and the
row statistics; plus the loss rows and the adapters' low-rank intermediates.

Reference: ActivationEstimate and the activation ladder of the fine-tuner (src/Idrak.Text/ActivationEstimate.cs;
FineTuning.cs: held -> recompute FF -> bf16 activations -> checkpoint blocks, estimated before the first step and stepped
down on out-of-memory).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

LADDER = ("held", "checkpoint_blocks")


@dataclass
class ActivationEstimate:
    policy: str
    bytes_per_token_layer: int
    total_bytes: int

    @property
    def gib(self) -> float:
        return self.total_bytes / 2 ** 30


def estimate(spec, tokens: int, policy: str = "held", element_bytes: int = 2, adapter_rank: int = 0,
             loss_chunk_rows: int = 512) -> ActivationEstimate:
    """Bytes of saved activations for ``tokens`` tokens in one step under ``policy``."""
    if policy not in LADDER:
        raise ValueError(f"unknown policy '{policy}'; ladder: {', '.join(LADDER)}")
    d, ff = spec.dim, spec.ff_dim
    qkv = (spec.heads + 2 * spec.kv_heads) * spec.head_dim
    gate_up = ff * (2 if spec.gated else 1)
    per_layer = element_bytes * (2 * d                 # inputs of the two norms
                                 + qkv                 # packed q, k, v (after RoPE)
                                 + spec.heads * spec.head_dim      # attention output
                                 + gate_up             # gate / up projection (pre-activation)
                                 + ff                  # activated product fed to the down projection
                                 + d)                  # residual stream copy
    per_layer += 4 * (2 + spec.heads)                  # norm statistics and the attention log-sum-exp, fp32
    if adapter_rank:
        per_layer += element_bytes * adapter_rank * 7  # one low-rank intermediate per adapted projection
    if policy == "checkpoint_blocks":
        held = element_bytes * d * spec.layers         # block inputs only ...
        held += per_layer                              # ... plus one block being recomputed
    else:
        held = per_layer * spec.layers
    total = held * tokens
    total += min(tokens, loss_chunk_rows) * spec.padded_vocabulary * 4 * 2     # one chunk of logits and its gradient, fp32
    return ActivationEstimate(policy, per_layer, int(total))


def choose_policy(spec, tokens: int, free_bytes: int, adapter_rank: int = 0, headroom: float = 0.85,
                  start: str = "held") -> ActivationEstimate:
    """The first rung from ``start`` downwards whose estimate fits ``headroom`` x ``free_bytes``; the last rung is
    returned even when it does not fit (the step will say so itself)."""
    rungs = LADDER[LADDER.index(start):]
    est = None
    for policy in rungs:
        est = estimate(spec, tokens, policy, adapter_rank=adapter_rank)
        if est.total_bytes <= headroom * free_bytes:
            return est
    return est


def next_rung(policy: str) -> Optional[str]:
    i = LADDER.index(policy)
    return LADDER[i + 1] if i + 1 < len(LADDER) else None


def apply_policy(model, policy: str) -> None:
    for m in model.modules():
        if hasattr(m, "checkpoint_blocks"):
            m.checkpoint_blocks = policy == "checkpoint_blocks"


def free_device_bytes(device) -> int:
    dev = torch.device(device)
    if dev.type != "cuda":
        return 1 << 62
    free, _ = torch.cuda.mem_get_info(dev)
    # blocks the caching allocator holds but does not use are free for this purpose
    return int(free + torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev))
