"""Activation checkpointing of a block: forward without recording, one graph node whose backward re-runs
the forward with the random state of the first pass and then differentiates it.

Reference: Checkpointing.Checkpoint / RunBlock (src/Idrak/Layers/Checkpointing.cs:15-91),
ModuleExtensions.ForwardCheckpointed (src/Idrak/Layers/ModuleExtensions.cs:44).
"""
from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint as _torch_checkpoint


def checkpoint(fn, *args, preserve_rng_state: bool = True):
    """Run ``fn(*args)`` keeping only its inputs; intermediate activations are recomputed in backward."""
    return _torch_checkpoint(fn, *args, use_reentrant=False, preserve_rng_state=preserve_rng_state)


def run_block(block: torch.nn.Module, x: torch.Tensor, *extra, enabled: bool = True):
    if enabled and torch.is_grad_enabled() and x.requires_grad:
        return checkpoint(block, x, *extra)
    return block(x, *extra)
