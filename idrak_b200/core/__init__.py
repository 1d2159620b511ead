"""Core API shape over PyTorch: autograd helpers, scopes, mixed precision, activation memory, registries."""
from .autograd import Function, GradientReadyHandle, backward, enable_grad, gradient_norm, no_grad, on_gradient_ready
from .checkpointing import checkpoint, run_block
from .registry import Slot, SlotTable
from .scopes import ComputeGraph, TensorScope, activation_memory, mixed_precision, product_precision
