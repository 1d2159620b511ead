"""Core API shape over PyTorch: autograd helpers, scopes, mixed precision, activation memory, registries."""
from .autograd import Function, GradientReadyHandle, backward, enable_grad, gradient_norm, no_grad, on_gradient_ready
from .checkpointing import checkpoint, run_block
from .registry import Slot, SlotTable
from .scopes import (ComputeGraph, TensorScope, activation_memory, compress_saved_to_bfloat16, mixed_precision,
                     product_precision, recompute)
from .backend import (Backend, CpuBackend, CudaBackend, DeviceMemoryExceeded, MemoryAccountant, Operation, backend_for,
                      create_separate_backend, operation_report, register_kernel, run)
from .device import DeferredTensor, DeferredTensors, Device
from .plugins import KindTable, LibraryDefaults, Option, OptionSchema, load_plugins, loaded_plugins
