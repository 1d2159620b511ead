"""What the current device can hold, and the tile shapes the kernels were built with.

``device_limits()`` reads the limits the launchers depend on (SM count, shared memory a block may opt into, L2 size,
resident blocks and threads per SM, tensor-memory columns, clocks) from the CUDA runtime through the native library;
without a GPU it returns the B200 figures the kernels were written for, marked ``measured=False``. ``kernel_shapes()``
is the table of compile-time tile shapes (rows x columns x K step, pipeline stages, threads, shared memory) of the
tensor-core kernels, and ``check_device()`` says, kernel by kernel, whether this device can launch them.

Reference: CudaDeviceLimits (src/Idrak.Gpu/Cuda/CudaDeviceLimits.cs: block size, shared-memory budget and the tile
shapes chosen from what the device reports).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import asdict, dataclass
from typing import Dict, List

_NAMES = ("sms", "max_threads_per_block", "shared_memory_per_block_optin", "shared_memory_per_sm", "l2_bytes",
          "registers_per_sm", "max_blocks_per_sm", "max_threads_per_sm", "warp_size", "memory_bus_bits",
          "memory_clock_khz", "sm_clock_khz", "compute_major", "compute_minor", "max_cluster_size",
          "tensor_memory_columns")

# the device the kernels were written for (used when no GPU is present)
_B200 = (148, 1024, 232448, 233472, 132120576, 65536, 32, 2048, 32, 8192, 3996000, 1965000, 10, 0, 8, 512)


@dataclass(frozen=True)
class DeviceLimits:
    sms: int
    max_threads_per_block: int
    shared_memory_per_block_optin: int
    shared_memory_per_sm: int
    l2_bytes: int
    registers_per_sm: int
    max_blocks_per_sm: int
    max_threads_per_sm: int
    warp_size: int
    memory_bus_bits: int
    memory_clock_khz: int
    sm_clock_khz: int
    compute_major: int
    compute_minor: int
    max_cluster_size: int
    tensor_memory_columns: int
    measured: bool = True

    @property
    def peak_memory_gbs(self) -> float:
        """Bus width x data rate (double data rate), the nominal figure."""
        return self.memory_bus_bits / 8 * self.memory_clock_khz * 2 / 1e6

    def blocks_for(self, threads: int, shared_bytes: int, registers_per_thread: int = 0) -> int:
        """How many blocks of this shape are resident on one SM (0: the block cannot launch)."""
        if threads > self.max_threads_per_block or shared_bytes > self.shared_memory_per_block_optin:
            return 0
        by_threads = self.max_threads_per_sm // max(threads, 1)
        by_shared = self.shared_memory_per_sm // max(shared_bytes + 1024, 1) if shared_bytes else self.max_blocks_per_sm
        by_regs = self.registers_per_sm // max(registers_per_thread * threads, 1) if registers_per_thread else self.max_blocks_per_sm
        return max(0, min(by_threads, by_shared, by_regs, self.max_blocks_per_sm))

    def as_dict(self) -> dict:
        return asdict(self)


def device_limits() -> DeviceLimits:
    import torch
    if torch.cuda.is_available():
        from .. import _native
        buf = (C.c_longlong * 16)()
        n = _native.lib().idrak_device_limits(buf, 16)
        if n == 16:
            return DeviceLimits(*[int(v) for v in buf], measured=True)
        raise RuntimeError(f"idrak_device_limits failed ({n})")
    return DeviceLimits(*_B200, measured=False)


@dataclass(frozen=True)
class KernelShape:
    kernel: str
    tile: str                 # rows x columns x K per stage (or what the kernel's unit of work is)
    stages: int
    threads: int
    shared_bytes: int         # dynamic shared memory asked for at launch (the flash and packed kernels: rounded up)
    tensor_memory_columns: int
    blocks_per_sm: int
    note: str = ""


def kernel_shapes() -> List[KernelShape]:
    """The compile-time shapes of the tensor-core kernels (``csrc/*.cu``)."""
    return [
        KernelShape("gemm_kernel<256>", "128 x 256 x 64", 4, 320, 4 * 49152 + 32768 + 256 + 1024, 512, 1,
                    "two accumulators of 256 columns ping-pong between the MMA warp and eight epilogue warps"),
        KernelShape("gemm_kernel<128>", "128 x 128 x 64", 6, 320, 6 * 32768 + 32768 + 256 + 1024, 256, 1, "N <= 128"),
        KernelShape("gemm_pair_kernel", "256 x 256 x 64 over two SMs", 4, 320, 4 * 49152 + 32768 + 256 + 1024, 512, 1,
                    "cta_group::2: each CTA holds half of the A rows and half of the B columns"),
        KernelShape("skinny_gemm_kernel", "128 features x (16 | 32 | 64) tokens x 64, K over a cluster of up to 8", 4, 192,
                    98304, 64, 2, "partial tiles summed through distributed shared memory"),
        KernelShape("flash_fwd_kernel<64>", "128 queries x 128 keys, head size 64", 2, 320, 100 * 1024, 256, 2, ""),
        KernelShape("flash_fwd_kernel<128>", "128 queries x 128 keys, head size 128", 2, 320, 197 * 1024, 512, 1, ""),
        KernelShape("flash_bwd_q_kernel<64>", "128 queries x 128 keys per block, persistent", 3, 320, 160 * 1024, 320, 1, ""),
        KernelShape("flash_bwd_kv_kernel<64>", "128 keys x 128 queries per block, persistent", 2, 320, 232192, 384, 1, ""),
        KernelShape("qgemm_kernel", "128 x 128 x 64, weights unpacked in shared memory", 4, 448, 4 * 32768 + 2048, 256, 1,
                    "eight unpacking warps"),
        KernelShape("tp_gemm_kernel", "128 x 256 x 64 with peer-memory gather / reduce-scatter", 4, 320,
                    4 * 49152 + 16384 + 1024, 512, 1, ""),
    ]


def check_device(limits: DeviceLimits | None = None) -> Dict[str, str]:
    """Kernel -> "ok" or the limit that stops it on this device."""
    lim = limits or device_limits()
    out = {}
    for k in kernel_shapes():
        if lim.compute_major != 10:
            out[k.kernel] = f"needs compute capability 10.x (tcgen05); this device is {lim.compute_major}.{lim.compute_minor}"
        elif k.shared_bytes > lim.shared_memory_per_block_optin:
            out[k.kernel] = f"needs {k.shared_bytes} bytes of shared memory per block; the device allows {lim.shared_memory_per_block_optin}"
        elif k.tensor_memory_columns * k.blocks_per_sm > lim.tensor_memory_columns:
            out[k.kernel] = f"needs {k.tensor_memory_columns * k.blocks_per_sm} tensor-memory columns per SM; the device has {lim.tensor_memory_columns}"
        elif k.threads > lim.max_threads_per_block:
            out[k.kernel] = f"needs {k.threads} threads per block"
        else:
            out[k.kernel] = "ok"
    return out
