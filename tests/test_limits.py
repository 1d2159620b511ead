"""Device limits and the kernel shape table."""
import dataclasses

import pytest
import torch

from idrak_b200.runtime.limits import DeviceLimits, check_device, device_limits, kernel_shapes


def test_limits_without_a_gpu_are_the_design_figures():
    lim = device_limits()
    if not torch.cuda.is_available():
        assert not lim.measured and lim.sms == 148 and lim.tensor_memory_columns == 512
    assert lim.shared_memory_per_block_optin >= 200 * 1024 and lim.warp_size == 32
    assert 7000 < lim.peak_memory_gbs < 9000
    assert lim.blocks_for(320, 100 * 1024) == 2 and lim.blocks_for(320, 232192) == 1
    assert lim.blocks_for(2048, 0) == 0 and lim.blocks_for(256, 300 * 1024) == 0


def test_every_kernel_fits_the_design_device_and_small_devices_are_named():
    b200 = DeviceLimits(*device_limits().as_dict().values()) if not torch.cuda.is_available() else device_limits()
    assert all(v == "ok" for v in check_device(b200).values()), check_device(b200)
    assert len({k.kernel for k in kernel_shapes()}) == len(kernel_shapes())
    hopper = dataclasses.replace(b200, compute_major=9, tensor_memory_columns=0)
    assert all("compute capability 10" in v for v in check_device(hopper).values())
    small = dataclasses.replace(b200, shared_memory_per_block_optin=99 * 1024)
    verdicts = check_device(small)
    assert "shared memory" in verdicts["gemm_kernel<256>"] and verdicts["skinny_gemm_kernel"] == "ok"


@pytest.mark.gpu
def test_limits_read_from_the_device():
    lim = device_limits()
    props = torch.cuda.get_device_properties(0)
    assert lim.measured and lim.sms == props.multi_processor_count and lim.compute_major == props.major
    assert lim.l2_bytes == props.L2_cache_size and all(v == "ok" for v in check_device(lim).values())
