"""A device-side wait that nobody satisfies gives up after its budget, reports where it was, and leaves the context
usable: the flag is simply never set - nothing is made to fault or hang."""
import time

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_status_and_context_survives():
    from idrak_b200 import _native, ops
    from idrak_b200.parallel.comm import Communicator
    made = False
    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29779", rank=0, world_size=1)
        made = True
    try:
        torch.cuda.set_device(0)
        comm = Communicator(device=torch.device("cuda", 0))
        torch.cuda.synchronize()
        _native.take_status()
        t0 = time.monotonic()
        comm.wait(300, add=3)                    # waits for epoch + 3 on a channel no one ever publishes
        torch.cuda.synchronize()
        waited = time.monotonic() - t0
        code, where, block, extra = _native.take_status()
        assert code == 5 and (where >> 16) == 21 and ((where >> 4) & 0xFFF) == 300 and (where & 0xF) == 0
        assert 1.5 < waited < 10.0               # the two-second budget, not a hang
        comm.wait(301, add=1)
        torch.cuda.synchronize()
        with pytest.raises(_native.NativeError, match="status 5"):
            _native.check_status("second wait")
        # the context is intact: a GEMM right after gives the right numbers
        a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(192, 128, device="cuda", dtype=torch.bfloat16)
        torch.testing.assert_close(ops.gemm(a, b).float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-1)
        comm.close()
    finally:
        if made:
            dist.destroy_process_group()
