"""The allocation-free column-sum entry point, called through its exported C symbol.

Collected last on purpose: the scratch array it uses lives in the library's device image and is shared by every
call, so the test also shows that it works after everything else in the suite has run on the device.
"""
import ctypes as C

import pytest
import torch

from idrak_b200 import _native
from idrak_b200.ops import colsum

pytestmark = pytest.mark.gpu


def _entry():
    lib = C.CDLL(str(_native.lib_path()))
    fn = lib.idrak_colsum_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.idrak_colsum_static_error.restype = C.c_char_p
    lib.idrak_colsum_static_max_floats.restype = C.c_longlong
    return lib, fn


def _call(fn, x, out, accumulate=False):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), out.data_ptr(), int(out.dtype == torch.float32),
              int(accumulate), stream)


def test_static_colsum_matches_the_workspace_entry_point_twice_in_a_row():
    lib, fn = _entry()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(11)
    first = True
    for rows, cols, ld, out_dtype in ((4096, 768, 768, torch.float32), (1000, 3072, 3072, torch.bfloat16),
                                      (333, 130, 136, torch.float32), (77, 50, 51, torch.float32)):
        x = torch.randn(rows, ld, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)[:, :cols]
        want = colsum(x, torch.empty(cols, dtype=out_dtype, device=dev))
        exact = x.float().sum(0)
        out = torch.full((cols,), 7.0, dtype=out_dtype, device=dev)
        if first:               # the first call on a device does the one-time set-up; make it outside the measurement
            assert _call(fn, x, out) == 0, lib.idrak_colsum_static_error().decode()
            first = False
        torch.cuda.synchronize()
        held = torch.cuda.memory_allocated(dev)
        for _ in range(2):      # two calls in a row share the scratch array, one after the other on one stream
            out.fill_(7.0)
            assert _call(fn, x, out) == 0, lib.idrak_colsum_static_error().decode()
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated(dev) == held
            tol = 2e-2 * max(1.0, rows ** 0.5) if out_dtype == torch.bfloat16 else 1e-3 * max(1.0, rows ** 0.5)
            # same partial sums folded in the same order as the allocating entry point: the same bits
            assert torch.equal(out, want), (rows, cols, out_dtype)
            torch.testing.assert_close(out.float(), exact, rtol=1e-2, atol=tol)
        if out_dtype == torch.float32:
            base = out.clone()
            assert _call(fn, x, out, accumulate=True) == 0
            torch.testing.assert_close(out, 2 * base, rtol=1e-5, atol=tol)
    _native.check_status()


def test_static_colsum_refuses_what_does_not_fit():
    lib, fn = _entry()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    cap = lib.idrak_colsum_static_max_floats()
    assert cap == 1 << 20
    rows, cols = 64 * 128, 8192 + 8                       # 128 row chunks x 8200 columns > capacity
    x = torch.zeros(rows, cols, dtype=torch.bfloat16, device=dev)
    out = torch.full((cols,), 3.0, dtype=torch.float32, device=dev)
    assert _call(fn, x, out) == -3
    msg = lib.idrak_colsum_static_error().decode()
    assert "8200" in msg and str(cap) in msg and "idrak_colsum" in msg
    torch.cuda.synchronize()
    assert bool((out == 3.0).all())                       # nothing was launched
    # few rows make a wide matrix fit: 1 chunk x 20000 columns
    y = torch.ones(50, 20000, dtype=torch.bfloat16, device=dev)
    o = torch.empty(20000, dtype=torch.float32, device=dev)
    assert _call(fn, y, o) == 0
    torch.cuda.synchronize()
    assert bool((o == 50.0).all())
    assert fn(None, 4, 4, 4, o.data_ptr(), 1, 0, None) == -2 and b"bad argument" in lib.idrak_colsum_static_error()
