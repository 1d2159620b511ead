import json

import pytest
import torch

from idrak_b200.diag.profiler import GpuProfiler, Profiler


def _work():
    a = torch.randn(128, 128)
    return torch.relu(a @ a).sum()


def test_profiler_reports_cold_warm_and_operators():
    rep = Profiler.run("toy", _work, cold=1, warm=3)
    assert len(rep.cold_ms) == 1 and len(rep.warm_ms) == 3 and rep.warm_median_ms > 0
    names = [r.name for r in rep.kernels]
    assert any("mm" in n for n in names) and abs(sum(r.share for r in rep.kernels) - 1.0) < 1e-6
    assert rep.kernels == sorted(rep.kernels, key=lambda r: -r.total_us)
    text = rep.table()
    assert "toy on" in text and "launches" in text
    assert rep.to_markdown().startswith("### toy") and "| kernel |" in rep.to_markdown()
    assert rep.to_csv().splitlines()[0] == "kernel,launches,total_us,mean_us,share,tflops"
    d = json.loads(rep.to_json())
    assert d["name"] == "toy" and len(d["kernels"]) == len(rep.kernels)
    with GpuProfiler(flops={"mm": 2.0 * 128 ** 3}) as gp:
        _work()
    mm = next(r for r in gp.rows() if "mm" in r.name)
    assert mm.launches >= 1 and mm.tflops is not None and mm.tflops > 0


@pytest.mark.gpu
def test_profiler_sees_this_librarys_kernels():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from idrak_b200.ops import gemm
    a = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16)
    rep = Profiler.run("gemm", lambda: gemm(a, b), flops={"gemm_kernel": 2.0 * 512 * 384 * 256})
    row = next(r for r in rep.kernels if "gemm_kernel" in r.name)
    assert row.launches == 1 and row.tflops > 0 and rep.warm_device_ms and rep.peak_memory_bytes > 0
