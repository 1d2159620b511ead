"""Fused tensor-parallel kernels (all-gather -> GEMM, GEMM -> reduce-scatter): one rank (the flag protocol and the
tile order run as they do with peers) and two ranks over NVLink, against fp32 PyTorch."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(out, nproc, port, rounds=3):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "tp_worker.py"), str(out),
           str(rounds)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return torch.load(out)


def _check(res, world, rounds):
    e = res["errors"]
    assert res["world"] == world and res["seq"] == 5 * rounds          # every fused op advanced the sequence
    assert e["ag"] < 0.06 and e["ag_gelu"] < 0.06 and e["ag_mn"] < 0.06, e
    assert e["rs"] < 0.08 and e["rs_mn"] < 0.08, e


@pytest.mark.gpu
def test_fused_tp_kernels_one_rank(tmp_path):
    _check(_run(tmp_path / "tp1.pt", 1, 29651), 1, 3)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fused_tp_kernels_two_ranks(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _check(_run(tmp_path / "tp2.pt", 2, 29652), 2, 3)
