"""Tensor parallelism with sequence-sharded activations, on fused compute + collective kernels.

A decoder block under tensor parallelism keeps its activations sharded by rows (tokens) between layers. The two
kinds of linear layer then are

* column-parallel (QKV, MLP up): all-gather the rows, multiply by this rank's slice of the output columns -
  ``TensorParallel.ag_gemm`` runs both in one kernel (peer pushes overlapped with the tcgen05 tiles);
* row-parallel (attention output, MLP down): multiply by this rank's slice of the input columns, then
  reduce-scatter the partial sums back to rows - ``TensorParallel.gemm_rs``, again one kernel.

``column_parallel_linear`` / ``row_parallel_linear`` are the autograd functions built on them; their backward
passes use the mirrored kernel (the gradient of an all-gather is a reduce-scatter and vice versa).
``TensorParallel(mode="nccl")`` runs the same layers on NCCL collectives + the plain GEMM as the baseline, and
on CPU tensors (gloo) for tests.

The reference has no tensor parallelism; the layer semantics follow its Linear (src/Idrak/Layers/Linear.cs:165)
and the collectives contract (src/Idrak.Abstraction/Cluster/Collectives.cs:34-80).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native, ops
from ..ops._util import ptr, stream_ptr
from .comm import Communicator

_BOUND = False
_ACT = {None: 0, "none": 0, "gelu": 1}


def _bind():
    global _BOUND
    if _BOUND:
        return
    vp, i, ll = C.c_void_p, C.c_int, C.c_longlong
    pp = C.POINTER(C.c_void_p)
    b = _native.bind
    b("idrak_tp_counter_words", i, [i])
    b("idrak_tp_max_rows_per_rank", i, [])
    b("idrak_tp_ag_gemm", i, [vp, vp, i, pp, ll, vp, i, i, vp, i, i, i, i, vp, i, vp, i, vp, vp, i, i, vp, vp])
    b("idrak_tp_gemm_rs", i, [vp, vp, i, vp, i, i, pp, ll, vp, i, i, i, i, vp, vp, i, vp, vp, vp, vp])
    b("idrak_tp_release", i, [vp, vp, vp])
    _BOUND = True


class TensorParallel:
    """Buffers and sequence state of the fused tensor-parallel kernels for one process group.

    ``max_rows``: the largest total row count M (tokens across all ranks) of any layer call; ``max_in`` /
    ``max_out``: the largest gathered width K and reduced width N. The gather area holds two halves of
    ``max_rows x max_in`` bf16, the staging area two halves of ``max_rows x max_out``.
    """

    def __init__(self, comm: Optional[Communicator] = None, max_rows: int = 0, max_in: int = 0, max_out: int = 0,
                 mode: str = "fused", group=None, push_ctas: int = 16, multimem: bool = True):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.mode = mode
        self.push_ctas = push_ctas
        self.comm = comm
        if mode == "fused":
            _bind()
            assert comm is not None and comm.native, "the fused mode needs a peer-memory communicator on CUDA"
            lib = _native.lib()
            self.max_rows, self.max_in, self.max_out = max_rows, max_in, max_out
            self.gather_half = max_rows * max_in
            self.stage_half = max_rows * max_out
            self.gather_mc = self.stage_mc = None
            self._symm = []
            import os
            if multimem and self.world > 1 and os.environ.get("IDRAK_TP_MULTIMEM", "1") != "0":
                self._try_multicast_buffers(comm.device)
            if self.gather_mc is None:
                self.gather = comm.symmetric(2 * self.gather_half * 2)
                self.stage = comm.symmetric(2 * self.stage_half * 2)
                self.gather_ptrs, self.stage_ptrs = self.gather.ptr_array, self.stage.ptr_array
            words = lib.idrak_tp_counter_words(max_rows)
            self.state = torch.zeros(1 + words, dtype=torch.int32, device=comm.device)   # [0] = seq, then counters
            dist.barrier(group=group)
            torch.cuda.synchronize()

    def _try_multicast_buffers(self, device) -> None:
        """Gather / staging areas from PyTorch's symmetric memory, which also binds them to an NVSwitch multicast
        object: one ``multimem.st`` then reaches every rank and one ``multimem.ld_reduce`` sums every rank's copy.
        Falls back to plain peer-mapped buffers when the machine or the build has no multicast support."""
        try:
            import torch.distributed._symmetric_memory as symm
            group = self.group if self.group is not None else dist.group.WORLD
            handles = []
            for nbytes in (2 * self.gather_half * 2, 2 * self.stage_half * 2):
                t = symm.empty(int(nbytes), dtype=torch.uint8, device=device)
                h = symm.rendezvous(t, group)
                handles.append((t, h))
            ok = all(int(h.multicast_ptr) != 0 for _, h in handles)
            flag = torch.tensor([1 if ok else 0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            if int(flag.item()) == 0:
                return
            (gt, gh), (st, sh) = handles
            gt.zero_()
            st.zero_()
            self._symm = handles
            self.gather_ptrs = (C.c_void_p * self.world)(*[int(p) for p in gh.buffer_ptrs])
            self.stage_ptrs = (C.c_void_p * self.world)(*[int(p) for p in sh.buffer_ptrs])
            self.gather_mc, self.stage_mc = int(gh.multicast_ptr), int(sh.multicast_ptr)
        except Exception as e:              # no multicast on this machine / build: the peer-store path still works
            self.multicast_error = repr(e)
            self.gather_mc = self.stage_mc = None

    # ------------------------------------------------------------------ helpers
    def fusable(self, rows_total: int, k: int, n: int, reduce: bool) -> bool:
        if self.mode != "fused":
            return False
        if rows_total % (self.world * 128) or rows_total > self.max_rows or k % 8:
            return False
        if rows_total // self.world > _native.lib().idrak_tp_max_rows_per_rank():
            return False
        return (n % 64 == 0 and n <= self.max_out) if reduce else (k <= self.max_in and n % 8 == 0)

    def _seq_ptr(self):
        return self.state.data_ptr()

    def _counter_ptr(self):
        return self.state.data_ptr() + 4

    # ------------------------------------------------------------------ collectives (baseline / fallback)
    def all_gather_rows(self, x_local: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x_local
        out = torch.empty((x_local.shape[0] * self.world,) + tuple(x_local.shape[1:]), dtype=x_local.dtype,
                          device=x_local.device)
        dist.all_gather_into_tensor(out, x_local.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, full: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return full
        out = torch.empty((full.shape[0] // self.world,) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
        if full.is_cuda:
            dist.reduce_scatter_tensor(out, full.contiguous(), group=self.group)
        else:                                   # gloo has no reduce-scatter: all-reduce and keep this rank's rows
            tmp = full.clone()
            dist.all_reduce(tmp, group=self.group)
            r = out.shape[0]
            out.copy_(tmp[self.rank * r:(self.rank + 1) * r])
        return out

    # ------------------------------------------------------------------ fused ops
    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, w_mn: bool = False, bias: Optional[torch.Tensor] = None,
                act: Optional[str] = None):
        """``act(all_gather(x_local) @ op(w) + bias)``. ``w``: ``[N, K]`` (or stored ``[K, N]`` with ``w_mn``).
        Returns ``y`` (and the pre-activation when ``act`` is "gelu")."""
        rows, K = x_local.shape
        M = rows * self.world
        N = w.shape[1] if w_mn else w.shape[0]
        if not self.fusable(M, K, N, False):
            full = self.all_gather_rows(x_local)
            return ops.gemm(full, w, b_mn=w_mn, bias=bias, act=act)
        assert x_local.dtype == torch.bfloat16 and x_local.stride(1) == 1 and w.stride(1) == 1
        y = torch.empty(M, N, dtype=torch.bfloat16, device=x_local.device)
        aux = torch.empty_like(y) if act == "gelu" else None
        rc = _native.lib().idrak_tp_ag_gemm(
            self.comm.ctx, x_local.data_ptr(), x_local.stride(0), self.gather_ptrs, self.gather_half,
            w.data_ptr(), w.stride(0), int(w_mn), y.data_ptr(), y.stride(0), M, N, K, ptr(bias), _ACT[act], ptr(aux),
            aux.stride(0) if aux is not None else 0, self._seq_ptr(), self._counter_ptr(), self.push_ctas, 0,
            self.gather_mc, stream_ptr())
        _native.check(rc, "idrak_tp_ag_gemm")
        return (y, aux) if act == "gelu" else y

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, w_mn: bool = False, bias: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Rows of this rank of ``sum_ranks(x @ op(w)) + bias + residual``. ``x``: ``[M, K_local]``; ``residual``:
        this rank's rows ``[M / world, N]``."""
        M, K = x.shape
        N = w.shape[1] if w_mn else w.shape[0]
        if not self.fusable(M, K, N, True):
            part = ops.gemm(x, w, b_mn=w_mn)
            out = self.reduce_scatter_rows(part)
            if bias is not None:
                out = out + bias
            if residual is not None:
                out = out + residual
            return out
        assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
        out = torch.empty(M // self.world, N, dtype=torch.bfloat16, device=x.device)
        rc = _native.lib().idrak_tp_gemm_rs(
            self.comm.ctx, x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), int(w_mn), self.stage_ptrs,
            self.stage_half, out.data_ptr(), out.stride(0), M, N, K, ptr(bias), ptr(residual),
            residual.stride(0) if residual is not None else 0, self._seq_ptr(), self._counter_ptr(), self.stage_mc,
            stream_ptr())
        _native.check(rc, "idrak_tp_gemm_rs")
        return out
