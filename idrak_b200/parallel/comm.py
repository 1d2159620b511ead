"""Communicator over NVLink peer memory.

``Communicator`` owns the symmetric flag / slot areas of a process group and hands out
``SymmetricBuffer``s: device allocations of the same size on every rank, shared through CUDA IPC so a
kernel on one GPU can load from and store to every peer's copy. Collectives on symmetric buffers
(``all_reduce``, ``reduce_scatter``, ``all_gather``, ``broadcast``, ``barrier``, small-vector
``all_reduce_small``) run as this library's kernels (``algorithm='oneshot'|'twoshot'``); the same calls
with ``algorithm='nccl'`` go through ``torch.distributed`` and serve as baseline and oracle.

The control plane (exchange of IPC handles, group membership) is ``torch.distributed``: NCCL on GPUs,
gloo in CPU tests. On CPU tensors every collective is the gloo one, so the host-side logic above this
layer (bucket layouts, shard maps, header exchange, stop agreement) is testable without a GPU.

Reference: ITransport / ICollectives (src/Idrak.Abstraction/Cluster/Transports.cs:27, Collectives.cs:34-80),
NvlinkTransport (src/Idrak.Network/Transports/NvlinkTransport.cs:16-37), CudaBackend.Peers.cs:12-52.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .. import _native

# channel map of the flag area (two consecutive channels where a collective needs a second phase)
CH_BARRIER, CH_NORM, CH_STEP_DONE, CH_ONESHOT, CH_RS, CH_AG, CH_AR, CH_BCAST, CH_BUCKET0 = 0, 4, 6, 8, 10, 12, 14, 16, 20

_c_void_p, _c_int, _c_ll, _c_float = C.c_void_p, C.c_int, C.c_longlong, C.c_float
_PP = C.POINTER(C.c_void_p)
_BOUND = False


def _bind():
    global _BOUND
    if _BOUND:
        return
    b = _native.bind
    b("idrak_symm_alloc", _c_int, [_PP, _c_ll])
    b("idrak_symm_free", _c_int, [_c_void_p])
    b("idrak_ipc_handle_bytes", _c_int, [])
    b("idrak_ipc_get_handle", _c_int, [_c_void_p, _c_void_p])
    b("idrak_ipc_open", _c_int, [_c_void_p, _PP])
    b("idrak_ipc_close", _c_int, [_c_void_p])
    b("idrak_comm_ctx_bytes", _c_int, [])
    b("idrak_comm_max_ranks", _c_int, [])
    b("idrak_comm_flag_channels", _c_int, [])
    b("idrak_comm_flag_bytes", _c_ll, [])
    b("idrak_comm_ctx_init", None, [_c_void_p, _c_int, _c_int, _PP, _PP, _c_int, _c_void_p, _c_void_p])
    b("idrak_comm_bump_epoch", _c_int, [_c_void_p, _c_void_p])
    b("idrak_comm_barrier", _c_int, [_c_void_p, _c_int, _c_void_p])
    b("idrak_comm_wait", _c_int, [_c_void_p, _c_int, C.c_uint, _c_void_p])
    b("idrak_allreduce_oneshot", _c_int, [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    b("idrak_reduce_scatter", _c_int, [_c_void_p, _PP, _c_void_p, _c_ll, _c_int, _c_int, _c_float, _c_int, _c_int,
                                       _c_void_p])
    b("idrak_all_gather", _c_int, [_c_void_p, _PP, _c_void_p, _c_ll, _c_int, _c_int, _c_void_p])
    b("idrak_allreduce_twoshot", _c_int, [_c_void_p, _PP, _c_ll, _c_int, _c_float, _c_int, _c_int, _c_void_p])
    b("idrak_broadcast", _c_int, [_c_void_p, _PP, _c_ll, _c_int, _c_int, _c_int, _c_void_p])
    b("idrak_dp_reduce_scatter", _c_int, [_c_void_p, _PP, _c_ll, _c_ll, _c_ll, _c_void_p, _c_void_p, _c_void_p,
                                          _c_int, _c_int, _c_void_p])
    b("idrak_dp_norm_exchange", _c_int, [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p])
    b("idrak_dp_adamw_allgather", _c_int, [_c_void_p, _PP, _c_ll, _c_ll, _c_ll, _c_void_p, _c_void_p, _c_void_p,
                                           _c_void_p, _c_void_p, _c_void_p, _c_float, _c_int, _c_int, _c_int,
                                           _c_void_p])
    _BOUND = True


class _RawDeviceMemory:
    """Exposes a raw device pointer to PyTorch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of the communicator, peer-mapped into this process."""

    GUARD = 256              # bytes of canary before and after the usable range
    PATTERN = 0xA5

    def __init__(self, comm: "Communicator", nbytes: int, name: str = ""):
        _bind()
        lib = _native.lib()
        self.comm, self.nbytes, self.name = comm, int(nbytes), name or f"buffer{len(comm._buffers)}"
        base = C.c_void_p()
        total = self.nbytes + 2 * self.GUARD
        _native.check(lib.idrak_symm_alloc(C.byref(base), total), "idrak_symm_alloc")
        self._base = base.value
        # guard bands around the usable range: a kernel (this rank's or a peer's) that runs past either end of the
        # buffer lands here, and check_canaries() names the buffer instead of the damage showing up elsewhere
        self._whole = torch.as_tensor(_RawDeviceMemory(self._base, total), device=comm.device)
        self._whole[: self.GUARD].fill_(self.PATTERN)
        self._whole[self.GUARD + self.nbytes:].fill_(self.PATTERN)
        self.local_ptr = self._base + self.GUARD
        hb = lib.idrak_ipc_handle_bytes()
        handle = (C.c_ubyte * hb)()
        _native.check(lib.idrak_ipc_get_handle(base, handle), "idrak_ipc_get_handle")
        handles: list = [None] * comm.world
        dist.all_gather_object(handles, bytes(handle), group=comm.group)
        self.peer_ptrs = []
        self._opened = []
        for r in range(comm.world):
            if r == comm.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            out = C.c_void_p()
            buf = (C.c_ubyte * hb).from_buffer_copy(handles[r])
            _native.check(lib.idrak_ipc_open(buf, C.byref(out)), f"idrak_ipc_open(rank {r})")
            self.peer_ptrs.append(out.value + self.GUARD)
            self._opened.append(out.value)
        self.ptr_array = (C.c_void_p * comm.world)(*self.peer_ptrs)
        self._holder = _RawDeviceMemory(self.local_ptr, self.nbytes)
        self.bytes_tensor = torch.as_tensor(self._holder, device=comm.device)
        comm._buffers.append(self)

    def canaries_intact(self) -> bool:
        """Whether both guard bands still hold the pattern (one small device read)."""
        if not self._base:
            return True
        g = self.GUARD
        lo, hi = self._whole[:g], self._whole[g + self.nbytes:]
        return bool(((lo == self.PATTERN).all() & (hi == self.PATTERN).all()).item())

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        """A typed view of the local copy."""
        item = torch.empty((), dtype=dtype).element_size()
        numel = (self.nbytes - offset_bytes) // item if numel is None else numel
        return self.bytes_tensor[offset_bytes: offset_bytes + numel * item].view(dtype)

    def close(self):
        lib = _native.lib()
        for p in self._opened:
            lib.idrak_ipc_close(C.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            self.bytes_tensor = None
            self._whole = None
            lib.idrak_symm_free(C.c_void_p(self._base))
            self.local_ptr = self._base = 0
        if self in self.comm._buffers:
            self.comm._buffers.remove(self)


class Communicator:
    """Peer-memory communicator of one process group (at most 8 ranks on one NVSwitch domain)."""

    SLOT_FLOATS = 1024

    def __init__(self, group=None, device: Optional[torch.device] = None):
        assert dist.is_initialized(), "torch.distributed must be initialised (env://)"
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.native = self.device.type == "cuda"
        self._closed = False
        self._buffers: list = []
        # per-collective call and byte counters of this rank: name -> [calls, bytes sent to peers, bytes read from peers]
        self.traffic: dict = {}
        if not self.native:
            return
        _bind()
        lib = _native.lib()
        if self.world > lib.idrak_comm_max_ranks():
            raise ValueError(f"peer-memory communicator supports up to {lib.idrak_comm_max_ranks()} ranks")
        self.flags = SymmetricBuffer(self, lib.idrak_comm_flag_bytes(), "flags")
        self.slots = SymmetricBuffer(self, lib.idrak_comm_max_ranks() * self.SLOT_FLOATS * 4, "slots")
        self.local = torch.zeros(1 + lib.idrak_comm_flag_channels(), dtype=torch.int32, device=self.device)
        self.ctx = (C.c_ubyte * lib.idrak_comm_ctx_bytes())()
        lib.idrak_comm_ctx_init(self.ctx, self.rank, self.world, self.flags.ptr_array, self.slots.ptr_array,
                                self.SLOT_FLOATS, self.local.data_ptr(), self.local.data_ptr() + 4)
        dist.barrier(group=self.group)
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ helpers
    def _s(self):
        from ..ops._util import stream_ptr
        return stream_ptr()

    def symmetric(self, nbytes: int, name: str = "") -> SymmetricBuffer:
        return SymmetricBuffer(self, (int(nbytes) + 255) // 256 * 256, name)

    def _count(self, what: str, sent: float, read: float) -> None:
        c = self.traffic.setdefault(what, [0, 0, 0])
        c[0] += 1
        c[1] += int(sent)
        c[2] += int(read)

    def check_canaries(self) -> None:
        """Raises when a guard band of any symmetric buffer of this rank was written (something ran past an end)."""
        bad = [b.name for b in self._buffers if not b.canaries_intact()]
        if bad:
            raise RuntimeError(f"rank {self.rank}: guard bytes of symmetric buffer(s) {', '.join(bad)} were overwritten")

    def network_summary(self, gather: bool = False):
        """This rank's collectives so far: calls, bytes stored into peers' memory, bytes loaded from it. ``gather=True``
        collects every rank's summary (a collective call) - one row per rank, e.g. for an end-of-run report."""
        mine = {"rank": self.rank, "collectives": {k: {"calls": v[0], "bytes_sent": v[1], "bytes_read": v[2]}
                                                   for k, v in sorted(self.traffic.items())},
                "bytes_sent": sum(v[1] for v in self.traffic.values()),
                "bytes_read": sum(v[2] for v in self.traffic.values())}
        if not gather:
            return mine
        rows = [None] * self.world
        dist.all_gather_object(rows, mine, group=self.group)
        return rows

    def bump_epoch(self):
        """Advance the epoch every collective of this step will publish. Call once per step on the stream
        that orders the step's work, identically on every rank."""
        _native.check(_native.lib().idrak_comm_bump_epoch(self.ctx, self._s()), "bump_epoch")

    # ------------------------------------------------------------------ collectives on symmetric buffers
    def barrier(self):
        if not self.native:
            return dist.barrier(group=self.group)
        self.bump_epoch()
        _native.check(_native.lib().idrak_comm_barrier(self.ctx, CH_BARRIER, self._s()), "barrier")

    def wait(self, channel: int, add: int = 0):
        """Wait (bounded) until every peer has published the current epoch (+add) on ``channel``."""
        _native.check(_native.lib().idrak_comm_wait(self.ctx, channel, add, self._s()), "wait")

    def all_reduce_small(self, values: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """All-reduce of a short fp32 vector (headers, norms, flags); identical bits on every rank."""
        if not self.native or not values.is_cuda:
            out = values.clone()
            dist.all_reduce(out, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM, group=self.group)
            return out
        v = values.float().contiguous()
        out = torch.empty_like(v)
        self._count("all_reduce_small", 0, (self.world - 1) * v.numel() * 4)
        self.bump_epoch()
        _native.check(_native.lib().idrak_allreduce_oneshot(self.ctx, v.data_ptr(), out.data_ptr(), v.numel(),
                                                            1 if op == "max" else 0, CH_ONESHOT, self._s()),
                      "allreduce_oneshot")
        return out

    def all_reduce(self, buf: SymmetricBuffer, dtype: torch.dtype, numel: int, scale: float = 1.0,
                   algorithm: str = "twoshot", max_blocks: int = 64):
        """In-place sum over ranks of the first ``numel`` elements of a symmetric buffer."""
        t = buf.tensor(dtype, numel)
        if algorithm == "nccl":
            dist.all_reduce(t, group=self.group)
            if scale != 1.0:
                t.mul_(scale)
            return t
        per = self.world * (8 if dtype == torch.bfloat16 else 4)
        assert numel % per == 0, f"numel must be a multiple of {per}"
        moved = (self.world - 1) / self.world * numel * t.element_size()
        self._count("all_reduce", moved, moved)           # reduce-scatter by loads, then all-gather by stores
        self.bump_epoch()
        _native.check(_native.lib().idrak_allreduce_twoshot(self.ctx, buf.ptr_array, numel,
                                                            1 if dtype == torch.bfloat16 else 0, float(scale), CH_AR,
                                                            max_blocks, self._s()), "allreduce_twoshot")
        return t

    def reduce_scatter(self, buf: SymmetricBuffer, dtype: torch.dtype, numel: int, out: torch.Tensor,
                       scale: float = 1.0, algorithm: str = "peer", max_blocks: int = 64):
        """``out`` (numel / world elements) = this rank's slice of the sum over ranks."""
        if algorithm == "nccl":
            t = buf.tensor(dtype, numel)
            tmp = torch.empty(numel // self.world, dtype=dtype, device=t.device)
            dist.reduce_scatter_tensor(tmp, t, group=self.group)
            out.copy_(tmp.float() * scale if out.dtype == torch.float32 else tmp * scale)
            return out
        self._count("reduce_scatter", 0, (self.world - 1) / self.world * numel * (2 if dtype == torch.bfloat16 else 4))
        self.bump_epoch()
        _native.check(_native.lib().idrak_reduce_scatter(self.ctx, buf.ptr_array, out.data_ptr(), numel,
                                                         1 if dtype == torch.bfloat16 else 0,
                                                         1 if out.dtype == torch.float32 else 0, float(scale), CH_RS,
                                                         max_blocks, self._s()), "reduce_scatter")
        return out

    def all_gather(self, buf: SymmetricBuffer, local_slice: torch.Tensor, algorithm: str = "peer",
                   max_blocks: int = 64):
        """Store ``local_slice`` as slice ``rank`` of every rank's ``buf``; on return ``buf`` holds all slices.
        A rank's stores wait until every peer has entered its own call (in stream order after whatever still read
        the buffer's earlier contents), so back-to-back gathers into one buffer need no barrier between them."""
        nbytes = local_slice.numel() * local_slice.element_size()
        if algorithm == "nccl":
            t = buf.tensor(local_slice.dtype, local_slice.numel() * self.world)
            dist.all_gather_into_tensor(t, local_slice.contiguous(), group=self.group)
            return t
        self._count("all_gather", (self.world - 1) * nbytes, 0)
        self.bump_epoch()
        _native.check(_native.lib().idrak_all_gather(self.ctx, buf.ptr_array, local_slice.data_ptr(), nbytes, CH_AG,
                                                     max_blocks, self._s()), "all_gather")
        return buf.tensor(local_slice.dtype, local_slice.numel() * self.world)

    def broadcast(self, buf: SymmetricBuffer, nbytes: int, root: int = 0, algorithm: str = "peer",
                  max_blocks: int = 64):
        if algorithm == "nccl":
            dist.broadcast(buf.tensor(torch.uint8, nbytes), src=dist.get_global_rank(self.group, root)
                           if self.group is not None else root, group=self.group)
            return
        self._count("broadcast", (self.world - 1) * nbytes if self.rank == root else 0, 0)
        self.bump_epoch()
        _native.check(_native.lib().idrak_broadcast(self.ctx, buf.ptr_array, (nbytes + 15) // 16 * 16, root, CH_BCAST,
                                                    max_blocks, self._s()), "broadcast")

    def close(self):
        if self._closed or not self.native:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        problem = None
        try:
            self.check_canaries()
        except RuntimeError as e:
            problem = e
        self.flags.close()
        self.slots.close()
        self._closed = True
        if problem is not None:
            raise problem
