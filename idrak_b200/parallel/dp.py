"""Data-parallel training with the gradient reduction fused into the optimizer.

``DataParallel(model, ...)`` re-homes the model's parameters and gradients into flat buffers in symmetric
(peer-mapped) memory and splits the flat range into buckets in reverse parameter order. While the
backward pass runs, each bucket whose gradients are complete is handed to a side stream where one
kernel reads that bucket's slice from every peer over NVLink, sums in rank order (token-weighted when
ranks hold different token counts) and keeps the fp32 result as this rank's shard gradient. After the
last bucket a one-block kernel exchanges the squared norms, and the AdamW kernel updates the rank's
shard (fp32 master weights and moments live only on their owner: the reference's ``Shard=optimizer``)
while storing the new bf16 weights straight into every peer's parameter buffer. No NCCL call is on
this path; ``mode='nccl'`` is the baseline that all-reduces the same buckets with NCCL and steps a
replicated optimizer.

Reference: GradientReduction (src/Idrak.Network/Training/GradientReduction.cs:166-216,396-492,506-640),
BucketLayout (GradientBuckets.cs:19-110), sharded sync (Sharding.cs:229-338), the per-parameter
"gradient ready" hook (src/Idrak.Abstraction/Tensors/Autograd.cs:146-164).
"""
from __future__ import annotations

import contextlib
import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from ..ops.optim import (FusedAdamW, H_B1, H_B2, H_BC1, H_BC2, H_CLIP, H_COUNT, H_EPS, H_GSCALE, H_LR, H_MAXNORM,
                         H_NORM)
from .comm import CH_BUCKET0, CH_NORM, CH_STEP_DONE, Communicator
from .flat import ALIGN_ELEMS, FlatBuffers


class _ShardedAdamW:
    """Optimizer facade of the fused path: hyper-parameters, step count and the sharded state tensors."""

    def __init__(self, lr, betas, eps, weight_decay, max_grad_norm, device):
        self.lr, self.betas, self.eps = lr, betas, eps
        self.weight_decay, self.max_grad_norm = weight_decay, max_grad_norm
        self.step_count = 0
        self.grad_scale = 1.0
        self.zero_grad_in_step = False
        self._hyper_host = torch.zeros(16, H_COUNT, dtype=torch.float32).pin_memory()
        self._hyper_dev = torch.zeros(H_COUNT, dtype=torch.float32, device=device)
        self.master = self.m = self.v = None

    def set_lr(self, lr):
        self.lr = lr

    def _hyper_values(self):
        b1, b2 = self.betas
        return {H_LR: self.lr, H_B1: b1, H_B2: b2, H_EPS: self.eps, H_BC1: 1.0 - b1 ** self.step_count,
                H_BC2: 1.0 - b2 ** self.step_count, H_MAXNORM: self.max_grad_norm, H_GSCALE: self.grad_scale}

    def advance_for_replay(self):
        self.step_count += 1
        h = self._hyper_host[0]
        for k, v in self._hyper_values().items():
            h[k] = v

    def upload(self):
        slot = 0 if torch.cuda.is_current_stream_capturing() else 1 + self.step_count % 15
        h = self._hyper_host[slot]
        for k, v in self._hyper_values().items():
            h[k] = v
        self._hyper_dev[:H_CLIP].copy_(h[:H_CLIP], non_blocking=True)
        self._hyper_dev[H_MAXNORM:].copy_(h[H_MAXNORM:], non_blocking=True)

    def grad_norm(self) -> float:
        return float(self._hyper_dev[H_NORM].item())

    def zero_grad(self, set_to_none: bool = False):
        pass

    def state_dict(self):
        return {"step": torch.tensor(float(self.step_count)), "master": self.master.cpu(), "m": self.m.cpu(),
                "v": self.v.cpu()}

    def load_state_dict(self, state):
        self.step_count = int(float(state["step"]))
        self.master.copy_(state["master"])
        self.m.copy_(state["m"])
        self.v.copy_(state["v"])


def bucket_channels_fit(n_buckets: int, flag_channels: int) -> bool:
    """Whether ``n_buckets`` gradient buckets can each have their own flag channel (plus the one after it)."""
    return CH_BUCKET0 + n_buckets + 1 <= flag_channels


_HOOK_PROBE = None


def _hook_fires_without_gradient() -> bool:
    """Whether this PyTorch calls a parameter's post-accumulate-grad hook even when the backward function returned
    ``None`` for it (newer versions do). Where it does, the hook alone says "this parameter's gradient is final" -
    also for gradients a kernel wrote straight into ``.grad`` - and the direct-write notification must not be
    counted on top of it."""
    global _HOOK_PROBE
    if _HOOK_PROBE is None:
        class _Probe(torch.autograd.Function):
            @staticmethod
            def forward(ctx, x, w):
                return x * 2

            @staticmethod
            def backward(ctx, g):
                return g * 2, None

        w = torch.nn.Parameter(torch.ones(1))
        x = torch.ones(1, requires_grad=True)
        fired = []
        handle = w.register_post_accumulate_grad_hook(lambda _p: fired.append(1))
        _Probe.apply(x, w).sum().backward()
        handle.remove()
        _HOOK_PROBE = bool(fired)
    return _HOOK_PROBE


class DataParallel:
    def __init__(self, model: torch.nn.Module, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float = 1.0, mode: str = "fused", group=None,
                 bucket_mb: float = 32.0, comm: Optional[Communicator] = None, rs_blocks: int = 32,
                 broadcast_from_rank0: bool = True):
        assert mode in ("fused", "nccl")
        self.model, self.mode, self.group = model, mode, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        params = [p for p in model.parameters() if p.requires_grad]
        self.device = params[0].device
        self.rs_blocks = rs_blocks
        # the shard update and parameter all-gather run after the backward pass, with the machine to themselves:
        # two CTAs of 512 threads per SM (the reduce-scatter, which shares the SMs with backward, keeps rs_blocks)
        self.update_blocks = 2 * _native.lib().idrak_sm_count() if self.device.type == "cuda" else 2 * rs_blocks
        self._side = torch.cuda.Stream(device=self.device)
        self._handles = []
        self._pending = None
        if broadcast_from_rank0:
            for p in params:
                dist.broadcast(p.data, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        decay_ids = {id(p) for p in params if p.dim() >= 2}

        if mode == "nccl":
            self.flat = FlatBuffers(params)
            groups = [{"params": [p for p in params if id(p) in decay_ids], "weight_decay": weight_decay},
                      {"params": [p for p in params if id(p) not in decay_ids], "weight_decay": 0.0}]
            self.optimizer = FusedAdamW(groups, lr=lr, betas=betas, eps=eps, max_grad_norm=max_grad_norm)
            self.comm = None
        else:
            if self.world not in (1, 2, 4, 8):
                raise ValueError("fused data parallel needs a world size of 1, 2, 4 or 8")
            self.comm = comm or Communicator(group, self.device)
            self._sym = []

            def alloc(n, dt):
                buf = self.comm.symmetric(n * torch.empty((), dtype=dt).element_size())
                self._sym.append(buf)
                return buf.tensor(dt, n)

            self.flat = FlatBuffers(params, allocator=alloc, pad_to=ALIGN_ELEMS * self.world)
            self._param_buf, self._grad_buf = self._sym[0], self._sym[1]
            self.optimizer = _ShardedAdamW(lr, betas, eps, weight_decay, max_grad_norm, self.device)
        self._make_buckets(int(bucket_mb * 1024 * 1024 / 2))
        if mode == "fused":
            self._init_shard(decay_ids)
        self._install_hooks(params)
        dist.barrier(group=group)

    # ------------------------------------------------------------------ layout
    def _make_buckets(self, bucket_elems: int):
        self.buckets = self.flat.buckets(bucket_elems)          # (start, end, [param indices])
        if self.mode == "fused":
            # bucket b signals on flag channel CH_BUCKET0 + b (and the kernels use the channel after it for their
            # second phase): a layout with more buckets than channels would index past the peers' flag areas
            channels = _native.lib().idrak_comm_flag_channels()
            while not bucket_channels_fit(len(self.buckets), channels):
                bucket_elems *= 2
                self.buckets = self.flat.buckets(bucket_elems)
        self._bucket_of = {}
        for b, (_, _, members) in enumerate(self.buckets):
            for i in members:
                self._bucket_of[i] = b
        self._remaining = [len(m) for _, _, m in self.buckets]
        self._reported = {}
        self._launched = [False] * len(self.buckets)

    def _init_shard(self, decay_ids):
        W, r = self.world, self.rank
        offs, off = [], 0
        for (s, e, _) in self.buckets:
            assert (e - s) % (W * 8) == 0
            offs.append(off)
            off += (e - s) // W
        self.shard_offsets, self.shard_numel = offs, off
        dev = self.device
        opt = self.optimizer
        opt.master = torch.empty(off, dtype=torch.float32, device=dev)
        opt.m = torch.zeros(off, dtype=torch.float32, device=dev)
        opt.v = torch.zeros(off, dtype=torch.float32, device=dev)
        self.shard_grad = torch.zeros(off, dtype=torch.float32, device=dev)
        for b, (s, e, _) in enumerate(self.buckets):
            sl = (e - s) // W
            opt.master[offs[b]: offs[b] + sl].copy_(self.flat.param[s + r * sl: s + (r + 1) * sl].float())
        flags = torch.zeros(self.flat.numel // ALIGN_ELEMS, dtype=torch.uint8)
        for pc in self.flat.pieces:
            if id(self.flat.params[pc.index]) in decay_ids:
                flags[pc.offset // ALIGN_ELEMS: (pc.offset + pc.numel + ALIGN_ELEMS - 1) // ALIGN_ELEMS] = 1
        self.decay_flags = flags.to(dev)
        self.sumsq_partials = torch.zeros(len(self.buckets) * self.rs_blocks, dtype=torch.float32, device=dev)
        self.rank_weights = None

    def set_rank_weights(self, weights: Optional[torch.Tensor]):
        """Per-rank gradient weights (tokens_r / sum of tokens) for token-weighted averaging; None = 1/world."""
        self.rank_weights = None if weights is None else weights.to(self.device, torch.float32).contiguous()

    def step_header(self, tokens, loss=None, stop: bool = False, presence: Optional[torch.Tensor] = None) -> dict:
        """The header every rank contributes before a step's gradients are reduced, exchanged in one small
        all-reduce: this rank's token count, its loss times that count, a stop request and (optionally) one
        presence flag per parameter. It sets the token weights of the gradient reduction on the device
        (``tokens_r / sum of tokens``, so the reduced gradient is the token-weighted mean whatever the ranks' batch
        sizes) and returns device tensors: ``tokens`` (global), ``loss`` (token-weighted mean), ``stop`` (> 0 when any
        rank asked to stop at this step boundary) and ``presence`` (how many ranks hold a gradient for each
        parameter). Nothing is read back to the host here. Call it before ``reduce_and_step`` of the step it
        describes, identically on every rank.

        Reference: the gradient header of GradientReduction (src/Idrak.Network/Training/GradientReduction.cs:780-812)
        and the stop agreement it carries (AllReduceStopAgreement.cs)."""
        W, r, dev = self.world, self.rank, self.device
        n_pres = 0 if presence is None else int(presence.numel())
        v = torch.zeros(W + 2 + n_pres, dtype=torch.float32, device=dev)
        t = tokens if torch.is_tensor(tokens) else torch.tensor(float(tokens), device=dev)
        t = t.to(dev, torch.float32).reshape(())
        v[r] = t
        if loss is not None:
            v[W] = (loss if torch.is_tensor(loss) else torch.tensor(float(loss), device=dev)).to(dev, torch.float32).reshape(()) * t
        v[W + 1] = 1.0 if stop else 0.0
        if n_pres:
            v[W + 2:] = presence.to(dev, torch.float32).reshape(-1)
        if self.mode == "fused" and self.comm is not None and v.numel() <= self.comm.SLOT_FLOATS:
            total = self.comm.all_reduce_small(v)
        else:
            total = v.clone()
            dist.all_reduce(total, group=self.group)
        tokens_all = total[:W].sum()
        weights = total[:W] / tokens_all.clamp(min=1.0)
        if self.mode == "fused":
            self.rank_weights = weights.contiguous()
        else:
            self._nccl_weight = weights[r] * W          # scales this rank's gradients before the 1/W all-reduce mean
        return {"tokens": tokens_all, "loss": total[W] / tokens_all.clamp(min=1.0), "stop": total[W + 1],
                "presence": total[W + 2:] if n_pres else None, "weights": weights}

    # ------------------------------------------------------------------ hooks
    def _install_hooks(self, params):
        index_of = {id(p): i for i, p in enumerate(self.flat.params)}
        for p in params:
            i = index_of[id(p)]
            self._handles.append(p.register_post_accumulate_grad_hook(lambda _p, i=i: self._grad_ready(i)))
            if not _hook_fires_without_gradient():
                p._idrak_ready = (lambda i=i: self._grad_ready(i))     # called by direct gradient writes

    def _grad_ready(self, index: int):
        if not self._overlapping:
            return
        b = self._bucket_of[index]
        if index in self._reported:
            import os
            first = self._reported[index] if os.environ.get("IDRAK_DP_DEBUG") else ""
            raise RuntimeError(f"data parallel: parameter {index} reported its gradient ready twice in one backward "
                               f"pass; its bucket would be reduced before the last write{first}")
        import os
        if os.environ.get("IDRAK_DP_DEBUG"):
            import traceback
            self._reported[index] = "\nfirst report from:\n" + "".join(traceback.format_stack(limit=8))
        else:
            self._reported[index] = True
        self._remaining[b] -= 1
        if self._remaining[b] == 0:
            self._launch_bucket(b)

    _overlapping = False

    @contextlib.contextmanager
    def overlap(self):
        """Wrap ``loss.backward()``: buckets are reduced on a side stream as their gradients complete."""
        self._remaining = [len(m) for _, _, m in self.buckets]
        self._reported = {}
        self._launched = [False] * len(self.buckets)
        self._work = []
        if self.mode == "fused":
            self.comm.bump_epoch()
        self._overlapping = True
        try:
            yield
        finally:
            self._overlapping = False

    def _launch_bucket(self, b: int):
        if self._launched[b]:
            return
        self._launched[b] = True
        s, e, _ = self.buckets[b]
        main = torch.cuda.current_stream()
        if self.mode == "nccl":
            view = self.flat.grad[s:e]
            w = getattr(self, "_nccl_weight", None)
            if w is not None:
                view.mul_(w.to(view.dtype))
            view.div_(self.world)
            self._work.append(dist.all_reduce(view, group=self.group, async_op=True))
            return
        from ..ops._util import stream_ptr
        stream_ptr()                  # this may be a backward thread: bind the device context to it
        ev = torch.cuda.Event()
        ev.record(main)
        self._side.wait_event(ev)
        with torch.cuda.stream(self._side):
            lib = _native.lib()
            part =self.sumsq_partials[b * self.rs_blocks: (b + 1) * self.rs_blocks]
            rc = lib.idrak_dp_reduce_scatter(
                self.comm.ctx, self._grad_buf.ptr_array, s, e - s, self.shard_offsets[b], self.shard_grad.data_ptr(),
                part.data_ptr(), self.rank_weights.data_ptr() if self.rank_weights is not None else None,
                CH_BUCKET0 + b, self.rs_blocks, self._side.cuda_stream)
            _native.check(rc, "idrak_dp_reduce_scatter")

    # ------------------------------------------------------------------ the update
    @torch.no_grad()
    def reduce_and_step(self):
        for b in range(len(self.buckets)):          # buckets whose parameters saw no gradient this step
            self._launch_bucket(b)
        opt = self.optimizer
        if self.mode == "nccl":
            for w in self._work:
                w.wait()
            opt.step()
            return
        opt.step_count += 1
        main = torch.cuda.current_stream()
        lib = _native.lib()
        opt.upload()                                 # on the main stream, before the side stream reads it
        ev = torch.cuda.Event()
        ev.record(main)
        self._side.wait_event(ev)
        with torch.cuda.stream(self._side):
            s_ptr = self._side.cuda_stream
            rc = lib.idrak_dp_norm_exchange(self.comm.ctx, self.sumsq_partials.data_ptr(),
                                            self.sumsq_partials.numel(), opt._hyper_dev.data_ptr(), CH_NORM, s_ptr)
            _native.check(rc, "idrak_dp_norm_exchange")
            nb = len(self.buckets)
            for b, (s, e, _) in enumerate(self.buckets):
                rc = lib.idrak_dp_adamw_allgather(
                    self.comm.ctx, self._param_buf.ptr_array, s, e - s, self.shard_offsets[b],
                    self.shard_grad.data_ptr(), opt.master.data_ptr(), opt.m.data_ptr(), opt.v.data_ptr(),
                    self.decay_flags.data_ptr(), opt._hyper_dev.data_ptr(), float(opt.weight_decay), CH_STEP_DONE,
                    1 if b == nb - 1 else 0, self.update_blocks, s_ptr)
                _native.check(rc, "idrak_dp_adamw_allgather")
            # every peer's last update kernel has published "done": their stores into my parameters landed and
            # they no longer read my gradients
            _native.check(lib.idrak_comm_wait(self.comm.ctx, CH_STEP_DONE, 0, s_ptr), "comm_wait")
        done = torch.cuda.Event()
        done.record(self._side)
        main.wait_event(done)

    def zero_grad(self):
        self.flat.zero_grad()

    # ------------------------------------------------------------------ optimizer state, independent of the world size
    def _gather_shard(self, shard: torch.Tensor) -> torch.Tensor:
        """The full flat fp32 vector whose slices the ranks hold (joined in rank order per bucket)."""
        W = self.world
        parts = [torch.empty_like(shard) for _ in range(W)]
        dist.all_gather(parts, shard.contiguous(), group=self.group)
        full = torch.zeros(self.flat.numel, dtype=torch.float32, device=shard.device)
        for b, (s, e, _) in enumerate(self.buckets):
            sl = (e - s) // W
            for r in range(W):
                full[s + r * sl: s + (r + 1) * sl] = parts[r][self.shard_offsets[b]: self.shard_offsets[b] + sl]
        return full

    def optimizer_state(self) -> dict:
        """``step``, ``m.{i}``, ``v.{i}`` (and ``master.{i}``) by parameter index - the same entries a single-process
        AdamW writes, so a run can resume at another world size (collective: every rank must call it)."""
        if self.mode == "nccl":
            return self.optimizer.state_dict()
        opt = self.optimizer
        out = {"step": torch.tensor(float(opt.step_count))}
        for key, shard in (("m", opt.m), ("v", opt.v), ("master", opt.master)):
            full = self._gather_shard(shard)
            for pc in self.flat.pieces:
                p = self.flat.params[pc.index]
                out[f"{key}.{pc.index}"] = full[pc.offset: pc.offset + pc.numel].view(p.shape).cpu()
        return out

    def refresh_master_from_parameters(self) -> None:
        """After the parameters were overwritten in place (a checkpoint load): rebuild this rank's fp32 master shard."""
        if self.mode == "nccl":
            if hasattr(self.optimizer, "refresh_master"):
                self.optimizer.refresh_master()
            return
        W, r, opt = self.world, self.rank, self.optimizer
        for b, (s, e, _) in enumerate(self.buckets):
            sl = (e - s) // W
            opt.master[self.shard_offsets[b]: self.shard_offsets[b] + sl].copy_(
                self.flat.param[s + r * sl: s + (r + 1) * sl].float())

    def load_optimizer_state(self, state: dict) -> None:
        if self.mode == "nccl":
            self.optimizer.load_state_dict(state)
            return
        opt, W, r = self.optimizer, self.world, self.rank
        opt.step_count = int(float(state["step"]))
        for key, shard in (("m", opt.m), ("v", opt.v), ("master", opt.master)):
            if f"{key}.0" not in state:
                continue                       # e.g. a file without master weights: keep the ones made from the parameters
            full = torch.zeros(self.flat.numel, dtype=torch.float32, device=shard.device)
            for pc in self.flat.pieces:
                full[pc.offset: pc.offset + pc.numel] = state[f"{key}.{pc.index}"].reshape(-1).to(shard.device)
            for b, (s, e, _) in enumerate(self.buckets):
                sl = (e - s) // W
                shard[self.shard_offsets[b]: self.shard_offsets[b] + sl] = full[s + r * sl: s + (r + 1) * sl]

    def close(self):
        for h in self._handles:
            h.remove()
        self._handles = []
        if self.comm is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            for buf in getattr(self, "_sym", []):
                buf.close()
            self.comm.close()
            self.comm = None
