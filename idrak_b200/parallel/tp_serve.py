"""Tensor-parallel serving: a decoder split by layer over the ranks of one NVSwitch domain.

Each rank holds a slice of every block - its share of the query and key/value heads (the packed QKV projection is
column-parallel), the matching columns of the output projection (row-parallel), its share of the feed-forward width
(gate / up column-parallel, down row-parallel) - and a slice of the vocabulary rows of the head. Norm weights and the
token embedding are replicated. A rank runs the ordinary kernels over its heads and its paged KV cache; the only
communication is after the two row-parallel products of a block, where ``TPServeContext.all_reduce_rows`` sums the
ranks' partial rows inside one kernel over NVLink peer memory, adds the residual and (when asked) applies the next
norm, and after the head, where greedy sampling merges per-rank arg-maxima (``argmax``) and any other sampler sees
the gathered logits (``gather_logits``).

The reference has no tensor parallelism (its serving runs one model copy per device, ChatEngineModel.cs:95-99); this
is the layer split the 8 B / 8 GPU serving configuration asks for, built on the same ``ModelRunner`` contract.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native
from ..models.decoder import Decoder, FeedForward, build_decoder
from ..models.spec import DecoderSpec
from .comm import Communicator

# flag channels of the communicator that no other collective uses: 1 for the row all-reduce, 2 and 3 for the arg-max merge
CH_TP_ROWS, CH_TP_ARGMAX = 1, 2

_BOUND = False


def _bind():
    global _BOUND
    if _BOUND:
        return
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    pp = C.POINTER(C.c_void_p)
    _native.bind("idrak_tp_allreduce_rows", i, [vp, pp, i, i, vp, vp, vp, vp, vp, f, i, i, vp, vp, vp])
    _native.bind("idrak_tp_argmax", i, [vp, vp, i, i, i, i, vp, vp, i, vp, vp])
    _BOUND = True


# --------------------------------------------------------------------------- sharding a decoder
def check_shardable(spec: DecoderSpec, world: int) -> None:
    problems = []
    if spec.heads % world or spec.kv_heads % world:
        problems.append(f"heads {spec.heads} / kv heads {spec.kv_heads} do not divide by {world}")
    if spec.ff_dim % (world * 8):
        problems.append(f"feed-forward width {spec.ff_dim} does not divide by {world} x 8")
    if spec.padded_vocabulary % (world * 8):
        problems.append(f"padded vocabulary {spec.padded_vocabulary} does not divide by {world} x 8")
    if spec.experts:
        problems.append("mixture-of-experts layers are not split")
    if spec.parallel_blocks or spec.post_norms:
        problems.append("only plain pre-norm blocks are split (no parallel blocks, no post-norms)")
    if problems:
        raise ValueError("this decoder cannot be served tensor-parallel over %d ranks: %s" % (world, "; ".join(problems)))


def local_spec(spec: DecoderSpec, world: int) -> DecoderSpec:
    """The spec of one rank's slice: its heads and its share of the feed-forward width; ``dim``, ``head_dim``, the
    vocabulary (the embedding is replicated) and everything else unchanged."""
    check_shardable(spec, world)
    return dataclasses.replace(spec, heads=spec.heads // world, kv_heads=spec.kv_heads // world,
                               ff_dim=spec.ff_dim // world)


def vocab_slice(spec: DecoderSpec, rank: int, world: int) -> Tuple[int, int]:
    per = spec.padded_vocabulary // world
    return rank * per, (rank + 1) * per


@torch.no_grad()
def shard_decoder(full: Decoder, rank: int, world: int) -> Decoder:
    """Rank ``rank``'s slice of ``full`` as a decoder of ``local_spec``: same module tree, narrower projections. Biases
    of row-parallel products (output projection, down projection) stay on rank 0 only, since the partial products
    are summed. The head becomes ``local.head`` = this rank's rows of the (padded) vocabulary."""
    spec = full.spec
    ls = local_spec(spec, world)
    p0 = next(full.parameters())
    with torch.device(p0.device):
        prev = torch.get_default_dtype()
        torch.set_default_dtype(p0.dtype if p0.dtype.is_floating_point else prev)
        try:
            local = build_decoder(ls)
        finally:
            torch.set_default_dtype(prev)
    local = local.to(p0.device, p0.dtype)
    H, Hkv, D = spec.heads, spec.kv_heads, spec.head_dim
    Hl, Hkvl = ls.heads, ls.kv_heads
    ff, ffl = spec.ff_dim, ls.ff_dim

    def qkv_rows(t):
        q = t[rank * Hl * D:(rank + 1) * Hl * D]
        k = t[H * D + rank * Hkvl * D: H * D + (rank + 1) * Hkvl * D]
        v = t[(H + Hkv) * D + rank * Hkvl * D: (H + Hkv) * D + (rank + 1) * Hkvl * D]
        return torch.cat([q, k, v], 0)

    local.embed.copy_(full.embed)
    if full.pos is not None:
        local.pos.copy_(full.pos)
    local.norm.load_state_dict(full.norm.state_dict())
    for fb, lb in zip(full.blocks, local.blocks):
        lb.attn_norm.load_state_dict(fb.attn_norm.state_dict())
        lb.mlp_norm.load_state_dict(fb.mlp_norm.state_dict())
        if spec.qk_norm:
            lb.attn.q_norm.load_state_dict(fb.attn.q_norm.state_dict())
            lb.attn.k_norm.load_state_dict(fb.attn.k_norm.state_dict())
        lb.attn.qkv_weight.copy_(qkv_rows(fb.attn.qkv_weight))
        if fb.attn.qkv_bias is not None:
            lb.attn.qkv_bias.copy_(qkv_rows(fb.attn.qkv_bias))
        lb.attn.o_weight.copy_(fb.attn.o_weight[:, rank * Hl * D:(rank + 1) * Hl * D])
        if fb.attn.o_bias is not None:
            lb.attn.o_bias.copy_(fb.attn.o_bias if rank == 0 else torch.zeros_like(fb.attn.o_bias))
        fm, lm = fb.mlp, lb.mlp
        assert isinstance(fm, FeedForward)
        if spec.gated:
            up = torch.cat([fm.up_weight[rank * ffl:(rank + 1) * ffl], fm.up_weight[ff + rank * ffl: ff + (rank + 1) * ffl]], 0)
            ub = None if fm.up_bias is None else torch.cat([fm.up_bias[rank * ffl:(rank + 1) * ffl],
                                                            fm.up_bias[ff + rank * ffl: ff + (rank + 1) * ffl]], 0)
        else:
            up = fm.up_weight[rank * ffl:(rank + 1) * ffl]
            ub = None if fm.up_bias is None else fm.up_bias[rank * ffl:(rank + 1) * ffl]
        lm.up_weight.copy_(up)
        if ub is not None:
            lm.up_bias.copy_(ub)
        lm.down_weight.copy_(fm.down_weight[:, rank * ffl:(rank + 1) * ffl])
        if fm.down_bias is not None:
            lm.down_bias.copy_(fm.down_bias if rank == 0 else torch.zeros_like(fm.down_bias))
    lo, hi = vocab_slice(spec, rank, world)
    head_rows = full.head_weight()[lo:hi]
    local.tp_head = torch.nn.Parameter(head_rows.detach().clone(), requires_grad=False)
    local.tp_head_bias = None if full.head_bias is None else torch.nn.Parameter(full.head_bias[lo:hi].detach().clone(),
                                                                               requires_grad=False)
    if local.head is not None:
        local.head = None                     # the full-vocabulary head of the local tree is not kept
    local.tp_full_spec = spec
    return local.eval()


@torch.no_grad()
def random_shard(spec: DecoderSpec, rank: int, world: int, device, dtype=torch.bfloat16, seed: int = 0) -> Decoder:
    """A rank's slice with random weights, built without ever holding the whole model (benchmarks of models that do
    not fit one GPU's memory budget comfortably). Replicated tensors use the same seed on every rank."""
    ls = local_spec(spec, world)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(device):
            local = build_decoder(ls)
    finally:
        torch.set_default_dtype(prev)
    local = local.to(device, dtype)
    g = torch.Generator(device=device).manual_seed(seed)           # replicated tensors: same values everywhere
    local.embed.copy_(torch.randn(local.embed.shape, generator=g, device=device, dtype=torch.float32).mul_(spec.init_std))
    lo, hi = vocab_slice(spec, rank, world)
    gl = torch.Generator(device=device).manual_seed(seed + 1 + rank)
    local.tp_head = torch.nn.Parameter(
        torch.randn(hi - lo, spec.dim, generator=gl, device=device, dtype=torch.float32).mul_(spec.init_std).to(dtype),
        requires_grad=False)
    local.tp_head_bias = None
    local.head = None
    local.tp_full_spec = spec
    return local.eval()


# --------------------------------------------------------------------------- the collectives of a serving step
class TPServeContext:
    """Symmetric buffers and call-site state of the serving collectives of one tensor-parallel group."""

    def __init__(self, comm: Communicator, dim: int, max_rows: int, max_prefill_rows: int = 0):
        _bind()
        self.comm, self.rank, self.world = comm, comm.rank, comm.world
        self.dim, self.max_rows = dim, max_rows
        dev = comm.device
        rows = max(max_rows, max_prefill_rows, 1)
        self._bufs = [comm.symmetric(rows * dim * 2) for _ in range(2)]
        self._views = [b.tensor(torch.bfloat16, rows * dim).view(rows, dim) for b in self._bufs]
        self._turn = 0
        self.rows_capacity = rows
        self._state = torch.zeros(8, dtype=torch.int32, device=dev)       # [0] rows seq, [1] rows counter, [2] argmax seq
        self._argmax_local = torch.zeros(2 * 512, dtype=torch.float32, device=dev)
        self._logit_buf = None
        dist.barrier(group=comm.group)

    def partial_buffer(self, rows: int) -> torch.Tensor:
        """The symmetric buffer the next ``all_reduce_rows`` will read: write this rank's partial rows here."""
        if rows > self.rows_capacity:
            raise ValueError(f"{rows} rows exceed the tensor-parallel buffers ({self.rows_capacity})")
        return self._views[self._turn][:rows]

    def all_reduce_rows(self, partial: torch.Tensor, residual: Optional[torch.Tensor] = None, norm=None):
        """``x = residual + sum over ranks(partial)``; with ``norm`` (a decoder ``Norm``) also ``norm(x)``.
        ``partial`` is ``[rows, dim]`` bf16; it is copied into the symmetric buffer unless it already is that buffer's
        view (``partial_buffer``). Returns ``(x, normed or None)``."""
        rows = partial.shape[0]
        view = self.partial_buffer(rows)
        if partial.data_ptr() != view.data_ptr():
            view.copy_(partial)
        from ..ops._util import stream_ptr
        out = torch.empty((rows, self.dim), dtype=torch.bfloat16, device=partial.device)
        normed = torch.empty_like(out) if norm is not None else None
        w = norm.effective_weight() if norm is not None else None
        b = getattr(norm, "bias", None) if norm is not None else None
        st = self._state
        rc = _native.lib().idrak_tp_allreduce_rows(
            self.comm.ctx, self._bufs[self._turn].ptr_array, rows, self.dim,
            residual.data_ptr() if residual is not None else None, out.data_ptr(),
            w.data_ptr() if w is not None else None, b.data_ptr() if b is not None else None,
            normed.data_ptr() if normed is not None else None, float(norm.eps) if norm is not None else 0.0,
            int(norm.kind != "layer") if norm is not None else 1, CH_TP_ROWS, st.data_ptr(), st.data_ptr() + 4,
            stream_ptr())
        _native.check(rc, "idrak_tp_allreduce_rows")
        self._turn ^= 1
        return out, normed

    def argmax(self, logits_local: torch.Tensor, n_local: int, offset: int) -> torch.Tensor:
        """Greedy token per row over all ranks' vocabulary slices (ties to the lowest index); int32 ``[rows]``."""
        rows = logits_local.shape[0]
        if rows > 512:
            raise ValueError("at most 512 rows per merged arg-max")
        from ..ops._util import stream_ptr
        ids = torch.empty(rows, dtype=torch.int32, device=logits_local.device)
        rc = _native.lib().idrak_tp_argmax(self.comm.ctx, logits_local.data_ptr(), logits_local.stride(0), rows, n_local,
                                           offset, self._argmax_local.data_ptr(), ids.data_ptr(), CH_TP_ARGMAX,
                                           self._state.data_ptr() + 8, stream_ptr())
        _native.check(rc, "idrak_tp_argmax")
        return ids

    def gather_logits(self, logits_local: torch.Tensor) -> torch.Tensor:
        """All ranks' vocabulary slices side by side ``[rows, padded vocabulary]`` (for samplers that need the whole
        distribution); a peer-memory all-gather into a symmetric buffer."""
        rows, per = logits_local.shape
        need = rows * per * self.world * 2
        if self._logit_buf is None or self._logit_buf.nbytes < need:
            if self._logit_buf is not None:
                self._logit_buf.close()
            self._logit_buf = self.comm.symmetric(max(need, 1 << 20))
        # slices are laid out rank-major ([world, rows, per]); give the caller [rows, world * per]
        gathered = self.comm.all_gather(self._logit_buf, logits_local.contiguous().reshape(-1))
        return gathered.view(self.world, rows, per).permute(1, 0, 2).reshape(rows, self.world * per)

    def close(self):
        torch.cuda.synchronize()
        dist.barrier(group=self.comm.group)
        for b in self._bufs:
            b.close()
        if self._logit_buf is not None:
            self._logit_buf.close()
