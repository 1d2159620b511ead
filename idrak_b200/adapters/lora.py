"""LoRA and DoRA adapters over a frozen base, applied per projection of the decoder.

An adapter for a projection ``y = x W^T`` (``W`` is ``[out, in]``) holds ``A [rank, in]`` and
``B [out, rank]`` and adds ``scale * (x A^T) B^T`` with ``scale = alpha / rank`` (``alpha / sqrt(rank)``
with rsLoRA). DoRA additionally learns a magnitude per output unit and renormalises the combined
weight: ``W' = m * (W + scale * B A) / ||W + scale * B A||_row``.

The decoder keeps q, k, v (and gate, up) packed in one matrix; adapters stay per target (``q``, ``k``,
``v``, ``o``, ``gate``, ``up``, ``down``, ``head``) and write into the matching column slice of the packed
projection's output, so checkpoints exchange with PEFT target by target.

On the GPU the low-rank path runs on the tcgen05 GEMM: ``t = x A^T`` (N = rank, one 128-wide tile
column) then ``y[:, slice] += scale * t B^T`` accumulated in place into the base projection's output.

Reference: ILinearAdapter / LoraAdapter / DoraAdapter (src/Idrak.Abstraction/Modules/LinearAdapters.cs:31-241),
PretrainedModel.AddAdapters (src/Idrak/Models/PretrainedModel.cs:1199), the `_lr` fused GEMM family
(src/Idrak.Gpu/Cuda/PtxKernels.TensorCore.cs:118-126).
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
from torch import nn

from .. import ops
from ..ops.gemm import lowrank_linear, lowrank_supported
from ..models.decoder import Decoder, FeedForward, SelfAttention

DEFAULT_TARGETS = ("q", "k", "v", "o", "gate", "up", "down")


class LoraAdapter(nn.Module):
    def __init__(self, in_features: int, out_features: int, rank: int = 16, alpha: float = 32.0,
                 rslora: bool = False, dtype=None, device=None):
        super().__init__()
        self.rank, self.alpha, self.rslora = rank, alpha, rslora
        self.scale = alpha / math.sqrt(rank) if rslora else alpha / rank
        self.A = nn.Parameter(torch.empty(rank, in_features, dtype=dtype, device=device))
        self.B = nn.Parameter(torch.zeros(out_features, rank, dtype=dtype, device=device))
        nn.init.kaiming_uniform_(self.A, a=math.sqrt(5))

    def delta(self, x: torch.Tensor) -> torch.Tensor:
        """``scale * (x A^T) B^T``."""
        t = ops.linear(x, self.A)
        return ops.linear(t, self.B) * self.scale

    def delta_weight(self) -> torch.Tensor:
        """``scale * B A`` as an ``[out, in]`` matrix (fp32)."""
        return (self.B.float() @ self.A.float()) * self.scale

    def add_to(self, y_slice: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        return y_slice + self.delta(x)


class DoraAdapter(LoraAdapter):
    """Weight-decomposed low-rank adaptation: LoRA direction plus a learned magnitude per output unit."""

    def __init__(self, base_weight: torch.Tensor, rank: int = 16, alpha: float = 32.0, rslora: bool = False):
        out_features, in_features = base_weight.shape
        super().__init__(in_features, out_features, rank, alpha, rslora, base_weight.dtype, base_weight.device)
        with torch.no_grad():
            self.magnitude = nn.Parameter(base_weight.float().norm(dim=1).to(base_weight.dtype))

    def apply(self, x: torch.Tensor, base_weight: torch.Tensor, base_out: torch.Tensor) -> torch.Tensor:
        """Full DoRA output given the frozen base projection's output ``x W^T`` (bias excluded)."""
        combined = base_weight.float() + self.delta_weight()
        norm = combined.norm(dim=1).detach()           # the norm is treated as a constant, as in the paper
        factor = (self.magnitude.float() / norm).to(base_out.dtype)
        return (base_out + self.delta(x)) * factor


class AdapterSet(nn.Module):
    """The adapters of one attention or feed-forward module, keyed by target name."""

    def __init__(self):
        super().__init__()
        self.items = nn.ModuleDict()

    def __contains__(self, k):
        return k in self.items

    def __getitem__(self, k):
        return self.items[k]


def _slices_attention(spec) -> Dict[str, Tuple[int, int]]:
    H, Hkv, D = spec.heads, spec.kv_heads, spec.head_dim
    return {"q": (0, H * D), "k": (H * D, (H + Hkv) * D), "v": ((H + Hkv) * D, (H + 2 * Hkv) * D)}


def _make(base_rows: torch.Tensor, rank, alpha, dora, rslora):
    dtype = base_rows.dtype if base_rows.dtype != torch.float32 or not base_rows.is_cuda else torch.bfloat16
    if dora:
        return DoraAdapter(base_rows.detach().to(dtype), rank, alpha, rslora)
    out_f, in_f = base_rows.shape
    return LoraAdapter(in_f, out_f, rank, alpha, rslora, dtype, base_rows.device)


def add_adapters(model: Decoder, rank: int = 16, alpha: float = 32.0, targets: Sequence[str] = DEFAULT_TARGETS,
                 dora: bool = False, rslora: bool = False, freeze_base: bool = True) -> List[nn.Parameter]:
    """Attach adapters to every block of ``model`` and (by default) freeze everything else.
    Returns the trainable adapter parameters."""
    spec = model.spec
    if freeze_base:
        for p in model.parameters():
            p.requires_grad_(False)
    from ..quant import dense_weight
    for blk in model.blocks:
        a: SelfAttention = blk.attn
        sl = _slices_attention(spec)
        aset = AdapterSet()
        qkv_w = dense_weight(a, "qkv")
        for t in ("q", "k", "v"):
            if t in targets:
                lo, hi = sl[t]
                aset.items[t] = _make(qkv_w[lo:hi], rank, alpha, dora, rslora)
        if "o" in targets:
            aset.items["o"] = _make(dense_weight(a, "o"), rank, alpha, dora, rslora)
        a.adapters = aset
        if isinstance(blk.mlp, FeedForward):
            f: FeedForward = blk.mlp
            fset = AdapterSet()
            hidden = f.hidden
            up_w = dense_weight(f, "up")
            if spec.gated:
                if "gate" in targets:
                    fset.items["gate"] = _make(up_w[:hidden], rank, alpha, dora, rslora)
                if "up" in targets:
                    fset.items["up"] = _make(up_w[hidden:], rank, alpha, dora, rslora)
            elif "up" in targets:
                fset.items["up"] = _make(up_w, rank, alpha, dora, rslora)
            if "down" in targets:
                fset.items["down"] = _make(dense_weight(f, "down"), rank, alpha, dora, rslora)
            f.adapters = fset
    if "head" in targets and model.head is not None:
        hs = AdapterSet()
        hs.items["head"] = _make(model.head[: spec.vocabulary], rank, alpha, dora, rslora)
        model.head_adapters = hs
    model.adapter_config = {"r": rank, "lora_alpha": alpha, "use_dora": dora, "use_rslora": rslora,
                            "target_modules": list(targets)}
    return adapter_parameters(model)


def adapter_parameters(model: nn.Module) -> List[nn.Parameter]:
    return [p for m in model.modules() if isinstance(m, LoraAdapter) for p in m.parameters(recurse=False)]


def named_adapters(model: Decoder) -> Iterable[Tuple[str, LoraAdapter]]:
    """(Idrak module path, adapter) pairs: ``layers.3.attn.q`` ..."""
    for i, blk in enumerate(model.blocks):
        for owner, prefix in ((blk.attn, f"layers.{i}.attn"), (blk.mlp, f"layers.{i}.mlp")):
            aset = getattr(owner, "adapters", None)
            if aset is None:
                continue
            for name, ad in aset.items.items():
                yield f"{prefix}.{name}", ad
    hs = getattr(model, "head_adapters", None)
    if hs is not None:
        yield "head", hs.items["head"]


def remove_adapters(model: Decoder) -> None:
    for blk in model.blocks:
        for owner in (blk.attn, blk.mlp):
            if hasattr(owner, "adapters"):
                del owner.adapters
    if hasattr(model, "head_adapters"):
        del model.head_adapters


@torch.no_grad()
def merge_adapters(model: Decoder) -> None:
    """Fold every adapter into its base weight (``W += scale * B A``; DoRA rescales rows) and remove it."""
    spec = model.spec
    for blk in model.blocks:
        a = blk.attn
        aset = getattr(a, "adapters", None)
        if aset is not None:
            sl = _slices_attention(spec)
            for t in ("q", "k", "v"):
                if t in aset:
                    lo, hi = sl[t]
                    a.qkv_weight[lo:hi].copy_(_merged(a.qkv_weight[lo:hi], aset[t]))
            if "o" in aset:
                a.o_weight.copy_(_merged(a.o_weight, aset["o"]))
        f = blk.mlp
        fset = getattr(f, "adapters", None)
        if fset is not None:
            hidden = f.down_weight.shape[1]
            if spec.gated:
                if "gate" in fset:
                    f.up_weight[:hidden].copy_(_merged(f.up_weight[:hidden], fset["gate"]))
                if "up" in fset:
                    f.up_weight[hidden:].copy_(_merged(f.up_weight[hidden:], fset["up"]))
            elif "up" in fset:
                f.up_weight.copy_(_merged(f.up_weight, fset["up"]))
            if "down" in fset:
                f.down_weight.copy_(_merged(f.down_weight, fset["down"]))
    hs = getattr(model, "head_adapters", None)
    if hs is not None:
        V = spec.vocabulary
        model.head[:V].copy_(_merged(model.head[:V], hs["head"]))
    remove_adapters(model)


def _merged(w: torch.Tensor, ad: LoraAdapter) -> torch.Tensor:
    combined = w.float() + ad.delta_weight()
    if isinstance(ad, DoraAdapter):
        combined = combined * (ad.magnitude.float() / combined.norm(dim=1))[:, None]
    return combined.to(w.dtype)


def _stacked_adapters(x, adapters, slices, out_features):
    """The adapters of one projection as a single pair ``A`` ``[R, in]``, ``B`` ``[out, R]``: the down matrices one under
    the other, each scaled up matrix in its own column block and its own row slice (zeros elsewhere), so that
    ``(x A^T) B^T`` is the sum of the adapters' contributions. ``None`` where the fused kernel does not apply."""
    order = sorted(((lo, hi, n) for n, (lo, hi) in slices.items() if n in adapters), key=lambda t: t[0])
    if not order:
        return None
    ads = [adapters[n] for _, _, n in order]
    total = sum(ad.rank for ad in ads)
    if not lowrank_supported(x, total) or any(ad.rank % 8 or ad.A.dtype != x.dtype for ad in ads):
        return None
    A = ads[0].A if len(ads) == 1 else torch.cat([ad.A for ad in ads], 0)
    blocks = [torch.nn.functional.pad(ad.B * ad.scale, (0, 0, lo, out_features - hi))
              for (lo, hi, _), ad in zip(order, ads)]
    B = blocks[0] if len(blocks) == 1 else torch.cat(blocks, 1)
    return A, B


# --------------------------------------------------------------------------- forward helpers used by the decoder
def project_with_adapters(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                          adapters: Optional[AdapterSet], slices: Dict[str, Tuple[int, int]],
                          residual: Optional[torch.Tensor] = None, packed=None) -> torch.Tensor:
    """``x W^T + b`` with each adapter's contribution added to its column slice of the output.
    ``packed`` is the int8 / int4 replacement of ``weight`` when the base has been quantised."""
    def base(bias_, residual_):
        if packed is not None:
            from ..quant.weights import qlinear
            return qlinear(x, packed, bias_, residual_)
        return ops.linear(x, weight, bias_, residual_)

    out_features = packed.cols if packed is not None else weight.shape[0]
    if adapters is None or len(adapters.items) == 0:
        return base(bias, residual)
    has_dora = any(isinstance(ad, DoraAdapter) for ad in adapters.items.values())
    if not has_dora:
        stacked = _stacked_adapters(x, adapters, slices, out_features)
        if stacked is not None:
            # the adapters ride in the base product as extra blocks of K: no second pass over the output
            A, B = stacked
            if packed is not None:
                from ..quant.weights import qlowrank_linear
                return qlowrank_linear(x, packed, bias, residual, A, B)
            return lowrank_linear(x, weight, bias, residual, A, B)
        y = base(bias, residual)
        parts, last = [], 0
        order = sorted(((lo, hi, n) for n, (lo, hi) in slices.items() if n in adapters), key=lambda t: t[0])
        if len(order) == 1 and order[0][0] == 0 and order[0][1] == out_features:
            return y + adapters[order[0][2]].delta(x)
        for lo, hi, n in order:
            if lo > last:
                parts.append(y[..., last:lo])
            parts.append(y[..., lo:hi] + adapters[n].delta(x))
            last = hi
        if last < y.shape[-1]:
            parts.append(y[..., last:])
        return torch.cat(parts, dim=-1)
    # DoRA rescales the base output, so bias and residual are applied after the rescale
    y = base(None, None)
    dense = weight if packed is None else packed.dequantize().t().to(x.dtype)      # [out, in]
    parts, last = [], 0
    for lo, hi, n in sorted(((lo, hi, n) for n, (lo, hi) in slices.items()), key=lambda t: t[0]):
        if lo > last:
            parts.append(y[..., last:lo])
        seg = y[..., lo:hi]
        if n in adapters:
            ad = adapters[n]
            seg = ad.apply(x, dense[lo:hi], seg) if isinstance(ad, DoraAdapter) else seg + ad.delta(x)
        parts.append(seg)
        last = hi
    if last < y.shape[-1]:
        parts.append(y[..., last:])
    y = torch.cat(parts, dim=-1)
    if bias is not None:
        y = y + bias
    return y + residual if residual is not None else y
