"""Small, self-contained cases of each hot kernel, for timing and for profiler captures.

    python -m idrak_b200.diag.kernel_cases gemm --m 8192 --n 8192 --k 4096 --iters 3
    python -m idrak_b200.diag.kernel_cases flash_fwd --batch 8 --heads 12 --seq 1024 --dim 64
    python -m idrak_b200.diag.kernel_cases list

Each case allocates its inputs (larger than the 126 MB L2 where the kernel is memory-bound, a few GB at most),
runs ``--warmup`` launches, then times ``--iters`` launches with CUDA events and prints one JSON line with the
time per launch and the achieved TFLOP/s or GB/s. Under a profiler use ``--warmup 1 --iters 3`` and capture by
kernel name. Between timed launches a buffer larger than L2 is rewritten when ``--flush-l2`` is given.

Reference: the benchmark runner of the reference (benchmarks/Idrak.Benchmarks/Program.cs) times its kernels the
same way - a named case per kernel family, warm-up, then a timed loop.
"""
from __future__ import annotations

import argparse
import json
import math
from typing import Callable, Dict, Tuple

import torch


def _timed(fn: Callable[[], None], warmup: int, iters: int, flush: bool) -> float:
    dev = torch.device("cuda")
    junk = torch.empty(160 << 20, dtype=torch.uint8, device=dev) if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if junk is not None:
            junk.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def _timed_graph(fn: Callable[[], None], warmup: int, iters: int, flush: bool, reps: int) -> float:
    """Device time of one ``fn`` with the host's launch cost taken out: ``reps`` copies of (L2 flush, fn) are captured
    into one CUDA graph, a second graph holds the flushes alone, and the difference of their replay times is
    divided by ``reps``. For kernels of a few microseconds, where the plain loop measures the host."""
    dev = torch.device("cuda")
    junk = torch.empty(160 << 20, dtype=torch.uint8, device=dev) if flush else None
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(warmup, 1)):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    def capture(with_fn: bool):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                if junk is not None:
                    junk.fill_(1)
                if with_fn:
                    fn()
        return g

    def replay_ms(g) -> float:
        g.replay()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / iters

    full = replay_ms(capture(True))
    base = replay_ms(capture(False)) if junk is not None else 0.0
    return (full - base) / reps


def case_gemm(a) -> Tuple[Callable, float, float]:
    """``--epi`` picks the fused epilogue: plain, bias, bias_res, bias_gelu (saves the pre-activation), gelu_grad
    (input gradient through a saved pre-activation; the weight operand is read MN-major like a backward pass)."""
    from ..ops.gemm import gemm
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    flops, nbytes = 2.0 * a.m * a.n * a.k, 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n)
    epi = getattr(a, "epi", "plain")
    if epi in ("gelu_grad", "mul_aux"):
        w = torch.randn(a.k, a.n, device="cuda", dtype=torch.bfloat16)          # [out, in] of the layer: B stored [K, N]
        aux = torch.randn(a.m, a.n, device="cuda", dtype=torch.bfloat16)
        return (lambda: gemm(x, w, b_mn=True, act=epi, aux=aux, out=out)), flops, nbytes + 2.0 * a.m * a.n
    w = torch.randn(a.n, a.k, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(a.n, device="cuda", dtype=torch.bfloat16) if epi != "plain" else None
    if epi == "bias_res":
        res = torch.randn(a.m, a.n, device="cuda", dtype=torch.bfloat16)
        return (lambda: gemm(x, w, bias=bias, residual=res, out=out)), flops, nbytes + 2.0 * a.m * a.n
    if epi in ("bias_gelu", "bias_gelu_d"):
        aux = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
        act = "gelu" if epi == "bias_gelu" else "gelu_d"
        return (lambda: gemm(x, w, bias=bias, act=act, aux=aux, out=out)), flops, nbytes + 2.0 * a.m * a.n
    return (lambda: gemm(x, w, bias=bias, out=out)), flops, nbytes


def case_gemm_wgrad(a):
    from ..ops.gemm import gemm
    dy = torch.randn(a.k, a.m, device="cuda", dtype=torch.bfloat16)      # [tokens, out]
    x = torch.randn(a.k, a.n, device="cuda", dtype=torch.bfloat16)       # [tokens, in]
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.float32)
    return (lambda: gemm(dy, x, a_mn=True, b_mn=True, out=out)), 2.0 * a.m * a.n * a.k, 2.0 * a.k * (a.m + a.n) + 4.0 * a.m * a.n


def case_cublas(a):
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(a.n, a.k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    return (lambda: torch.matmul(x, w.t(), out=out)), 2.0 * a.m * a.n * a.k, 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n)


def _qkv(a):
    q = torch.randn(a.batch, a.seq, a.heads, a.dim, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(a.batch, a.seq, a.kv_heads or a.heads, a.dim, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    return q, k, v


def case_flash_fwd(a):
    from ..ops.attention import flash_forward
    q, k, v = _qkv(a)
    flops = 4.0 * a.batch * a.heads * a.seq * a.seq * a.dim / 2          # causal: half the square
    return (lambda: flash_forward(q, k, v, True)), flops, 2.0 * (2 * q.numel() + 2 * k.numel())


def case_flash_bwd(a):
    from ..ops.attention import flash_backward, flash_forward
    q, k, v = _qkv(a)
    out, lse = flash_forward(q, k, v, True)
    dout = torch.randn_like(out)
    flops = 10.0 * a.batch * a.heads * a.seq * a.seq * a.dim / 2
    return (lambda: flash_backward(dout, q, k, v, out, lse, True)), flops, 2.0 * (4 * q.numel() + 4 * k.numel())


def case_xent(a):
    from ..ops.loss import softmax_xent_
    rows, vocab = a.m, a.n
    ld = (vocab + 127) // 128 * 128
    logits = torch.randn(rows, ld, device="cuda", dtype=torch.bfloat16)
    targets = torch.randint(0, vocab, (rows,), device="cuda", dtype=torch.int32)
    return (lambda: softmax_xent_(logits, targets, vocab, 1.0 / rows)), 0.0, 4.0 * rows * ld


def case_norm(a):
    from ..ops.rowops import norm_forward
    x = torch.randn(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(a.n, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(a.n, device="cuda", dtype=torch.bfloat16)
    return (lambda: norm_forward(x, w, b, 1e-5, False)), 0.0, 4.0 * a.m * a.n


def case_norm_bwd(a):
    """LayerNorm backward with the residual gradient added and the column sums of dx produced (--m rows, --n columns)."""
    from ..ops.rowops import norm_backward, norm_forward
    x = torch.randn(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(a.n, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(a.n, device="cuda", dtype=torch.bfloat16)
    _, mean, rstd, _ = norm_forward(x, w, b, 1e-5, False)
    dy, dres = torch.randn_like(x), torch.randn_like(x)
    return (lambda: norm_backward(dy, x, w, mean, rstd, False, True, dres, sums_of_dx=True)), 0.0, 8.0 * a.m * a.n


def case_adamw(a):
    from ..ops.optim import FusedAdamW
    n = a.m * a.n
    p = torch.nn.Parameter(torch.randn(n, device="cuda", dtype=torch.bfloat16))
    p.grad = torch.randn_like(p)
    opt = FusedAdamW([p], lr=1e-3, max_grad_norm=1.0)
    return (lambda: opt.step()), 0.0, float(n) * (2 + 2 + 2 + 16)        # grad, p in/out, fp32 m and v in/out


def case_decode_attn(a):
    from ..ops.decode import paged_decode
    hkv = a.kv_heads or a.heads
    blocks_per_seq = (a.seq + 15) // 16
    nb = a.batch * blocks_per_seq
    kc = torch.randn(nb, 16, hkv, a.dim, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    table = torch.arange(nb, device="cuda", dtype=torch.int32).view(a.batch, blocks_per_seq)
    lens = torch.full((a.batch,), a.seq, device="cuda", dtype=torch.int32)
    q = torch.randn(a.batch, a.heads, a.dim, device="cuda", dtype=torch.bfloat16)
    return (lambda: paged_decode(q, kc, vc, table, lens, max_len_hint=a.seq)), 4.0 * a.batch * a.heads * a.seq * a.dim, 4.0 * kc.numel()


def case_skinny(a):
    """Few-row projection (--m <= 64 rows, --n features, --k): --epi plain | bias_res | gated | norm picks the epilogue;
    bytes are the weights streamed once."""
    from ..ops.skinny import skinny_linear
    gate = "silu" if a.epi == "gated" else None
    rows = 2 * a.n if gate else a.n
    w = torch.randn(rows, a.k, device="cuda", dtype=torch.bfloat16) * a.k ** -0.5
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(rows, device="cuda", dtype=torch.bfloat16) if a.epi == "bias_res" else None
    res = torch.randn(a.m, a.n, device="cuda", dtype=torch.bfloat16) if a.epi == "bias_res" else None
    eps = 1e-5 if a.epi == "norm" else None
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    return (lambda: skinny_linear(x, w, bias, res, gate, eps, out)), 2.0 * a.m * rows * a.k, 2.0 * rows * a.k


def case_skinny8(a):
    """The few-row product over int8 weights (--m <= 64, --n, --k; --epi gated for a stacked gate / up matrix): bytes
    are the codes streamed once."""
    from ..ops.skinny import skinny8_linear
    from ..quant import Int8Weight
    gate = "silu" if a.epi == "gated" else None
    cols = 2 * a.n if gate else a.n
    w8 = Int8Weight.quantize(torch.randn(a.k, cols, device="cuda") * a.k ** -0.5)
    w8.kmajor()
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    return (lambda: skinny8_linear(x, w8, None, None, gate, out)), 2.0 * a.m * cols * a.k, 1.0 * cols * a.k


def case_skinny_dense(a):
    """The same product on the dense GEMM with its split-K choice (what decode used before) for comparison."""
    from ..ops.gemm import gemm
    w = torch.randn(a.n, a.k, device="cuda", dtype=torch.bfloat16) * a.k ** -0.5
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    return (lambda: gemm(x, w)), 2.0 * a.m * a.n * a.k, 2.0 * a.n * a.k


def case_qgemm(a):
    from ..quant.weights import qgemm, quantize_weight
    w = quantize_weight(torch.randn(a.k, a.n, device="cuda", dtype=torch.bfloat16), a.kind)
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    bits = 4 if a.kind == "int4" else 8
    return (lambda: qgemm(x, w)), 2.0 * a.m * a.n * a.k, a.k * a.n * bits / 8 + 2.0 * a.m * (a.k + a.n)


def case_qdequant(a):
    """Unpack a packed [--k, --n] weight (--kind int4 | int8) to bf16: bytes = codes + scales read, bf16 written."""
    from ..quant.weights import dequantize_bf16, quantize_weight
    w = quantize_weight(torch.randn(a.k, a.n, device="cuda", dtype=torch.bfloat16), a.kind)
    bits = 4 if a.kind == "int4" else 8
    return (lambda: dequantize_bf16(w)), 0.0, a.k * a.n * (bits / 8 + 2.0)


def _role_timers(fn: Callable[[], None]) -> dict:
    """One launch with the dense GEMM's role timers on: mean cycles per tile, over the CTAs that ran tiles."""
    import ctypes as C
    from .. import _native
    lib = _native.lib()
    sms = lib.idrak_sm_count()
    buf = torch.zeros(sms * 8, device="cuda", dtype=torch.int64)
    setter = _native.bind("idrak_gemm_role_timers", None, [C.c_void_p])
    setter(buf.data_ptr())
    try:
        fn()
        torch.cuda.synchronize()
    finally:
        setter(None)
    t = buf.view(sms, 8).cpu().double()
    ran = t[:, 6] > 0
    t = t[ran]
    tiles = t[:, 6].clamp(min=1)
    mean = lambda c: round(float((t[:, c] / tiles).mean()), 1)
    return {"ctas": int(ran.sum()), "tiles_per_cta": round(float(tiles.mean()), 2),
            "mma_loop_cycles_per_tile": mean(0), "mma_wait_accumulator": mean(1), "mma_wait_operands": mean(2),
            "epilogue_wait_accumulator": mean(4), "epilogue_drain": mean(5)}


CASES: Dict[str, Callable] = {
    "gemm": case_gemm, "gemm_wgrad": case_gemm_wgrad, "cublas": case_cublas, "flash_fwd": case_flash_fwd,
    "flash_bwd": case_flash_bwd, "xent": case_xent, "norm": case_norm, "norm_bwd": case_norm_bwd, "adamw": case_adamw,
    "skinny": case_skinny, "skinny8": case_skinny8, "skinny_dense": case_skinny_dense,
    "decode_attn": case_decode_attn, "qgemm": case_qgemm, "qdequant": case_qdequant,
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("case", choices=sorted(CASES) + ["list"])
    for name, default in (("m", 8192), ("n", 8192), ("k", 4096), ("batch", 8), ("heads", 12), ("kv-heads", 0),
                          ("seq", 1024), ("dim", 64), ("warmup", 3), ("iters", 10)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--kind", default="int4", choices=["int4", "int8"])
    ap.add_argument("--epi", default="plain", choices=["plain", "bias", "bias_res", "bias_gelu", "gelu_grad", "bias_gelu_d", "mul_aux", "gated", "norm"])
    ap.add_argument("--role-timers", action="store_true",
                    help="gemm cases: after timing, run one more launch with the kernel's role timers on and print "
                         "the mean cycles per tile each warp role spent waiting")
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--graph", type=int, default=0, metavar="REPS",
                    help="time REPS captured copies per replay of a CUDA graph (takes the host's launch cost out)")
    a = ap.parse_args(argv)
    if a.case == "list":
        print("\n".join(sorted(CASES)))
        return 0
    torch.cuda.set_device(0)
    fn, flops, nbytes = CASES[a.case](a)
    ms = (_timed_graph(fn, a.warmup, a.iters, a.flush_l2, a.graph) if a.graph > 0
          else _timed(fn, a.warmup, a.iters, a.flush_l2))
    from .. import _native
    _native.check_status()
    roles = _role_timers(fn) if a.role_timers else None
    out = {"case": a.case, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1) if flops else None,
           "gbs": round(nbytes / ms / 1e6, 1), "args": {k: v for k, v in vars(a).items() if k != "case"}}
    if roles:
        out["roles"] = roles
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
