"""Stress runs: many steps, odd shapes, several threads; device memory must not grow from step to step.

``run_stress(step, ...)`` calls ``step(index)`` repeatedly (on ``threads`` threads, each with its own CUDA stream when
the device is a GPU), samples the memory in use after every step once the warm-up is over and fails when the level at
the end exceeds the level after warm-up by more than ``allowed_growth`` bytes. ``default_workload(device)`` is the
step ``idrak check --stress`` runs: decoder training steps over cycling odd sequence lengths plus short generations.

Reference: Stress.Run (src/Idrak.Abstraction.Testing/Stress.cs:137-144).
"""
from __future__ import annotations

import dataclasses
import gc
import threading
import time
from typing import Callable, List, Optional

import torch


@dataclasses.dataclass
class StressReport:
    steps: int
    threads: int
    seconds: float
    memory_after_warmup: int
    memory_at_end: int
    peak: int
    errors: List[str]
    stopped_early: bool = False

    @property
    def growth(self) -> int:
        return self.memory_at_end - self.memory_after_warmup

    @property
    def ok(self) -> bool:
        return not self.errors


def _host_tensor_bytes() -> int:
    gc.collect()
    seen, total = set(), 0
    for o in gc.get_objects():
        try:
            if torch.is_tensor(o) and o.device.type == "cpu":
                st = o.untyped_storage()
                if st.data_ptr() not in seen:
                    seen.add(st.data_ptr())
                    total += st.nbytes()
        except Exception:
            continue
    return total


def memory_in_use(device) -> int:
    device = torch.device(device)
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        return torch.cuda.memory_allocated(device)
    return _host_tensor_bytes()


def run_stress(step: Callable[[int], None], steps: int = 50, warmup: int = 5, device="cuda", threads: int = 1,
               allowed_growth: int = 0, should_stop: Optional[Callable[[], bool]] = None,
               probe: Optional[Callable[[], int]] = None) -> StressReport:
    device = torch.device(device)
    probe = probe or (lambda: memory_in_use(device))
    errors: List[str] = []
    lock = threading.Lock()
    levels: List[int] = []
    stopped = [False]
    t0 = time.perf_counter()

    def run(thread_index: int):
        stream = torch.cuda.Stream(device) if device.type == "cuda" and threads > 1 else None
        for i in range(thread_index, steps + warmup, threads):
            if should_stop is not None and should_stop():
                stopped[0] = True
                return
            try:
                if stream is not None:
                    with torch.cuda.stream(stream):
                        step(i)
                    stream.synchronize()
                else:
                    step(i)
            except Exception as e:
                with lock:
                    errors.append(f"step {i} (thread {thread_index}): {type(e).__name__}: {e}"[:300])
                return
            if threads == 1 and i >= warmup - 1:
                levels.append(probe())

    if threads == 1:
        run(0)
    else:
        # warm-up on one thread first so lazily created state (handles, scratch buffers) is counted before the baseline
        for i in range(warmup):
            step(i)
        levels.append(probe())
        pool = [threading.Thread(target=run, args=(k,), daemon=True) for k in range(threads)]
        for t in pool:
            t.start()
        for t in pool:
            t.join()
        levels.append(probe())
    if device.type == "cuda":
        from .. import _native
        try:
            torch.cuda.synchronize(device)
            _native.check_status("stress")
        except Exception as e:
            errors.append(str(e)[:300])
    base, end = (levels[0], levels[-1]) if levels else (0, 0)
    if end - base > allowed_growth:
        errors.append(f"memory in use grew by {end - base} bytes over {steps} steps (allowed {allowed_growth})")
    return StressReport(steps, threads, time.perf_counter() - t0, base, end, max(levels) if levels else 0, errors, stopped[0])


def default_workload(device="cuda", seed: int = 0) -> Callable[[int], None]:
    """Training steps of a small decoder over cycling odd shapes (sequence lengths that are not tile multiples, batch
    sizes 1-3), every fourth step a short greedy generation through the paged engine."""
    from ..models import DecoderSpec, build_decoder
    from ..ops import FusedAdamW
    from ..serve import GenerationOptions, LLMEngine
    device = torch.device(device)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    spec = DecoderSpec.llama(layers=2, dim=128, heads=2, kv_heads=1, ff_dim=256, vocab=512, max_positions=512)
    model = build_decoder(spec, seed=seed).to(device, dtype)
    opt = FusedAdamW(list(model.parameters()), lr=1e-3) if device.type == "cuda" else torch.optim.AdamW(model.parameters(), lr=1e-3)
    engine = LLMEngine(model, num_blocks=64, max_batch=4)
    shapes = [(1, 7), (2, 129), (3, 200), (1, 511), (2, 64), (1, 1), (3, 333)]
    lock = threading.Lock()

    def step(i: int) -> None:
        with lock:                        # one model: threads take turns, what is tested is stream / allocator hygiene
            B, S = shapes[i % len(shapes)]
            g = torch.Generator().manual_seed(seed * 7919 + i)
            ids = torch.randint(0, 512, (B, S + 1), generator=g).to(device=device, dtype=torch.int32)
            model.train()
            loss = model.loss(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            if i % 4 == 3:
                model.eval()
                engine.generate([[1 + i % 50, 2, 3]], GenerationOptions.greedy_options(6))
    return step
