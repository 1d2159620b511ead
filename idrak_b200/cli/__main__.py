"""``python -m idrak_b200.cli <command>`` - the command-line face of the package.

  health    devices | check | doctor | kernels | memory | bench CASE ...
  models    inspect PATH | convert SRC DST | quantize SRC DST --kind int4 | merge MODEL ADAPTER DST | package ...
  run       complete | chat | batch | embed | tokenize | template
  train     tune | pretrain | perplexity
  serve     serve | ping
  cluster   cluster bench
  config    config

Every command prints plain text or JSON lines and returns a non-zero exit code with a one-line message on bad
input. Reference: the command groups of the ``idrak`` tool (README.md:277-289, src/Idrak.Cli.Commands/Commands/*).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional


class CliError(Exception):
    pass


def _load(path: str, device: str, dtype: Optional[str] = None, adapters: Optional[str] = None):
    import torch
    from ..models.pretrained import load_pretrained
    dt = {None: None, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32,
          "float32": torch.float32, "fp16": torch.float16}[dtype]
    if dt is None:
        dt = torch.bfloat16 if device.startswith("cuda") else torch.float32
    return load_pretrained(path, device=device, dtype=dt, adapters=adapters)


def _tokenizer(path: str):
    from ..text import load_tokenizer, tokenizer_from_gguf
    if path.endswith(".gguf"):
        from ..formats.gguf import GgufFile
        return tokenizer_from_gguf(GgufFile(path).metadata)
    return load_tokenizer(path)


def _device(arg: Optional[str]) -> str:
    import torch
    return arg or ("cuda:0" if torch.cuda.is_available() else "cpu")


def _options(a):
    from ..serve import GenerationOptions
    o = GenerationOptions(max_tokens=a.max_tokens)
    for k in ("temperature", "top_k", "top_p", "min_p", "repeat_penalty", "seed"):
        v = getattr(a, k, None)
        if v is not None:
            setattr(o, k, v)
    if getattr(a, "stop", None):
        o.stop = tuple(a.stop)
    return o


# ------------------------------------------------------------------ health
def cmd_devices(a) -> int:
    import torch
    out = {"cuda": torch.cuda.is_available(), "devices": []}
    for i in range(torch.cuda.device_count() if torch.cuda.is_available() else 0):
        p = torch.cuda.get_device_properties(i)
        free, total = torch.cuda.mem_get_info(i)
        out["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                               "memory": total, "free": free})
    print(json.dumps(out, indent=1))
    return 0


def cmd_check(a) -> int:
    """Library present, kernels load, one tiny training step and one decode run (CPU when there is no GPU)."""
    import torch
    from .. import _native
    from ..models import DecoderSpec, build_decoder
    from ..serve import GenerationOptions, LLMEngine
    report = {"library": str(_native.lib_path()), "library_found": _native.lib_path().exists()}
    dev = _device(a.device)
    dtype = torch.bfloat16 if dev.startswith("cuda") else torch.float32
    spec = DecoderSpec.llama(layers=2, dim=128, heads=2, kv_heads=1, ff_dim=256, vocab=512, max_positions=128)
    m = build_decoder(spec, seed=0).to(dev, dtype)
    ids = torch.randint(0, 512, (2, 64), device=dev, dtype=torch.int32)
    loss = m.loss(ids, ids)
    loss.backward()
    report["train_step_loss"] = round(float(loss), 4)
    eng = LLMEngine(m.eval(), num_blocks=32, max_batch=2)
    report["decode_tokens"] = len(eng.generate([[1, 2, 3]], GenerationOptions.greedy_options(8))[0].output)
    if dev.startswith("cuda"):
        torch.cuda.synchronize()
        _native.check_status("check")
    report["ok"] = report["decode_tokens"] == 8 and report["train_step_loss"] > 0
    if getattr(a, "conformance", False):
        # every operation call of the scenario table, recorded on the CPU and replayed on the device
        from ..testing import check
        rep = check(dev)
        report["conformance"] = json.loads(rep.to_json())
        report["ok"] = report["ok"] and rep.ok
    if getattr(a, "contracts", False):
        from ..testing import SUITES
        report["contracts"] = {name: make().self_test() for name, make in sorted(SUITES.items())}
        report["ok"] = report["ok"] and not any(report["contracts"].values())
    if getattr(a, "stress", 0):
        from ..testing import run_stress
        from ..testing.stress import default_workload
        rep = run_stress(default_workload(dev), steps=a.stress, warmup=14, device=dev,
                         allowed_growth=0 if dev.startswith("cuda") else 1 << 16)
        report["stress"] = {"steps": rep.steps, "seconds": round(rep.seconds, 2), "growth_bytes": rep.growth,
                            "peak_bytes": rep.peak, "errors": rep.errors}
        report["ok"] = report["ok"] and rep.ok
    if getattr(a, "regressions", None):
        from ..testing import replay_folder
        outs = replay_folder(a.regressions, dev)
        report["regressions"] = {"cases": len(outs), "failing": [f"{o.op}: {o.detail}" for o in outs if o.status != "ok"]}
        report["ok"] = report["ok"] and not report["regressions"]["failing"]
    print(json.dumps(report, indent=1))
    return 0 if report["ok"] else 1


def cmd_doctor(a) -> int:
    import torch
    from .. import _native
    from ..config import settings
    lines = [f"python {sys.version.split()[0]}, torch {torch.__version__}, cuda available: {torch.cuda.is_available()}",
             f"native library: {_native.lib_path()} ({'found' if _native.lib_path().exists() else 'MISSING - run python -m idrak_b200.build'})"]
    for mod in ("tokenizers", "jinja2", "fastapi", "uvicorn", "sentencepiece", "numpy"):
        try:
            __import__(mod)
            lines.append(f"{mod}: ok")
        except Exception as e:
            lines.append(f"{mod}: missing ({e})")
    problems = settings.validate()
    lines += [f"environment: {p}" for p in problems] or ["environment: ok"]
    print("\n".join(lines))
    return 1 if problems or not _native.lib_path().exists() else 0


def cmd_kernels(a) -> int:
    from .. import _native
    names = sorted(n for n in _native.exported_names())
    print("\n".join(names))
    return 0


def cmd_memory(a) -> int:
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"cuda": False}))
        return 0
    out = []
    for i in range(torch.cuda.device_count()):
        free, total = torch.cuda.mem_get_info(i)
        out.append({"device": i, "total": total, "free": free, "allocated": torch.cuda.memory_allocated(i),
                    "reserved": torch.cuda.memory_reserved(i)})
    print(json.dumps(out, indent=1))
    return 0


def cmd_bench(a) -> int:
    from ..diag import kernel_cases
    return kernel_cases.main(a.rest)


# ------------------------------------------------------------------ models
def cmd_inspect(a) -> int:
    from ..formats import inspect_file
    print(json.dumps(inspect_file(a.path, tensors=a.tensors), indent=1, default=str))
    return 0


def cmd_convert(a) -> int:
    from ..models.pretrained import save_huggingface, save_idrak
    model = _load(a.src, "cpu", a.dtype or "fp32")
    import torch
    dt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[a.dtype or "fp32"]
    if a.to == "hf":
        save_huggingface(model, a.dst, dtype=dt)
    elif a.to == "idrak":
        save_idrak(model, a.dst, dtype=dt)
    else:
        from ..formats.ikw import save_module
        save_module(model, a.dst, "bfloat16" if dt == torch.bfloat16 else "float16" if dt == torch.float16 else "float32")
    print(json.dumps({"written": a.dst, "format": a.to, "parameters": sum(p.numel() for p in model.parameters())}))
    return 0


def cmd_quantize(a) -> int:
    import torch
    if not torch.cuda.is_available():
        raise CliError("quantize needs a CUDA device (the packing kernels run there)")
    from ..quant import quantize_model
    model = _load(a.src, "cuda:0", "bf16")
    n = quantize_model(model, a.kind)
    from ..quant import save_packed
    save_packed(model, a.dst)
    print(json.dumps({"written": a.dst, "kind": a.kind, "packed_matrices": n}))
    return 0


def cmd_merge(a) -> int:
    from ..adapters.lora import merge_adapters
    from ..models.pretrained import save_huggingface
    model = _load(a.model, "cpu", "fp32", adapters=a.adapter)
    merge_adapters(model)
    save_huggingface(model, a.dst)
    print(json.dumps({"written": a.dst}))
    return 0


def cmd_package(a) -> int:
    """Bundle a model folder (weights + tokenizer + config) into one .ikm file, or list one."""
    from ..formats import ikm
    if a.list:
        with ikm.open_package(a.path) as r:
            print(json.dumps({"created": r.created, "entries": [{"kind": e.kind, "name": e.name} for e in r.entries]},
                             indent=1))
        return 0
    if not a.source:
        raise CliError("package needs --source FOLDER (or --list)")
    model = _load(a.source, "cpu", "fp32")
    w = ikm.create(a.path)
    w.model(model)
    for name in sorted(os.listdir(a.source)):
        full = os.path.join(a.source, name)
        if not os.path.isfile(full):
            continue
        stem = os.path.splitext(name)[0]
        if name == "tokenizer.json":
            with open(full, "r", encoding="utf-8") as f:
                w.tokenizer(json.load(f))
        elif name.endswith(".json") and name not in ("model.safetensors.index.json",):
            with open(full, "r", encoding="utf-8") as f:
                w.json(json.load(f), stem)
        elif name.endswith((".txt", ".jinja")):
            with open(full, "r", encoding="utf-8") as f:
                w.text(f.read(), stem)
    print(json.dumps({"written": w.save()}))
    return 0


# ------------------------------------------------------------------ run
def _generator(a):
    from ..generation import TextGenerator
    dev = _device(a.device)
    model = _load(a.model, dev, getattr(a, "dtype", None), adapters=getattr(a, "adapter", None))
    tok = _tokenizer(a.tokenizer or a.model)
    return TextGenerator(model.eval(), tok, max_batch=getattr(a, "max_batch", 8))


def cmd_complete(a) -> int:
    gen = _generator(a)
    prompt = a.prompt if a.prompt is not None else sys.stdin.read()
    if a.stream:
        for piece in gen.stream(prompt, _options(a)):
            sys.stdout.write(piece)
            sys.stdout.flush()
        sys.stdout.write("\n")
    else:
        r = gen.generate(prompt, _options(a))
        print(r.text if not a.json else json.dumps({"text": r.text, "finish_reason": r.finish_reason,
                                                    "prompt_tokens": r.prompt_tokens,
                                                    "completion_tokens": r.completion_tokens}))
    return 0


def cmd_chat(a) -> int:
    gen = _generator(a)
    messages = [{"role": "system", "content": a.system}] if a.system else []
    if a.message:
        r = gen.chat(messages + [{"role": "user", "content": a.message}], _options(a))
        print(r.text)
        return 0
    while True:                                   # interactive: one line per turn, empty line or EOF ends
        try:
            line = input("> ")
        except EOFError:
            break
        if not line.strip():
            break
        messages.append({"role": "user", "content": line})
        text = ""
        for piece in gen.stream(messages, _options(a)):
            sys.stdout.write(piece)
            sys.stdout.flush()
            text += piece
        sys.stdout.write("\n")
        messages.append({"role": "assistant", "content": text})
    return 0


def cmd_batch(a) -> int:
    """One prompt per input line (or a JSON object with "prompt" / "messages"); one JSON line out per input."""
    gen = _generator(a)
    prompts = []
    with open(a.input, "r", encoding="utf-8") as f:
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            if line.lstrip().startswith("{"):
                obj = json.loads(line)
                prompts.append(obj.get("messages") or obj["prompt"])
            else:
                prompts.append(line)
    results = gen.generate_batch(prompts, _options(a))
    out = open(a.output, "w", encoding="utf-8") if a.output else sys.stdout
    for p, r in zip(prompts, results):
        out.write(json.dumps({"prompt": p, "text": r.text, "finish_reason": r.finish_reason,
                              "completion_tokens": r.completion_tokens}, ensure_ascii=False) + "\n")
    if a.output:
        out.close()
    return 0


def cmd_embed(a) -> int:
    gen = _generator(a)
    for text in a.text:
        v = gen.engine.runner.embed_text(gen.tokenizer.encode(text), a.pooling)
        print(json.dumps({"text": text, "embedding": [round(float(x), 6) for x in v.tolist()]}))
    return 0


def cmd_tokenize(a) -> int:
    tok = _tokenizer(a.tokenizer)
    if a.output:                                  # write a token file from text files
        from ..formats.tokens import write_tokens
        ids: List[int] = []
        docs = 0
        eos = list(tok.eos_token_ids[:1])
        for path in a.files:
            with open(path, "r", encoding="utf-8") as f:
                for doc in f.read().split(a.separator):
                    if doc.strip():
                        ids += tok.encode(doc, add_special_tokens=False) + eos
                        docs += 1
        rec = write_tokens(a.output, ids, tok.vocab_size, documents=docs, separator=eos[0] if eos else None)
        print(json.dumps(rec))
        return 0
    text = a.text if a.text is not None else sys.stdin.read()
    ids = tok.encode(text)
    print(json.dumps({"ids": ids, "count": len(ids), "pieces": [tok.decode([i], skip_special_tokens=False) for i in ids]},
                     ensure_ascii=False))
    return 0


def cmd_template(a) -> int:
    from ..text.chat import ChatTemplate
    tok = _tokenizer(a.tokenizer)
    msgs = json.loads(a.messages) if a.messages else [{"role": "user", "content": "Hello"}]
    t = ChatTemplate.for_tokenizer(tok)
    print(t.render(msgs, add_generation_prompt=not a.no_generation_prompt))
    print(f"# tool-call format: {t.tool_call_format}", file=sys.stderr)
    return 0


# ------------------------------------------------------------------ train
def _read_examples(path: str) -> List[dict]:
    out = []
    with open(path, "r", encoding="utf-8") as f:
        head = f.read(1)
        f.seek(0)
        if head == "[":
            return json.load(f)
        for line in f:
            if line.strip():
                out.append(json.loads(line))
    return out


def cmd_tune(a) -> int:
    from ..text.finetuning import FineTuner, FineTuningOptions
    dev = _device(a.device)
    model = _load(a.model, dev, a.dtype)
    tok = _tokenizer(a.tokenizer or a.model)
    o = FineTuningOptions(rank=a.rank, alpha=a.alpha, dora=a.dora, base=a.base, learning_rate=a.lr, epochs=a.epochs,
                          max_steps=a.max_steps, batch_tokens=a.batch_tokens, max_length=a.max_length,
                          accumulation=a.accumulation, loss=a.loss, save_every=a.save_every, seed=a.seed,
                          resume_from=a.resume)
    train = _read_examples(a.data)
    evaluation = _read_examples(a.eval) if a.eval else None
    res = FineTuner.train(model, tok, train, evaluation, o, a.out,
                          progress=lambda s, l: print(json.dumps({"step": s, "loss": round(l, 4)}), flush=True))
    print(json.dumps({"steps": res.steps, "tokens": res.tokens, "final_loss": res.losses[-1] if res.losses else None,
                      "eval": res.eval_losses, "adapter": res.adapter_folder}))
    return 0


def cmd_pretrain(a) -> int:
    import torch
    import torch.distributed as dist
    from ..models import DecoderSpec, build_decoder
    from ..text.pretraining import PretrainOptions, PretrainStage, Pretrainer
    with open(a.plan, "r", encoding="utf-8") as f:
        plan = json.load(f)
    if "RANK" in os.environ and not dist.is_initialized():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
    dev = _device(a.device) if not dist.is_initialized() or not torch.cuda.is_available() else f"cuda:{torch.cuda.current_device()}"
    if a.model:
        model = _load(a.model, dev, a.dtype)
    else:
        spec = DecoderSpec.from_json(plan["spec"]) if isinstance(plan.get("spec"), dict) else \
            getattr(DecoderSpec, plan.get("preset", "gpt2"))()
        model = build_decoder(spec, seed=plan.get("seed", 0)).to(dev, torch.bfloat16 if dev.startswith("cuda") else torch.float32)
    stages = [PretrainStage(**s) for s in plan["stages"]]
    keys = {k: v for k, v in plan.items() if k in PretrainOptions.__dataclass_fields__ and k != "stages"}
    o = PretrainOptions(stages=stages, out_dir=a.out, resume_from=a.resume, **keys)
    rank0 = not dist.is_initialized() or dist.get_rank() == 0
    res = Pretrainer.train(model, o, progress=(lambda s, l: print(json.dumps({"step": s, "loss": round(l, 4)}), flush=True))
                           if rank0 else None)
    if rank0:
        print(json.dumps({"steps": res.steps, "tokens": res.tokens, "tokens_per_second": round(res.tokens_per_second, 1),
                          "final_loss": res.losses[-1] if res.losses else None, "checkpoints": res.checkpoints}))
    return 0


def cmd_perplexity(a) -> int:
    import math
    import torch
    from ..formats.tokens import TokenFile
    dev = _device(a.device)
    model = _load(a.model, dev, a.dtype).eval()
    f = TokenFile(a.tokens, a.seq_len)
    n = min(len(f), a.windows)
    total = 0.0
    with torch.no_grad():
        for i in range(n):
            x, y = f.window(i)
            total += float(model.loss(x[None].int().to(dev), y[None].int().to(dev)))
    loss = total / max(n, 1)
    print(json.dumps({"windows": n, "loss": round(loss, 5), "perplexity": round(math.exp(loss), 4)}))
    return 0


# ------------------------------------------------------------------ serve / cluster / config
def cmd_serve(a) -> int:
    from ..config import settings
    from ..serve.api import serve
    from ..serve.inference_engine import InferenceEngine
    builder = InferenceEngine.create()
    dev = _device(a.device)
    for item in a.model:
        name, _, path = item.partition("=")
        if not path:
            name, path = os.path.basename(os.path.normpath(item)), item
        builder.add_chat(name, (lambda p=path: (_load(p, dev, a.dtype).eval(), _tokenizer(p))),
                         queue_limit=settings.get("IDRAK_QUEUE_LIMIT"), timeout=settings.get("IDRAK_REQUEST_TIMEOUT"),
                         keep_alive=settings.get("IDRAK_KEEP_ALIVE"),
                         engine_args={"max_batch": settings.get("IDRAK_MAX_BATCH")})
    serve(builder.build(), host=a.host, port=a.port)
    return 0


def cmd_ping(a) -> int:
    import urllib.request
    with urllib.request.urlopen(a.url.rstrip("/") + "/api/version", timeout=a.timeout) as r:
        print(r.read().decode())
    return 0


def cmd_cluster_bench(a) -> int:
    from ..diag import tp_bench
    return tp_bench.main(a.rest)


def cmd_config(a) -> int:
    from ..config import describe, settings
    print(describe())
    problems = settings.validate()
    for p in problems:
        print("problem:", p, file=sys.stderr)
    return 1 if problems else 0


def cmd_tuning(a) -> int:
    """Show (or forget) the measured decisions kept for this GPU."""
    from ..runtime.tuning import tuner
    t = tuner()
    if a.forget is not None:
        print(f"forgot {t.forget(a.forget)} decisions")
        return 0
    print(f"file   {t.path}\ndevice {t.key}\ntuning {'on' if t.enabled else 'off (set IDRAK_AUTOTUNE=1 to measure)'}")
    for name, e in sorted(t.entries().items()):
        ratios = ", ".join(f"{k}: {v:.3f}" for k, v in e.get("ratios", {}).items())
        print(f"  {name}  ->  {e['choice']}  (default {e['default']} {e.get('default_ms', 0):.4f} ms; ratios {ratios})")
    return 0


def cmd_limits(a) -> int:
    """The device's limits and whether each tensor-core kernel's compile-time shape fits them."""
    from ..runtime.limits import check_device, device_limits, kernel_shapes
    lim = device_limits()
    print("device limits" + ("" if lim.measured else " (no GPU here: the figures the kernels were written for)"))
    for k, v in lim.as_dict().items():
        if k != "measured":
            print(f"  {k:32s} {v}")
    print(f"  {'peak_memory_gbs (nominal)':32s} {lim.peak_memory_gbs:.0f}")
    verdicts = check_device(lim)
    print("kernel shapes")
    for k in kernel_shapes():
        print(f"  {k.kernel:26s} {k.tile}; {k.stages} stages, {k.threads} threads, {k.shared_bytes} B shared, "
              f"{k.tensor_memory_columns} tensor-memory columns, {k.blocks_per_sm} per SM: {verdicts[k.kernel]}")
    return 0 if all(v == "ok" for v in verdicts.values()) else 1


# ------------------------------------------------------------------ parser
def _sampling(p):
    p.add_argument("--max-tokens", type=int, default=256)
    p.add_argument("--temperature", type=float)
    p.add_argument("--top-k", type=int)
    p.add_argument("--top-p", type=float)
    p.add_argument("--min-p", type=float)
    p.add_argument("--repeat-penalty", type=float)
    p.add_argument("--seed", type=int)
    p.add_argument("--stop", action="append")


def _model_args(p, tokenizer=True):
    p.add_argument("--model", required=True, help="model folder, .gguf file or .ikm package")
    if tokenizer:
        p.add_argument("--tokenizer", help="tokenizer folder / file (default: the model's)")
    p.add_argument("--adapter", help="PEFT adapter folder to attach")
    p.add_argument("--device")
    p.add_argument("--dtype", choices=["bf16", "fp32", "fp16"])


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="idrak", description="idrak_b200 command line")
    sub = ap.add_subparsers(dest="command", required=True)

    def add(name, fn, help_):
        p = sub.add_parser(name, help=help_)
        p.set_defaults(fn=fn)
        return p

    add("devices", cmd_devices, "list CUDA devices")
    add("limits", cmd_limits, "the device's limits and which kernel shapes fit them")
    p = add("tuning", cmd_tuning, "show the measured per-device decisions (split-K factors, ...)")
    p.add_argument("--forget", nargs="?", const="", metavar="PREFIX", help="drop decisions whose name starts with PREFIX (all without one)")
    p = add("check", cmd_check, "run one tiny training step and one decode; optionally the conformance kit")
    p.add_argument("--device")
    p.add_argument("--conformance", action="store_true", help="replay every recorded operation call on the device against the CPU")
    p.add_argument("--contracts", action="store_true", help="run the contract suites against their references and broken twins")
    p.add_argument("--stress", type=int, default=0, metavar="STEPS", help="run STEPS mixed steps; device memory must not grow")
    p.add_argument("--regressions", metavar="FOLDER", help="replay saved failing cases")
    from . import extra, more
    extra.register(add)
    more.register(add)
    add("doctor", cmd_doctor, "report what is installed and what is missing")
    add("kernels", cmd_kernels, "list the native library's entry points")
    add("memory", cmd_memory, "device memory in use")
    add("bench", cmd_bench, "time one kernel case (see diag.kernel_cases)").add_argument("rest", nargs=argparse.REMAINDER)
    p = add("inspect", cmd_inspect, "describe a weights / package / token file")
    p.add_argument("path")
    p.add_argument("--tensors", action="store_true")
    p = add("convert", cmd_convert, "re-write a model in another format")
    p.add_argument("src")
    p.add_argument("dst")
    p.add_argument("--to", choices=["hf", "idrak", "ikw"], default="hf")
    p.add_argument("--dtype", choices=["fp32", "bf16", "fp16"])
    p = add("quantize", cmd_quantize, "pack a model's projections to int8 / int4")
    p.add_argument("src")
    p.add_argument("dst")
    p.add_argument("--kind", choices=["int8", "int4"], default="int4")
    p = add("merge", cmd_merge, "fold a PEFT adapter into the base weights")
    p.add_argument("model")
    p.add_argument("adapter")
    p.add_argument("dst")
    p = add("package", cmd_package, "write or list an .ikm package")
    p.add_argument("path")
    p.add_argument("--source")
    p.add_argument("--list", action="store_true")
    p = add("complete", cmd_complete, "continue a prompt")
    _model_args(p)
    _sampling(p)
    p.add_argument("--prompt")
    p.add_argument("--stream", action="store_true")
    p.add_argument("--json", action="store_true")
    p = add("chat", cmd_chat, "chat with a model (one message or interactive)")
    _model_args(p)
    _sampling(p)
    p.add_argument("--system")
    p.add_argument("--message")
    p = add("batch", cmd_batch, "run a file of prompts through continuous batching")
    _model_args(p)
    _sampling(p)
    p.add_argument("--input", required=True)
    p.add_argument("--output")
    p.add_argument("--max-batch", type=int, default=32)
    p = add("embed", cmd_embed, "sentence vectors from the final hidden states")
    _model_args(p)
    p.add_argument("--pooling", choices=["mean", "last"], default="mean")
    p.add_argument("text", nargs="+")
    p = add("tokenize", cmd_tokenize, "show token ids, or write a token file from text files")
    p.add_argument("--tokenizer", required=True)
    p.add_argument("--text")
    p.add_argument("--output")
    p.add_argument("--separator", default="\n\n")
    p.add_argument("files", nargs="*")
    p = add("template", cmd_template, "render a chat template")
    p.add_argument("--tokenizer", required=True)
    p.add_argument("--messages")
    p.add_argument("--no-generation-prompt", action="store_true")
    p = add("tune", cmd_tune, "LoRA / DoRA fine-tuning")
    _model_args(p)
    p.add_argument("--data", required=True)
    p.add_argument("--eval")
    p.add_argument("--out", required=True)
    p.add_argument("--rank", type=int, default=16)
    p.add_argument("--alpha", type=float, default=32.0)
    p.add_argument("--dora", action="store_true")
    p.add_argument("--base", choices=["bf16", "int8", "int4"], default="bf16")
    p.add_argument("--lr", type=float, default=2e-4)
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--max-steps", type=int, default=0)
    p.add_argument("--batch-tokens", type=int, default=4096)
    p.add_argument("--max-length", type=int, default=2048)
    p.add_argument("--accumulation", type=int, default=1)
    p.add_argument("--loss", choices=["sft", "dpo"], default="sft")
    p.add_argument("--save-every", type=int, default=0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--resume")
    p = add("pretrain", cmd_pretrain, "pre-train from a JSON plan (stages, batch sizes, model spec)")
    p.add_argument("--plan", required=True)
    p.add_argument("--model")
    p.add_argument("--out")
    p.add_argument("--resume")
    p.add_argument("--device")
    p.add_argument("--dtype", choices=["bf16", "fp32"])
    p = add("perplexity", cmd_perplexity, "loss and perplexity over a token file")
    _model_args(p, tokenizer=False)
    p.add_argument("--tokens", required=True)
    p.add_argument("--seq-len", type=int, default=1024)
    p.add_argument("--windows", type=int, default=64)
    p = add("serve", cmd_serve, "serve models over HTTP (/v1, /api)")
    p.add_argument("--model", action="append", required=True, help="NAME=PATH or PATH; repeatable")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--device")
    p.add_argument("--dtype", choices=["bf16", "fp32", "fp16"])
    p = add("ping", cmd_ping, "ask a running server for its version")
    p.add_argument("--url", default="http://127.0.0.1:8000")
    p.add_argument("--timeout", type=float, default=5.0)
    p = add("cluster-bench", cmd_cluster_bench, "fused tensor-parallel kernels vs NCCL (run under torchrun)")
    p.add_argument("rest", nargs=argparse.REMAINDER)
    add("config", cmd_config, "the settings table and the current values")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        return int(args.fn(args) or 0)
    except CliError as e:
        print(f"idrak: {e}", file=sys.stderr)
        return 2
    except (FileNotFoundError, ValueError, KeyError, NotImplementedError) as e:
        print(f"idrak {args.command}: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    raise SystemExit(main())
