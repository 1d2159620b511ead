"""Commands over the data, retrieval, ONNX, imaging and audio packages.

    idrak data   convert|dedupe|split|mix ...      records between formats, near-duplicate removal, splits, mixtures
    idrak index  build / idrak search              BM25 (and vector, with a model) retrieval over text files
    idrak onnx   export|run|inspect                networks to ONNX, ONNX graphs on tensors
    idrak page                                     a synthetic text page with effects, as PNG + word boxes
    idrak image  resize|effects                    Pillow-exact resampling, seeded scan effects on image files
    idrak audio  features|resample                 log-mel features, resampled WAV files

Reference: the Data, Retrieval, Models (convert / export) and Voices command groups of the reference's tool
(src/Idrak.Cli.Commands/Commands).
"""
from __future__ import annotations

import json
import os
import sys


def _out(obj) -> None:
    print(json.dumps(obj, ensure_ascii=False))


# ---------------------------------------------------------------------------------------------------------------------
def cmd_data(a) -> int:
    from .. import data as D
    if a.action == "convert":
        n = D.write_jsonl(D.read_records(a.inputs[0]), a.output)
        _out({"written": n, "to": a.output})
    elif a.action == "dedupe":
        rows = D.dedupe(D.read_records(a.inputs[0]), key=lambda r: str(r.get(a.field, r)), near=a.near, threshold=a.threshold)
        _out({"kept": D.write_jsonl(rows, a.output), "to": a.output})
    elif a.action == "split":
        first, rest = D.split_rows(list(D.read_records(a.inputs[0])), a.fraction, a.seed)
        stem, ext = os.path.splitext(a.output)
        _out({"first": D.write_jsonl(first, f"{stem}.a{ext or '.jsonl'}"), "rest": D.write_jsonl(rest, f"{stem}.b{ext or '.jsonl'}")})
    elif a.action == "mix":
        weights = [float(w) for w in a.weights.split(",")] if a.weights else None
        rows = D.mix([D.read_records(p) for p in a.inputs], weights, a.seed)
        _out({"written": D.write_jsonl(rows, a.output), "to": a.output})
    elif a.action == "count":
        _out({"records": sum(1 for _ in D.read_records(a.inputs[0]))})
    return 0


def cmd_index(a) -> int:
    from .. import data as D
    from ..rag import chunks_of
    texts = [(r.get("source", r.get("path", "")), str(r.get(a.field, ""))) for p in a.inputs for r in D.read_records(p)]
    chunks = chunks_of(texts, a.size, a.overlap)
    os.makedirs(a.output, exist_ok=True)
    with open(os.path.join(a.output, "chunks.jsonl"), "w", encoding="utf-8") as f:
        for c in chunks:
            f.write(json.dumps({"text": c.text, "source": c.source, "start": c.start}, ensure_ascii=False) + "\n")
    _out({"chunks": len(chunks), "index": a.output})
    return 0


def cmd_search(a) -> int:
    from ..rag import Bm25Index, Chunk
    with open(os.path.join(a.index, "chunks.jsonl"), "r", encoding="utf-8") as f:
        chunks = [Chunk(**json.loads(line)) for line in f if line.strip()]
    for h in Bm25Index(chunks).search(a.query, a.k):
        _out({"score": round(h.score, 4), "source": h.chunk.source, "start": h.chunk.start, "text": h.chunk.text})
    return 0


def cmd_onnx(a) -> int:
    import numpy as np
    import torch
    from .. import onnx as ox
    if a.action == "inspect":
        m = ox.proto.Model.parse(open(a.path, "rb").read())
        ops = {}
        for n in m.graph.nodes:
            ops[n.op_type] = ops.get(n.op_type, 0) + 1
        _out({"opset": m.opset, "producer": m.producer, "inputs": [(v.name, v.shape) for v in m.graph.inputs if v.name not in m.graph.initializers],
              "outputs": [(v.name, v.shape) for v in m.graph.outputs], "nodes": len(m.graph.nodes), "operators": ops,
              "parameters": int(sum(np.asarray(t).size for t in m.graph.initializers.values())),
              "unsupported": sorted(set(ops) - set(ox.OPS))})
    elif a.action == "export":
        from ..nn import Network
        desc = json.load(open(a.path, "r", encoding="utf-8"))
        model = Network.from_json(desc).build()
        if a.weights:
            from ..formats.safetensors import load_file
            model.load_state_dict(load_file(a.weights))
        shape = ["N"] + list(desc["input"]["shape"])
        data = ox.export(model.eval(), shape)
        open(a.output, "wb").write(data)
        _out({"written": a.output, "bytes": len(data)})
    elif a.action == "run":
        module = ox.load(a.path)
        x = torch.from_numpy(np.load(a.input)) if a.input else None
        if x is None:
            raise SystemExit("--input FILE.npy is needed")
        y = module(x)
        y = y if isinstance(y, tuple) else (y,)
        for name, t in zip(module.output_names, y):
            if a.output:
                np.save(a.output if len(y) == 1 else f"{a.output}.{name}.npy", t.detach().numpy())
            _out({"output": name, "shape": list(t.shape), "mean": float(t.float().mean())})
    return 0


def _load_font(path):
    from ..imaging import TrueTypeFont
    if path:
        return TrueTypeFont(open(path, "rb").read())
    try:
        from PIL import ImageFont
        return TrueTypeFont(ImageFont.load_default(size=24).font_bytes)
    except Exception:
        raise SystemExit("no --font given and Pillow's built-in TrueType font is not available")


def cmd_page(a) -> int:
    from .. import imaging as im
    font = _load_font(a.font)
    text = open(a.text, "r", encoding="utf-8").read() if os.path.isfile(a.text) else a.text
    page = im.compose_page(font, text, a.width, a.height, a.size, margins=(a.margin,) * 4, align=a.align, device=a.device)
    image = page.image
    if a.effects:
        names = a.effects.split(",") if a.effects != "random" else None
        x = image.expand(-1, -1, 3).contiguous()[None]
        x = im.apply(x, names, a.seed, a.strength) if names else im.random_pipeline(x, a.seed, 5)
        image = x[0]
    open(a.output, "wb").write(im.encode_png(image.cpu().numpy().squeeze(-1) if image.shape[-1] == 1 else image.cpu().numpy()))
    boxes = os.path.splitext(a.output)[0] + ".words.jsonl"
    with open(boxes, "w", encoding="utf-8") as f:
        for w in page.words:
            f.write(json.dumps({"text": w.text, "box": [round(v, 2) for v in (w.x0, w.y0, w.x1, w.y1)], "line": w.line}) + "\n")
    _out({"image": a.output, "words": len(page.words), "boxes": boxes})
    return 0


def cmd_image(a) -> int:
    import torch
    from .. import imaging as im
    px = torch.from_numpy(im.decode(open(a.input, "rb").read()))
    if px.dim() == 2:
        px = px[..., None]
    if a.device:
        px = px.to(a.device)
    if a.action == "resize":
        out = im.resize(px, (a.height, a.width), a.filter)
    else:
        out = im.apply(px[None], a.effects.split(","), a.seed, a.strength)[0]
    arr = out.cpu().numpy()
    open(a.output, "wb").write(im.encode(arr[..., 0] if arr.shape[-1] == 1 else arr, os.path.splitext(a.output)[1] or "png"))
    _out({"written": a.output, "shape": list(arr.shape)})
    return 0


def cmd_audio(a) -> int:
    import numpy as np
    from .. import audio as A
    x, rate = A.read_wav(a.input)
    if a.action == "resample":
        A.write_wav(a.output, A.resample(x, rate, a.rate), a.rate)
        _out({"written": a.output, "rate": a.rate})
    else:
        mono = A.resample(x.mean(0), rate, 16000)
        feats = A.log_mel(mono, A.MelSpec.whisper(a.mels))
        np.save(a.output, feats.numpy())
        _out({"written": a.output, "shape": list(feats.shape)})
    return 0


def cmd_profile(a) -> int:
    """Profile a small training step of the tiny decoder (or of a model folder) cold and warm, with the kernel table."""
    import torch
    from ..diag.profiler import Profiler
    from ..models import DecoderSpec, build_decoder
    from ..ops import FusedAdamW
    dev = torch.device(a.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    spec = DecoderSpec.gpt2(layers=a.layers, dim=a.dim, heads=max(a.dim // 64, 1), vocab=a.vocab, max_positions=a.seq)
    model = build_decoder(spec, seed=0).to(dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
    opt = FusedAdamW(model.parameters(), lr=1e-4)
    ids = torch.randint(0, a.vocab, (a.batch, a.seq + 1), device=dev, dtype=torch.int32)

    def step():
        loss = model.loss(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
        loss.backward()
        opt.step()
        opt.zero_grad()
        return loss

    rep = Profiler.run(f"train step {a.layers}L d{a.dim} {a.batch}x{a.seq}", step, warm=a.warm)
    print({"table": rep.table, "markdown": rep.to_markdown, "csv": rep.to_csv, "json": rep.to_json}[a.format]())
    return 0


def register(add) -> None:
    p = add("profile", cmd_profile, "profile a training step: cold / warm time, memory, device time per kernel")
    p.add_argument("--layers", type=int, default=4)
    p.add_argument("--dim", type=int, default=256)
    p.add_argument("--vocab", type=int, default=1024)
    p.add_argument("--batch", type=int, default=4)
    p.add_argument("--seq", type=int, default=128)
    p.add_argument("--warm", type=int, default=5)
    p.add_argument("--device")
    p.add_argument("--format", choices=["table", "markdown", "csv", "json"], default="table")
    p = add("data", cmd_data, "convert / dedupe / split / mix / count record files (JSONL, JSON, CSV, TSV, text, Parquet)")
    p.add_argument("action", choices=["convert", "dedupe", "split", "mix", "count"])
    p.add_argument("inputs", nargs="+")
    p.add_argument("--output", "-o")
    p.add_argument("--field", default="text")
    p.add_argument("--near", action="store_true", help="also drop near-duplicates (MinHash)")
    p.add_argument("--threshold", type=float, default=0.8)
    p.add_argument("--fraction", type=float, default=0.9)
    p.add_argument("--weights")
    p.add_argument("--seed", type=int, default=0)
    p = add("index", cmd_index, "chunk text records into a retrieval index folder")
    p.add_argument("inputs", nargs="+")
    p.add_argument("--output", "-o", required=True)
    p.add_argument("--field", default="text")
    p.add_argument("--size", type=int, default=400)
    p.add_argument("--overlap", type=int, default=50)
    p = add("search", cmd_search, "BM25 search in an index folder")
    p.add_argument("index")
    p.add_argument("query")
    p.add_argument("-k", type=int, default=4)
    p = add("onnx", cmd_onnx, "inspect / run an ONNX file, or export a network description")
    p.add_argument("action", choices=["inspect", "run", "export"])
    p.add_argument("path")
    p.add_argument("--input")
    p.add_argument("--output", "-o")
    p.add_argument("--weights")
    p = add("page", cmd_page, "render a synthetic text page (PNG + word boxes), optionally with scan effects")
    p.add_argument("text", help="the text, or a file holding it")
    p.add_argument("--output", "-o", required=True)
    p.add_argument("--font")
    p.add_argument("--width", type=int, default=1240)
    p.add_argument("--height", type=int, default=1754)
    p.add_argument("--size", type=float, default=28.0)
    p.add_argument("--margin", type=float, default=60.0)
    p.add_argument("--align", choices=["left", "right", "center", "justify"], default="left")
    p.add_argument("--effects", help="comma-separated effect names, or 'random'")
    p.add_argument("--strength", type=float, default=0.5)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--device")
    p = add("image", cmd_image, "resize an image file (Pillow-exact filters) or apply scan effects")
    p.add_argument("action", choices=["resize", "effects"])
    p.add_argument("input")
    p.add_argument("--output", "-o", required=True)
    p.add_argument("--width", type=int, default=256)
    p.add_argument("--height", type=int, default=256)
    p.add_argument("--filter", default="bicubic")
    p.add_argument("--effects", default="gaussian_noise")
    p.add_argument("--strength", type=float, default=0.5)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--device")
    p = add("audio", cmd_audio, "log-mel features of a WAV file, or a resampled copy")
    p.add_argument("action", choices=["features", "resample"])
    p.add_argument("input")
    p.add_argument("--output", "-o", required=True)
    p.add_argument("--rate", type=int, default=16000)
    p.add_argument("--mels", type=int, default=80)
