"""File formats: safetensors, .ikw weights, .ikm packages, GGUF, PyTorch zip checkpoints, token files."""
from . import ikm, ikw, safetensors, tokens

__all__ = ["ikm", "ikw", "safetensors", "tokens"]


def inspect_file(path, tensors: bool = False) -> dict:
    """What a weights / package / token file holds: format, sizes, metadata and (optionally) every tensor."""
    import json
    import os
    path = str(path)
    out = {"path": path, "bytes": os.path.getsize(path) if os.path.isfile(path) else None}
    if os.path.isdir(path):
        out["kind"] = "folder"
        out["files"] = sorted(os.listdir(path))
        cfg = os.path.join(path, "config.json")
        if os.path.isfile(cfg):
            with open(cfg) as f:
                out["config"] = json.load(f)
        return out
    if path.endswith(".safetensors"):
        from .safetensors import SafeTensorsReader
        with SafeTensorsReader.open(path) as r:
            out.update(kind="safetensors", metadata=r.metadata, tensor_count=len(list(r.keys())))
            if tensors:
                out["tensors"] = {k: {"dtype": v.dtype, "shape": list(v.shape)} for k, v in r.tensors.items()}
    elif path.endswith(".gguf"):
        from .gguf import GgufFile
        g = GgufFile(path)
        meta = {k: (v if not isinstance(v, (list, tuple)) or len(v) <= 8 else f"[{len(v)} items]")
                for k, v in g.metadata.items()}
        out.update(kind="gguf", version=g.version, metadata=meta, tensor_count=len(g.tensors))
        if tensors:
            out["tensors"] = {t.name: {"type": t.type_name, "shape": list(t.shape)} for t in g.tensors.values()}
    elif path.endswith(".ikw"):
        c = ikw.read(path)
        out.update(kind="ikw", version=c.version, tensor_count=len(c.tensors))
        if tensors:
            out["tensors"] = [{"dtype": str(t.dtype), "shape": list(t.shape)} for t in c.tensors]
    elif path.endswith(".ikm"):
        with ikm.open_package(path) as r:
            out.update(kind="ikm", created=r.created, entries=[{"kind": e.kind, "name": e.name} for e in r.entries])
    elif os.path.exists(tokens.record_path(path)):
        with open(tokens.record_path(path)) as f:
            out.update(kind="tokens", record=json.load(f))
    else:
        raise ValueError(f"{path}: not a file type this package reads (.safetensors, .gguf, .ikw, .ikm, token file)")
    return out
