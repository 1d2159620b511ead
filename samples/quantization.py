"""Weight quantisation of a decoder: pack the projection matrices of every block to int8 or int4 (group scales),
compare the logits and the memory with the bf16 model, and save / reload the packed model. Needs a B200.

    python samples/quantization.py --kind int4

Reference: samples/Idrak.Samples.Quantization/Program.cs.
"""
import argparse
import copy
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from idrak_b200.models import DecoderSpec, build_decoder  # noqa: E402
from idrak_b200.quant import load_packed, quantize_model, save_packed  # noqa: E402


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", choices=["int8", "int4"], default="int4")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--dim", type=int, default=1024)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("this sample runs the packed-weight kernels and needs a GPU")
    torch.manual_seed(0)
    spec = DecoderSpec.llama(layers=a.layers, dim=a.dim, heads=a.dim // 128, kv_heads=max(1, a.dim // 512), ff_dim=4 * a.dim,
                             vocab=32000, max_positions=2048)
    dense = build_decoder(spec).to("cuda", torch.bfloat16).eval()
    packed = copy.deepcopy(dense)
    count = quantize_model(packed, a.kind)
    ids = torch.randint(0, 32000, (2, 256), device="cuda")
    with torch.no_grad():
        ref, out = dense(ids).float(), packed(ids).float()
    rel = float((out - ref).norm() / ref.norm())
    agree = float((out.argmax(-1) == ref.argmax(-1)).float().mean())

    def megabytes(m):
        seen, total = set(), 0
        for t in list(m.parameters()) + list(m.buffers()):
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total / 2 ** 20
    with tempfile.TemporaryDirectory() as folder:
        save_packed(packed, folder)
        again = load_packed(folder)
        with torch.no_grad():
            same = torch.equal(again(ids).float(), out)
        on_disk = sum(os.path.getsize(os.path.join(folder, f)) for f in os.listdir(folder)) / 2 ** 20
    print(f"{count} matrices packed to {a.kind}; relative logit error {rel:.4f}; top-1 agreement {100 * agree:.1f} %")
    print(f"dense parameters {megabytes(dense):.0f} MiB; packed folder {on_disk:.0f} MiB; reload identical: {same}")
    return {"relative_error": rel, "agreement": agree, "reload_identical": same}


if __name__ == "__main__":
    main()
