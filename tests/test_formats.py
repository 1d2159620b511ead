"""safetensors / .ikw / .ikm / token files / PEFT folders: round trips and the reference's own fixtures."""
import gzip
import io
import json
import os
import shutil
import struct

import numpy as np
import pytest
import torch

from idrak_b200.adapters import add_adapters, merge_adapters, named_adapters
from idrak_b200.adapters import peft
from idrak_b200.formats import ikm, ikw, tokens
from idrak_b200.formats.safetensors import SafeTensorsReader, load_file, save_file, save_sharded
from idrak_b200.models import DecoderSpec, build_decoder
from idrak_b200.models.checkpoint import (from_hf_tensors, idrak_tensors, load_idrak_tensors, to_hf_tensors)

# folder of the reference project's test data (its tests/Idrak.Tests/data); tests that read it skip when it is not given
REF = os.environ.get("IDRAK_REFERENCE_DATA", "")
needs_ref = pytest.mark.skipif(not os.path.isdir(REF), reason="IDRAK_REFERENCE_DATA does not name the fixture folder")


def test_safetensors_round_trip_all_float_types(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.randn(2, 2).to(torch.float16),
         "i": torch.arange(6, dtype=torch.int32).reshape(2, 3), "e": torch.zeros(0, 4)}
    p = tmp_path / "x.safetensors"
    save_file(t, p, metadata={"format": "pt", "k": "v"})
    with SafeTensorsReader.open(p) as r:
        assert r.metadata == {"format": "pt", "k": "v"}
        assert set(r.keys()) == set(t)
        for k, v in t.items():
            got = r.read(k)
            assert got.dtype == v.dtype and torch.equal(got, v)
    # header is 8-byte aligned and offsets are contiguous
    raw = p.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    assert n % 8 == 0
    header = json.loads(raw[8:8 + n])
    assert header["a"]["dtype"] == "F32" and header["b"]["dtype"] == "BF16"


def test_safetensors_sharded_index(tmp_path):
    t = {f"w{i}": torch.randn(64, 64) for i in range(6)}
    files = save_sharded(t, tmp_path, max_shard_bytes=40000)
    assert len(files) > 1 and (tmp_path / "model.safetensors.index.json").exists()
    with SafeTensorsReader.open(tmp_path) as r:
        assert set(r.keys()) == set(t)
        assert torch.equal(r.read("w3"), t["w3"])


def test_safetensors_quantized_scales_are_applied_and_hidden(tmp_path):
    w = torch.randint(-127, 128, (8, 16), dtype=torch.int8)
    scale = torch.rand(8) + 0.5
    zp = torch.full((8,), 3.0)
    f8 = torch.randn(256, 256).to(torch.float8_e4m3fn)
    blk = torch.rand(2, 2) + 0.5
    save_file({"l.weight": w, "l.weight_scale": scale, "l.weight_zero_point": zp, "m.weight": f8,
               "m.weight_scale_inv": blk, "m.input_scale": torch.ones(1), "lonely": torch.zeros(2, dtype=torch.int8)},
              tmp_path / "q.safetensors")
    with SafeTensorsReader.open(tmp_path / "q.safetensors") as r:
        assert set(r.keys()) == {"l.weight", "m.weight"}
        assert r.quantization_scales["m.input_scale"] == "activations"
        assert "lonely" in r.left_out
        expect = (w.float() - zp[:, None]) * scale[:, None]
        assert torch.allclose(r.read("l.weight"), expect)
        expect_m = f8.float() * blk.repeat_interleave(128, 0).repeat_interleave(128, 1)
        assert torch.allclose(r.read("m.weight"), expect_m)


@needs_ref
def test_reference_f8_i8_fixture_reads(tmp_path):
    src = os.path.join(REF, "safetensors", "f8-i8.safetensors.gz")
    dst = tmp_path / "f8-i8.safetensors"
    with gzip.open(src, "rb") as f, open(dst, "wb") as g:
        shutil.copyfileobj(f, g)
    with SafeTensorsReader.open(dst) as r:
        assert len(r.tensors) > 0
        names = set(r.tensors)
        assert "e4m3.all" in names
        codes = r.read_float("e4m3.all")            # every one of the 256 codes: two of them are NaN
        assert codes.numel() == 256 and int(torch.isnan(codes).sum()) == 2
        assert codes[1].item() == 2.0 ** -9 and codes[0x7E].item() == 448.0
        for name in names:
            assert r.read_float(name).numel() > 0


def test_ikw_versions_round_trip(tmp_path):
    ts = [torch.randn(4, 3), torch.randn(5), torch.randn(2, 2, 2)]
    for fmt, tol in ((ikw.FLOAT32, 0.0), (ikw.FLOAT16, 1e-2), (ikw.BFLOAT16, 5e-2)):
        p = tmp_path / f"f{fmt}.ikw"
        ikw.write(p, ts, fmt, exact=[False, True, False], int8_layers=[1], bfloat16_layers=[0], int4_layers=[2],
                  bfloat16_embeddings=[0])
        c = ikw.read(p)
        assert c.version == 5 and c.int8_layers == [1] and c.bfloat16_layers == [0] and c.int4_layers == [2]
        assert c.bfloat16_embeddings == [0]
        assert c.formats == [fmt, ikw.FLOAT32, fmt]
        assert torch.equal(c.tensors[1], ts[1])                     # exact tensors keep their bits
        for a, b in zip(c.tensors, ts):
            assert a.shape == b.shape and (a - b).abs().max().item() <= tol
    ikw.write(tmp_path / "v2.ikw", ts, version=2)
    raw = (tmp_path / "v2.ikw").read_bytes()
    assert raw[:4] == b"IKW2" and struct.unpack("<i", raw[4:8])[0] == 3
    assert all(torch.equal(a, b) for a, b in zip(ikw.read(tmp_path / "v2.ikw").tensors, ts))
    ikw.write(tmp_path / "v3.ikw", ts)
    assert (tmp_path / "v3.ikw").read_bytes()[:4] == b"IKW3"


def test_decoder_checkpoint_layouts_round_trip(tmp_path):
    for spec in (DecoderSpec.tiny_gpt(),
                 DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=96, vocab=100, max_positions=32)):
        m = build_decoder(spec, seed=3)
        named = idrak_tensors(m)
        assert named["embed.weight"].shape == (spec.vocabulary, spec.dim)
        assert named["layers.0.attn.q.weight"].shape == (spec.dim, spec.heads * spec.head_dim)     # [in, out]
        m2 = build_decoder(spec, seed=4)
        load_idrak_tensors(m2, named)
        ids = torch.randint(0, spec.vocabulary, (2, 8))
        assert torch.equal(m(ids), m2(ids))
        # .ikw of the whole module
        ikw.save_module(m, tmp_path / "m.ikw")
        m3 = build_decoder(spec, seed=5)
        ikw.load_module(m3, tmp_path / "m.ikw")
        assert torch.equal(m(ids), m3(ids))
        # Hugging Face naming
        style = "gpt2" if spec.learned_positions else "llama"
        hf = to_hf_tensors(m, style)
        m4 = build_decoder(spec, seed=6)
        load_idrak_tensors(m4, from_hf_tensors(spec, hf, style))
        assert torch.equal(m(ids), m4(ids))
    with pytest.raises(ValueError):
        ikw.load_module(build_decoder(DecoderSpec.tiny_gpt()), tmp_path / "m.ikw")


def test_ikm_package_round_trip(tmp_path):
    spec = DecoderSpec.tiny_gpt()
    m = build_decoder(spec, seed=1)
    path = tmp_path / "model.ikm"
    ikm.create(path).model(m).json({"a": 1}, "info").text("hello", "readme").tokenizer({"type": "byte"}).save()
    import zipfile
    with zipfile.ZipFile(path) as z:
        names = set(z.namelist())
        man = json.loads(z.read("manifest.json"))
    assert man["format"] == "idrak-package/1"
    assert {"weights/model.ikw", "architecture/model.json", "json/info.json", "text/readme.txt",
            "tokenizers/model.json", "manifest.json"} <= names
    assert {"kind": "Weights", "name": "model", "file": "weights/model.ikw"} in man["entries"]
    with ikm.open_package(path) as r:
        assert r.json("info") == {"a": 1} and r.text("readme") == "hello"
        m2 = r.build_model()
    ids = torch.randint(0, 256, (1, 16))
    assert torch.equal(m(ids), m2(ids))


def test_ikm_trainable_entry_is_the_indexed_parameter_file(tmp_path):
    """``trainable/NAME.nsp``: u32 'IKP1', i32 count, then per tensor its index among the parameters, rank, dims and
    float32 values - checked on load against the model's index range and shapes."""
    import struct
    import zipfile
    lin = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    for q in lin[0].parameters():
        q.requires_grad_(False)
    path = tmp_path / "t.ikm"
    ikm.create(path).trainable_weights(lin, "head").save()
    with zipfile.ZipFile(path) as z:
        raw = z.read("trainable/head.nsp")
    magic, count = struct.unpack_from("<Ii", raw, 0)
    assert magic == 0x31504B49 and count == 2
    index, rank, d0, d1 = struct.unpack_from("<iiii", raw, 8)
    assert (index, rank, d0, d1) == (2, 2, 2, 3)
    first = struct.unpack_from("<6f", raw, 24)
    assert list(first) == [float(x) for x in lin[1].weight.detach().reshape(-1)]
    other = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    with ikm.open_package(path) as r:
        r.load_trainable(other, "head")                      # requires_grad of the target plays no part
    assert torch.equal(other[1].weight, lin[1].weight) and torch.equal(other[1].bias, lin[1].bias)
    assert not torch.equal(other[0].weight, lin[0].weight)
    wrong = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 5))
    with ikm.open_package(path) as r, pytest.raises(ValueError, match="Parameter 2: file has"):
        r.load_trainable(wrong, "head")
    small = torch.nn.Sequential(torch.nn.Linear(4, 3))
    with ikm.open_package(path) as r, pytest.raises(ValueError, match="refers to parameter 2"):
        r.load_trainable(small, "head")
    with pytest.raises(ValueError, match="magic IKP1"):
        ikm.load_trainable_bytes(lin, b"IKW3" + raw[4:])


def test_ikm_entry_names_and_paths_are_unique(tmp_path):
    w = ikm.create(tmp_path / "p.ikm").scaler("StandardScaler", "0 1", "x")
    with pytest.raises(ValueError, match="already has"):
        w.scaler("MinMaxScaler", "0 1", "x")                 # both would be scalers/x.txt
    for bad in ("a/b", "a\\b"):
        with pytest.raises(ValueError, match="cannot contain"):
            w.text("t", bad)


def test_token_file_record_and_windows(tmp_path):
    ids = np.arange(1000) % 300
    rec = tokens.write_tokens(tmp_path / "t.bin", ids, vocabulary=300, documents=3, separator=2)
    assert rec["type"] == "uint16" and rec["format"] == "idrak-tokens/1"
    tf = tokens.TokenFile(tmp_path / "t.bin", length=64)
    x, y = tf.window(2)
    assert torch.equal(x[1:], y[:-1]) and x[0].item() == (128 % 300)
    assert len(tf) == (1000 - 65) // 64 + 1
    assert tokens.parse_type("u16") == "uint16" and tokens.parse_type("Int32") == "int32"
    with pytest.raises(ValueError):
        tokens.parse_type("float32")


@needs_ref
def test_reference_token_fixture():
    tf = tokens.TokenFile(os.path.join(REF, "pretrain", "tokens.bin"), length=32)
    assert tf.record["tokens"] == 25422 and tf.ids.shape[0] == 25422 and int(tf.ids.max()) < 512


def test_peft_folder_round_trip_and_refusals(tmp_path):
    spec = DecoderSpec.llama(layers=2, dim=64, heads=4, kv_heads=2, ff_dim=96, vocab=100, max_positions=32)
    for dora in (False, True):
        m = build_decoder(spec, seed=2)
        ps = add_adapters(m, rank=4, alpha=8, dora=dora)
        with torch.no_grad():
            for p in ps:
                p.add_(torch.randn_like(p) * 0.05)
        folder = tmp_path / f"ad{int(dora)}"
        peft.save_adapters(m, folder, "base")
        cfg = json.loads((folder / "adapter_config.json").read_text())
        assert cfg["peft_type"] == "LORA" and cfg["r"] == 4 and cfg["use_dora"] == dora and cfg["bias"] == "none"
        sd = load_file(folder / "adapter_model.safetensors")
        key = "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight"
        assert sd[key].shape == (4, 64) and sd[key].dtype == torch.float32
        assert sd["base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight"].shape == (64, 4)
        assert ("base_model.model.model.layers.0.self_attn.q_proj.lora_magnitude_vector" in sd) == dora
        m2 = build_decoder(spec, seed=2)
        got = peft.load_adapters(m2, folder)
        assert got["loaded_modules"] == 14
        ids = torch.randint(0, 100, (2, 8))
        assert torch.allclose(m(ids), m2(ids), atol=1e-6)
        merge_adapters(m2)
        assert torch.allclose(m(ids), m2(ids), atol=1e-5)
    bad = tmp_path / "bad"
    shutil.copytree(tmp_path / "ad0", bad)
    cfg = json.loads((bad / "adapter_config.json").read_text())
    for key, val, word in (("rank_pattern", {"q_proj": 8}, "rank_pattern"), ("bias", "all", "bias"),
                           ("use_qalora", True, "use_qalora"), ("peft_type", "IA3", "peft_type")):
        c2 = dict(cfg)
        c2[key] = val
        (bad / "adapter_config.json").write_text(json.dumps(c2))
        with pytest.raises(NotImplementedError, match=word):
            peft.read_config(bad)
    c3 = dict(cfg)
    c3["use_dora"] = True
    (bad / "adapter_config.json").write_text(json.dumps(c3))
    with pytest.raises(peft.PeftConfigError, match="lora_magnitude_vector"):
        peft.load_adapters(build_decoder(spec, seed=2), bad)


def test_pth_reader_is_an_allow_list_unpickler_of_its_own(tmp_path):
    """Tensors (views, scalars, bf16, parameters) come back equal; a pickle that wants to call anything else is refused
    by name before anything runs."""
    import collections
    import os
    from idrak_b200.formats import pth
    sd = collections.OrderedDict(a=torch.randn(3, 4), b=torch.arange(6).reshape(2, 3).t(), c=torch.tensor(2.5),
                                 d=torch.randn(4).to(torch.bfloat16), e=torch.nn.Parameter(torch.ones(2)))
    sd["module.view"] = sd["a"][1:, :2]
    torch.save({"state_dict": sd, "epoch": 3}, tmp_path / "m.pth")
    got = pth.load_checkpoint(tmp_path / "m.pth")
    assert set(got) == {"a", "b", "c", "d", "e", "view"}
    for k, v in sd.items():
        assert torch.equal(got[k.replace("module.", "")], v.detach())
    marker = tmp_path / "ran"

    class Evil:
        def __reduce__(self):
            return (os.system, (f"touch {marker}",))
    torch.save({"x": Evil()}, tmp_path / "evil.pth")
    with pytest.raises(pth.UnsafeCheckpoint, match="system"):
        pth.load_checkpoint(tmp_path / "evil.pth")
    assert not marker.exists()
    torch.save([1, 2], tmp_path / "list.pth")
    with pytest.raises(ValueError, match="not a mapping"):
        pth.load_checkpoint(tmp_path / "list.pth")
