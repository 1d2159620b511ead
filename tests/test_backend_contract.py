"""Device contract, dispatcher, accountant, deferred tensors, plug-ins / kinds, .npy files and the activation scopes."""
import io
import os
import sys
import types

import numpy as np
import pytest
import torch

from idrak_b200 import core
from idrak_b200.core import backend as be
from idrak_b200.core.plugins import KindTable, LibraryDefaults, Option, OptionSchema, load_plugins
from idrak_b200.formats import npy


def test_dispatcher_prefers_plug_in_then_device_then_fallback():
    x = torch.randn(4, 8)
    w = torch.ones(8)
    want = core.run("rms_norm", x, w, 1e-6)
    assert torch.allclose(want, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6))
    with core.register_kernel("rms_norm", "cpu", lambda x, w, eps: torch.zeros_like(x)) as slot:
        assert float(core.run("rms_norm", x, w, 1e-6).abs().sum()) == 0.0
        assert [r for r in core.operation_report(be.backend_for("cpu")) if r["operation"] == "rms_norm"][0]["source"] == "plug-in"
    assert torch.equal(core.run("rms_norm", x, w, 1e-6), want)              # removed: the built-in kernel is back
    before = be.FALLBACKS.get("silu_mul", 0)
    gu = torch.randn(3, 16)
    got = core.run("silu_mul", gu)                                            # composed from another operation
    assert torch.allclose(got, torch.nn.functional.silu(gu[:, :8]) * gu[:, 8:], atol=1e-6)
    assert be.FALLBACKS["silu_mul"] == before + 1
    with pytest.raises(NotImplementedError, match="fp8_product"):
        core.run("fp8_product", x, x)                                         # fallback none: refused by name on the CPU
    with pytest.raises(KeyError, match="Known:"):
        core.run("no_such_operation", x)


def test_host_fallback_downloads_runs_and_uploads():
    class Elsewhere(be.Backend):          # a device with no kernels at all
        kind = "elsewhere"

        def __init__(self):
            super().__init__(torch.device("cpu"))
            self.moves = []

        def download(self, t):
            self.moves.append("down")
            return super().download(t)
    b = Elsewhere()
    x = torch.randn(5, 6)
    out = core.run("gelu", x, backend=b)
    assert torch.allclose(out, torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-6) and b.moves == ["down"]


def test_accountant_caps_carved_backends_and_reports_by_tag():
    b = core.create_separate_backend("cpu", cap_bytes=4096)
    t = b.allocate((256,), torch.float32, tag="weights")
    u = b.allocate((512,), torch.bfloat16, tag="cache")
    rep = b.memory_usage()
    assert rep["in_use"] == 2048 and rep["by_tag"] == {"weights": 1024, "cache": 1024} and rep["cap"] == 4096
    with pytest.raises(core.DeviceMemoryExceeded) as e:
        b.allocate((1024,), torch.float32, tag="activations")
    assert e.value.wanted == 4096 and "activations" in str(e.value)
    b.give_back(u)
    b.allocate((512,), torch.float32)
    assert b.memory_usage()["peak"] == 3072
    other = core.backend_for("cpu")
    assert other.memory_usage()["cap"] is None and other is core.backend_for("cpu")
    moved = b.copy_to(t, other)
    assert moved.shape == t.shape
    staging = b.create_host_staging(100)
    assert staging.dtype == torch.uint8 and staging.numel() == 100


def test_ranges_copies_and_evict_restore():
    b = core.backend_for("cpu")
    t = torch.arange(20.0)
    assert torch.equal(b.download_range(t, 5, 3), torch.tensor([5.0, 6.0, 7.0]))
    b.upload_range(t, 2, torch.tensor([-1.0, -2.0]))
    assert t[2] == -1 and t[3] == -2
    dst, src = torch.zeros(12), torch.arange(12.0)
    b.copy_2d(dst, src, rows=2, cols=3, dst_ld=6, src_ld=4)
    assert dst.tolist() == [0, 1, 2, 0, 0, 0, 4, 5, 6, 0, 0, 0]
    assert "memory_report" in b.capabilities and "graph_capture" not in b.capabilities


def test_deferred_tensors_read_nothing_until_moved(tmp_path):
    from idrak_b200.formats.safetensors import save_file
    a, c = torch.randn(8, 4), torch.arange(6, dtype=torch.int32)
    save_file({"layer.weight": a, "layer.ids": c, "half": a.to(torch.bfloat16)}, str(tmp_path / "m.safetensors"))
    d = core.DeferredTensors(str(tmp_path / "m.safetensors"))
    assert d.names() == ["half", "layer.ids", "layer.weight"] and d.total_bytes() == 128 + 24 + 64
    e = d.tensor("layer.weight")
    assert tuple(e.shape) == (8, 4) and e.dtype == torch.float32 and e.device == "deferred" and "Deferred" in repr(e)
    assert torch.equal(e.to("cpu"), a) and torch.equal(d.tensor("half").to("cpu", torch.float32), a.to(torch.bfloat16).float())
    got = d.materialize(["layer.ids", "layer.weight"], "cpu")
    assert torch.equal(got["layer.ids"], c)
    with torch.device("meta"):
        lin = torch.nn.Linear(4, 8, bias=False)
    assert d.load_into(lin, "cpu", prefix="layer.") == [] and torch.equal(lin.weight, a)
    with pytest.raises(KeyError):
        d.tensor("nope")
    (tmp_path / "cut.safetensors").write_bytes((tmp_path / "m.safetensors").read_bytes()[:-10])
    cut = core.DeferredTensors(str(tmp_path / "cut.safetensors"))       # the index still opens: only the data is short
    with pytest.raises(IOError, match="cut short"):
        for n in cut.names():
            cut.tensor(n).to("cpu")


def test_device_names():
    D = core.Device
    assert D.parse("cpu") == torch.device("cpu") and D.parse("gpu:1") == torch.device("cuda", 1)
    assert D.parse("CUDA:3").index == 3 and D.default().type in ("cpu", "cuda")
    assert D.available()[0] == torch.device("cpu")
    with pytest.raises(ValueError, match="Known"):
        D.parse("tpu:0")
    assert D.backend("cpu").kind == "cpu"


def test_option_schema_kinds_defaults_and_plugins(monkeypatch):
    schema = OptionSchema(Option("rate", float, 0.1, minimum=0.0, maximum=1.0), Option("mode", str, "a", choices=("a", "b")),
                          Option("steps", int, required=True), Option("on", bool, False))
    assert schema.validate({"steps": "5", "rate": 1, "on": "yes"}, "thing") == {"rate": 1.0, "mode": "a", "steps": 5, "on": True}
    for bad, err in (({"steps": 1, "rat": 2}, KeyError), ({}, KeyError), ({"steps": 1, "mode": "c"}, ValueError),
                     ({"steps": 1, "rate": 2.0}, ValueError), ({"steps": "x"}, ValueError), ({"steps": 1.5}, ValueError)):
        with pytest.raises(err):
            schema.validate(bad, "thing")
    kinds = KindTable("schedule", lambda t: t.register("constant", lambda value: ("constant", value),
                                                       OptionSchema(Option("value", float, 1.0)), "fallback"))
    assert kinds.create("constant") == ("constant", 1.0) and kinds.kinds() == ["constant"]
    kinds.register("constant", lambda value: ("mine", value), OptionSchema(Option("value", float, 2.0)))
    assert kinds.create("constant") == ("mine", 2.0)                       # a shadow registration wins over the default
    with pytest.raises(KeyError, match="Known: constant"):
        kinds.create("cosine")
    ran = []
    LibraryDefaults.add("test-registry", lambda: ran.append(1))
    assert ran == []
    LibraryDefaults.ensure("test-registry")
    LibraryDefaults.ensure("test-registry")
    assert ran == [1] and "test-registry" in LibraryDefaults.ensured()
    mod = types.ModuleType("idrak_test_plugin")
    mod.name = "test plug-in"
    mod.register = lambda api: api.register_kernel("add", "cpu", lambda a, b: a - b)
    monkeypatch.setitem(sys.modules, "idrak_test_plugin", mod)
    assert load_plugins(["idrak_test_plugin"]) == ["test plug-in"] and load_plugins(["idrak_test_plugin"]) == []
    try:
        assert float(core.run("add", torch.ones(2), torch.ones(2)).sum()) == 0.0
    finally:
        for slot in list(be.PLUGIN_KERNELS._slots.get(("add", "cpu"), [])):
            slot.remove()
    empty = types.ModuleType("idrak_empty_plugin")
    monkeypatch.setitem(sys.modules, "idrak_empty_plugin", empty)
    with pytest.raises(AttributeError, match="register"):
        load_plugins(["idrak_empty_plugin"])


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.float16, np.int64, np.int32, np.int8, np.uint8, np.bool_])
def test_npy_round_trips_with_numpy(tmp_path, dtype):
    a = (np.random.RandomState(0).randn(3, 4, 5) * 10).astype(dtype)
    p = str(tmp_path / "a.npy")
    np.save(p, a)
    assert torch.equal(npy.load_npy(p), torch.from_numpy(a))
    np.save(p, np.asfortranarray(a))
    assert torch.equal(npy.load_npy(p), torch.from_numpy(a))
    npy.save_npy(torch.from_numpy(a), p)
    assert np.array_equal(np.load(p), a)
    assert np.array_equal(np.load(io.BytesIO(npy.save_npy(torch.from_numpy(a[0, 0])))), a[0, 0])


def test_npy_big_endian_npz_and_refusals(tmp_path):
    a = np.arange(10, dtype=">f4").reshape(2, 5)
    p = str(tmp_path / "be.npy")
    np.save(p, a)
    assert torch.equal(npy.load_npy(p), torch.arange(10.0).reshape(2, 5))
    npy.save_npz({"x": torch.ones(3), "y": torch.zeros(2, 2, dtype=torch.int64)}, str(tmp_path / "z.npz"), compress=True)
    z = np.load(str(tmp_path / "z.npz"))
    assert z["x"].tolist() == [1, 1, 1] and npy.load_npz(str(tmp_path / "z.npz"))["y"].shape == (2, 2)
    assert npy.load_npy(npy.save_npy(torch.ones(2, dtype=torch.bfloat16))).dtype == torch.float32
    with pytest.raises(ValueError, match="magic"):
        npy.load_npy(b"not numpy at all")
    with pytest.raises(ValueError, match="cut short"):
        npy.load_npy(npy.save_npy(torch.ones(100))[:-8])
    np.save(p, np.zeros(2, dtype=[("a", "f4"), ("b", "i4")]))
    with pytest.raises(ValueError, match="structured"):
        npy.load_npy(p)


def test_saved_activations_compressed_to_bfloat16_and_recomputed_parts():
    lin = torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.GELU(), torch.nn.Linear(64, 64))
    x = torch.randn(128, 64, requires_grad=True)
    lin(x).sum().backward()
    want = x.grad.clone()
    x.grad = None
    with core.compress_saved_to_bfloat16(min_elements=256) as scope:
        y = lin(x).sum()
    y.backward()
    assert scope.stats["tensors"] >= 2 and scope.stats["bytes_saved"] >= 2 * 128 * 64 * 2
    assert torch.allclose(x.grad, want, atol=2e-2, rtol=2e-2) and not torch.equal(x.grad, want)
    from idrak_b200.models import DecoderSpec, build_decoder
    model = build_decoder(DecoderSpec.llama(layers=2, dim=32, heads=2, kv_heads=2, ff_dim=64, vocab=50, max_positions=16), seed=0)
    ids = torch.randint(0, 50, (2, 8))
    model.loss(ids, ids).backward()
    ref = model.blocks[0].mlp.up_weight.grad.clone()
    model.zero_grad()
    calls = {"n": 0}
    original = model.blocks[0].mlp.forward.__func__

    def counting(self, *a, **k):
        calls["n"] += 1
        return original(self, *a, **k)
    model.blocks[0].mlp.forward = types.MethodType(counting, model.blocks[0].mlp)
    with core.recompute(model, "feed_forward"):
        loss = model.loss(ids, ids)
    loss.backward()
    assert calls["n"] == 2, "once forward, once again in backward"
    assert torch.allclose(model.blocks[0].mlp.up_weight.grad, ref, atol=1e-6)
    with pytest.raises(ValueError):
        with core.recompute(model, "everything"):
            pass


def test_tensor_scope_frees_what_it_owns_and_keeps_what_is_taken_out():
    with core.TensorScope() as scope:
        a = scope.own(torch.ones(1000))
        b = scope.keep(scope.own(torch.ones(1000)))
    assert a.untyped_storage().nbytes() == 0 and b.untyped_storage().nbytes() == 4000 and float(b.sum()) == 1000.0
