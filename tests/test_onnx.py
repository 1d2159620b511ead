import json
import os

import numpy as np
import pytest
import torch

from idrak_b200 import onnx as ox
from idrak_b200.nn import Network
from idrak_b200.onnx import proto as P

REF = os.environ.get("IDRAK_REFERENCE_DATA", "")


def test_protobuf_round_trip_of_every_message_kind():
    g = P.Graph("g")
    g.initializers["w"] = np.arange(6, dtype=np.float32).reshape(2, 3)
    g.initializers["i"] = np.array([-1, 2 ** 40], np.int64)
    g.initializers["s"] = np.array(3.5, np.float64)
    inner = P.Graph("body", [P.Node("Relu", ["a"], ["b"])])
    g.nodes.append(P.Node("Op", ["x", "", "w"], ["y", "z"], {"f": 0.25, "i": -7, "s": "text", "ints": [1, -2, 3], "floats": [0.5, 1.5],
                                                             "strings": ["a", "b"], "t": P.Tensor("", np.array([1, 2], np.int32)), "g": inner},
                          name="n0", domain="custom"))
    g.inputs.append(P.ValueInfo("x", P.FLOAT, ["N", 3]))
    g.outputs.append(P.ValueInfo("y", P.INT64, [2, 2]))
    m = P.Model.parse(P.Model(g, opset=17).serialize())
    assert m.opset == 17 and m.ir_version == 8 and m.producer == "idrak_b200"
    n = m.graph.nodes[0]
    assert (n.op_type, n.inputs, n.outputs, n.name, n.domain) == ("Op", ["x", "", "w"], ["y", "z"], "n0", "custom")
    a = n.attributes
    assert a["f"] == 0.25 and a["i"] == -7 and a["s"] == "text" and a["ints"] == [1, -2, 3] and a["floats"] == [0.5, 1.5]
    assert a["strings"] == [b"a", b"b"] and a["t"].array.tolist() == [1, 2] and a["g"].nodes[0].op_type == "Relu"
    assert np.array_equal(m.graph.initializers["w"], g.initializers["w"]) and m.graph.initializers["i"].tolist() == [-1, 2 ** 40]
    assert m.graph.initializers["s"].shape == () and float(m.graph.initializers["s"]) == 3.5
    assert m.graph.inputs[0].shape == ["N", 3] and m.graph.outputs[0].elem_type == P.INT64
    with pytest.raises(P.ProtoError):
        P.Model.parse(b"\x08\x01")
    with pytest.raises(P.ProtoError):
        P.Model.parse(b"\x3a\xff\x01")


def _round_trip(model, shape, ids=False, atol=1e-5):
    model.eval()
    data = ox.export(model, ["N"] + list(shape))
    module = ox.load(data)
    for batch in (1, 3):
        x = torch.randint(0, 20, (batch, *shape)) if ids else torch.randn(batch, *shape)
        with torch.no_grad():
            ref, got = model(x), module(x)
        assert got.shape == ref.shape and torch.allclose(ref, got, atol=atol), (ref - got).abs().max()
    return module


def test_export_then_import_reproduces_the_networks():
    torch.manual_seed(0)
    _round_trip(Network.input(9).linear(16).relu().linear(8).tanh().linear(3).softmax().build(), [9])
    cnn = (Network.image(3, 16, 16).conv2d(8, 3, padding=1).batch_norm().relu().max_pool2d(2).conv2d(8, 3, stride=2, padding=1, groups=2)
           .group_norm(4).gelu().upsample(2.0).avg_pool2d(2).adaptive_avg_pool2d(2).flatten().dropout(0.1).linear(5).sigmoid().build())
    cnn[1].running_mean.normal_()
    cnn[1].running_var.uniform_(0.5, 2.0)
    _round_trip(cnn, [3, 16, 16])
    seq = (Network.tokens(10).embedding(20, 16).positional().transformer(4, 32).transformer(4, 32, causal=True, norms="after")
           .rms_norm().gelu(exact=True).quick_gelu().linear(7).build())
    m = _round_trip(seq, [10], ids=True, atol=1e-4)
    assert m.input_names == ["input"] and m.output_names == ["output"]
    gap = Network.image(2, 8, 8).conv_transpose2d(4, 2, stride=2).global_avg_pool2d().linear(3).build()
    _round_trip(gap, [2, 8, 8])
    with pytest.raises(NotImplementedError, match="Recurrent"):
        ox.export(Network.sequence(4, 3).lstm(5).build(), ["N", 4, 3])


def test_runtime_operators_on_hand_made_graphs():
    g = P.Graph("ops")
    g.inputs.append(P.ValueInfo("x", P.FLOAT, [2, 3, 4]))
    g.initializers["starts"], g.initializers["ends"] = np.array([-1], np.int64), np.array([-(2 ** 62)], np.int64)
    g.initializers["axes"], g.initializers["steps"] = np.array([2], np.int64), np.array([-1], np.int64)
    g.nodes += [P.Node("Slice", ["x", "starts", "ends", "axes", "steps"], ["rev"]),
                P.Node("Shape", ["x"], ["shape"]),
                P.Node("Gather", ["shape", "starts"], ["last"], {"axis": 0}),
                P.Node("ConstantOfShape", ["last"], ["ones"], {"value": P.Tensor("", np.array([2.0], np.float32))}),
                P.Node("Mul", ["rev", "ones"], ["scaled"]),
                P.Node("ReduceSum", ["scaled", "axes"], ["sum"], {"keepdims": 0}),
                P.Node("Transpose", ["sum"], ["t"], {"perm": [1, 0]}),
                P.Node("Unsqueeze", ["t", "axes"], ["u"]),
                P.Node("Concat", ["u", "u"], ["cat"], {"axis": 2}),
                P.Node("Cast", ["cat"], ["y"], {"to": P.DOUBLE})]
    g.outputs.append(P.ValueInfo("y", P.DOUBLE, [3, 2, 2]))
    m = ox.OnnxModule(P.Model.parse(P.Model(g).serialize()))
    x = torch.arange(24.0).reshape(2, 3, 4)
    y = m(x)
    assert y.dtype == torch.float64 and y.shape == (3, 2, 2)
    assert torch.equal(y[:, :, 0], (x.flip(2) * 2).sum(2).t().double())
    bad = P.Graph("bad", [P.Node("NoSuchOp", ["x"], ["y"])])
    with pytest.raises(NotImplementedError, match="NoSuchOp"):
        ox.OnnxModule(P.Model(bad))


def test_lstm_and_gru_operators_match_the_library_layers():
    torch.manual_seed(1)
    for kind in ("lstm", "gru"):
        ref = (torch.nn.LSTM if kind == "lstm" else torch.nn.GRU)(3, 4, batch_first=False, bidirectional=True)
        H = 4
        def onnx_order(t):               # PyTorch gates: LSTM i f g o, GRU r z n -> ONNX: i o f c / z r h
            parts = t.split(H, 0)
            return torch.cat([parts[0], parts[3], parts[1], parts[2]] if kind == "lstm" else [parts[1], parts[0], parts[2]], 0)
        W = torch.stack([onnx_order(ref.weight_ih_l0), onnx_order(ref.weight_ih_l0_reverse)]).detach()
        R = torch.stack([onnx_order(ref.weight_hh_l0), onnx_order(ref.weight_hh_l0_reverse)]).detach()
        B = torch.stack([torch.cat([onnx_order(ref.bias_ih_l0), onnx_order(ref.bias_hh_l0)]),
                         torch.cat([onnx_order(ref.bias_ih_l0_reverse), onnx_order(ref.bias_hh_l0_reverse)])]).detach()
        x = torch.randn(5, 2, 3)
        attrs = {"hidden_size": H, "direction": "bidirectional"}
        if kind == "gru":
            attrs["linear_before_reset"] = 1
        out = ox.OPS[kind.upper()](attrs, x, W, R, B)
        with torch.no_grad():
            y_ref, state = ref(x)
        y = out[0].permute(0, 2, 1, 3).reshape(5, 2, 2 * H)
        assert torch.allclose(y, y_ref, atol=1e-5)
        assert torch.allclose(out[1], state[0] if kind == "lstm" else state, atol=1e-5)


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference fixtures not mounted")
def test_pytorch_exported_files_give_the_recorded_outputs():
    ref = json.load(open(os.path.join(REF, "vision-sequence", "reference.json")))
    for name, key in (("conv.onnx", "onnx_conv"), ("recurrent.onnx", "onnx_recurrent")):
        m = ox.load(os.path.join(REF, "vision-sequence", name))
        x = torch.tensor(ref[key]["input"]["values"], dtype=torch.float32).reshape(ref[key]["input"]["shape"])
        want = torch.tensor(ref[key]["output"]["values"], dtype=torch.float32).reshape(ref[key]["output"]["shape"])
        got = m(x)
        got = got[0] if isinstance(got, tuple) else got
        assert got.shape == want.shape and torch.allclose(got, want, atol=1e-5), name
