"""The dw-conv -> BN(inference) -> quantizer graph pass: pattern matching on CPU, and on the
GPU the fused graph against the unfused graph and the oracle."""
import numpy as np
import pytest

from dwbnq import graph


def _chain(quant_op="FixedPointQuantize", quant_args=None, bn_args=None, extra_consumer=False):
    nodes = [
        {"op": "DepthwiseConvolution", "inputs": ["x", "w", "b"], "outputs": ["c"],
         "args": {"base_axis": 1, "pad": (1, 1), "stride": (1, 1), "dilation": (1, 1), "multiplier": 1}},
        {"op": "BatchNormalization", "inputs": ["c", "beta", "gamma", "mean", "var"], "outputs": ["n"],
         "args": dict({"axes": [1], "decay_rate": 0.9, "eps": 1e-5, "batch_stat": False}, **(bn_args or {}))},
    ]
    if quant_op == "MinMaxQuantize":
        nodes.append({"op": quant_op, "inputs": ["n", "qr_min", "qr_max", "ql_min", "ql_max"], "outputs": ["y"],
                      "args": quant_args or {"decay": 0.999, "x_min_max": True, "ema": False, "eps": 0.01}})
    elif quant_op:
        nodes.append({"op": quant_op, "inputs": ["n"], "outputs": ["y"], "args": quant_args or {}})
    if extra_consumer:
        nodes.append({"op": "FixedPointQuantize", "inputs": ["n"], "outputs": ["z"], "args": {}})
    return nodes


def _mm_shapes(c=8, per_channel=True):
    r = (1, c, 1, 1) if per_channel else (1, 1, 1, 1)
    return {"x": (2, c, 14, 14), "w": (c, 3, 3), "qr_min": r, "qr_max": r, "ql_min": r, "ql_max": r}


def test_chain_is_fused_into_one_node():
    for op in ("FixedPointQuantize", "Pow2Quantize", "MinMaxQuantize"):
        fused = graph.fuse_dw_bn_quant(_chain(op), graph_outputs=["y"], shapes=_mm_shapes())
        assert [n["op"] for n in fused] == [graph.FUSED]
        f = fused[0]
        assert f["outputs"] == ["y"] and f["quant"]["op"] == op
        assert f["inputs"][:3] == ["x", "w", "b"] and f["inputs"][3:7] == ["beta", "gamma", "mean", "var"]
    # conv -> BN without a quantizer is fused with quantizer None
    fused = graph.fuse_dw_bn_quant(_chain(None), graph_outputs=["n"])
    assert [n["op"] for n in fused] == [graph.FUSED] and fused[0]["quant"] is None


def test_patterns_that_must_not_fuse():
    # training-mode BN
    g = graph.fuse_dw_bn_quant(_chain(bn_args={"batch_stat": True}), ["y"])
    assert [n["op"] for n in g] == ["DepthwiseConvolution", "BatchNormalization", "FixedPointQuantize"]
    # BN over another axis
    g = graph.fuse_dw_bn_quant(_chain(bn_args={"axes": [2]}), ["y"])
    assert g[0]["op"] == "DepthwiseConvolution"
    # the BN output has a second consumer: conv+BN fuse, the quantizers stay
    g = graph.fuse_dw_bn_quant(_chain(extra_consumer=True), ["y", "z"])
    assert [n["op"] for n in g] == [graph.FUSED, "FixedPointQuantize", "FixedPointQuantize"]
    assert g[0]["quant"] is None and g[0]["outputs"] == ["n"]
    # the conv output is itself a graph output: nothing fuses
    g = graph.fuse_dw_bn_quant(_chain(), ["y", "c"])
    assert [n["op"] for n in g] == ["DepthwiseConvolution", "BatchNormalization", "FixedPointQuantize"]
    # the BN output is a graph output: the quantizer is not absorbed
    g = graph.fuse_dw_bn_quant(_chain(), ["y", "n"])
    assert [n["op"] for n in g] == [graph.FUSED, "FixedPointQuantize"]
    # MinMaxQuantize with per-tensor ranges ([1,1,1,1]) or with unknown range shapes: the fused
    # kernel is per-channel, so the quantizer stays its own node behind the fused conv + BN
    for shapes in (_mm_shapes(per_channel=False), None, {"w": (8, 3, 3)}):
        g = graph.fuse_dw_bn_quant(_chain("MinMaxQuantize"), ["y"], shapes=shapes)
        assert [n["op"] for n in g] == [graph.FUSED, "MinMaxQuantize"], shapes
        assert g[0]["quant"] is None and g[0]["outputs"] == ["n"] and g[1]["inputs"][0] == "n"
    # a bare [C] range vector counts as per-channel
    v = dict(_mm_shapes(), qr_min=(8,), qr_max=(8,), ql_min=(8,), ql_max=(8,))
    assert [n["op"] for n in graph.fuse_dw_bn_quant(_chain("MinMaxQuantize"), ["y"], shapes=v)] == [graph.FUSED]
    # unrelated nodes pass through untouched and in order
    other = {"op": "ReLU6", "inputs": ["y"], "outputs": ["r"], "args": {}}
    g = graph.fuse_dw_bn_quant(_chain() + [other], ["r"])
    assert [n["op"] for n in g] == [graph.FUSED, "ReLU6"]


class _FakeNnabla:
    """The surface of nnabla that from_nnabla touches: Variable.visit(callback) walks the
    functions in forward order; a function has info.type_name, info.args, inputs, outputs;
    a variable has shape."""

    class Variable:
        def __init__(self, shape, parent=None):
            self.shape, self.parent = tuple(shape), parent

        def visit(self, f):
            seen, order = set(), []

            def walk(v):
                fn = v.parent
                if fn is None or id(fn) in seen:
                    return
                seen.add(id(fn))
                for i in fn.inputs:
                    walk(i)
                order.append(fn)

            walk(self)
            for fn in order:
                f(fn)

    class Function:
        def __init__(self, type_name, args, inputs, out_shape):
            import types
            self.info = types.SimpleNamespace(type_name=type_name, args=args)
            self.inputs = list(inputs)
            self.outputs = [_FakeNnabla.Variable(out_shape, parent=self)]


def test_from_nnabla_walks_a_graph_and_the_result_fuses(monkeypatch):
    import sys
    import types
    monkeypatch.setitem(sys.modules, "nnabla", types.ModuleType("nnabla"))
    V, F = _FakeNnabla.Variable, _FakeNnabla.Function
    c = 8
    for per_channel in (True, False):
        r = (1, c, 1, 1) if per_channel else (1, 1, 1, 1)
        x, w, b = V((2, c, 14, 14)), V((c, 3, 3)), V((c,))
        beta, gamma, mean, var = (V((1, c, 1, 1)) for _ in range(4))
        qr_min, qr_max, ql_min, ql_max = (V(r) for _ in range(4))
        conv = F("DepthwiseConvolution", {"base_axis": 1, "pad": [1, 1], "stride": [1, 1], "dilation": [1, 1],
                                          "multiplier": 1}, [x, w, b], (2, c, 14, 14))
        bn = F("BatchNormalization", {"axes": [1], "decay_rate": 0.9, "eps": 1e-5, "batch_stat": False,
                                      "no_scale": False, "no_bias": False},
               [conv.outputs[0], beta, gamma, mean, var], (2, c, 14, 14))
        q = F("MinMaxQuantize", {"decay": 0.999, "x_min_max": True, "ema": False, "ste_fine_grained": True,
                                 "eps": 0.01}, [bn.outputs[0], qr_min, qr_max, ql_min, ql_max], (2, c, 14, 14))
        relu = F("ReLU6", {}, [q.outputs[0]], (2, c, 14, 14))
        nodes, names, shapes = graph.from_nnabla(relu.outputs[0])
        assert [n["op"] for n in nodes] == ["DepthwiseConvolution", "BatchNormalization", "MinMaxQuantize", "ReLU6"]
        assert nodes[0]["inputs"] == [names[x], names[w], names[b]] and nodes[2]["args"]["x_min_max"] is True
        assert shapes[names[w]] == (c, 3, 3) and shapes[names[qr_min]] == r
        fused = graph.fuse_dw_bn_quant(nodes, [names[relu.outputs[0]]], shapes=shapes)
        if per_channel:
            assert [n["op"] for n in fused] == [graph.FUSED, "ReLU6"]
            assert fused[0]["inputs"][-4:] == [names[v] for v in (qr_min, qr_max, ql_min, ql_max)]
            assert fused[0]["outputs"] == nodes[2]["outputs"]
        else:
            assert [n["op"] for n in fused] == [graph.FUSED, "MinMaxQuantize", "ReLU6"]


def test_from_nnabla_needs_nnabla():
    with pytest.raises(ImportError):
        graph.from_nnabla(object())


@pytest.mark.gpu
def test_fused_graph_equals_unfused_graph_and_oracle(oracle, cuda_device):
    import torch
    from dwbnq import workloads
    for spec, qop, qargs in (
            (workloads.cfg0(n=3)[0], "FixedPointQuantize", {"sign": True, "n": 8, "delta": 2.0 ** -4}),
            (workloads.cfg2(n=2)[0], "Pow2Quantize", {"sign": True, "with_zero": True, "n": 8, "m": 1}),
            (workloads.cfg3(n=6)[0], "MinMaxQuantize", {"decay": 0.999, "x_min_max": True, "ema": False, "eps": 0.01})):
        d = workloads.make_layer_data(spec)
        nodes = _chain(qop, qargs)
        nodes[0]["args"].update(pad=(spec.pad,) * 2, stride=(spec.stride,) * 2)
        names = ["x", "w", "b", "beta", "gamma", "mean", "var"] + (
            ["qr_min", "qr_max", "ql_min", "ql_max"] if qop == "MinMaxQuantize" else [])

        def fresh():
            return {k: torch.from_numpy(d[k].copy()).to(cuda_device) for k in names}

        t_unfused = graph.execute(nodes, fresh())
        fused = graph.fuse_dw_bn_quant(nodes, ["y"], shapes={k: tuple(d[k].shape) for k in names})
        assert len(fused) == 1
        t_fused = graph.execute(fused, fresh())
        assert torch.equal(t_unfused["y"].view(torch.int32), t_fused["y"].view(torch.int32)), spec.name
        q = workloads.quant_for_ops(spec, d)
        want = oracle.fused_layer(d["x"], d["w"], d["b"], d["beta"], d["gamma"], d["mean"], d["var"], 1e-5,
                                  (spec.stride,) * 2, (spec.pad,) * 2, q, nthreads=oracle.max_threads())
        if qop == "MinMaxQuantize":
            want, qmin, qmax = want
            np.testing.assert_array_equal(t_fused["qr_min"].cpu().numpy(), qmin)
            np.testing.assert_array_equal(t_fused["qr_max"].cpu().numpy(), qmax)
        got = t_fused["y"].cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), spec.name


@pytest.mark.gpu
def test_graph_runner_replays_the_fused_layers(oracle, cuda_device):
    """The fused node list captured into a CUDA graph: replays reproduce the eager result,
    also after the input tensor has been overwritten in place."""
    import torch
    from dwbnq import workloads
    spec = workloads.cfg1(n=2)[6]  # 28x28 stride 2
    d = workloads.make_layer_data(spec)
    nodes = graph.fuse_dw_bn_quant(_chain("FixedPointQuantize", {"sign": False, "n": 8, "delta": 2.0 ** -3}), ["y"])
    nodes[0]["conv_args"].update(pad=(spec.pad,) * 2, stride=(spec.stride,) * 2)
    names = ["x", "w", "b", "beta", "gamma", "mean", "var"]
    t = {k: torch.from_numpy(d[k].copy()).to(cuda_device) for k in names}
    runner = graph.GraphRunner(nodes, t)
    q = {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}
    for scale in (1.0, -0.5):
        x = (d["x"] * np.float32(scale)).astype(np.float32)
        t["x"].copy_(torch.from_numpy(x))
        out = runner.replay()
        torch.cuda.synchronize()
        want = oracle.fused_layer(x, d["w"], d["b"], d["beta"], d["gamma"], d["mean"], d["var"], 1e-5,
                                  (spec.stride,) * 2, (spec.pad,) * 2, q, nthreads=oracle.max_threads())
        got = out["y"].cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), scale


def _pw_chain(act="ReLU6", quant_op="FixedPointQuantize", quant_args=None, conv_args=None, extra_consumer=None):
    nodes = [
        {"op": "Convolution", "inputs": ["x", "w", "b"], "outputs": ["c"],
         "args": dict({"base_axis": 1, "pad": (0, 0), "stride": (1, 1), "dilation": (1, 1), "group": 1,
                       "channel_last": False}, **(conv_args or {}))},
        {"op": "BatchNormalization", "inputs": ["c", "beta", "gamma", "mean", "var"], "outputs": ["n"],
         "args": {"axes": [1], "decay_rate": 0.9, "eps": 1e-5, "batch_stat": False}},
    ]
    last = "n"
    if act:
        nodes.append({"op": act, "inputs": [last], "outputs": ["a"], "args": {}})
        last = "a"
    if quant_op:
        nodes.append({"op": quant_op, "inputs": [last], "outputs": ["y"], "args": quant_args or {}})
    if extra_consumer:
        nodes.append({"op": "FixedPointQuantize", "inputs": [extra_consumer], "outputs": ["z"], "args": {}})
    return nodes


PW_SHAPES = {"x": (2, 8, 14, 14), "w": (16, 8, 1, 1)}


def test_pointwise_chain_is_fused_into_one_node():
    for act, qop in (("ReLU6", "FixedPointQuantize"), ("ReLU", "Pow2Quantize"), (None, "FixedPointQuantize"),
                     ("ReLU6", None), (None, None)):
        out_name = "y" if qop else ("a" if act else "n")
        fused = graph.fuse_pw_bn_quant(_pw_chain(act, qop), [out_name], PW_SHAPES)
        assert [n["op"] for n in fused] == [graph.FUSED_PW], (act, qop)
        f = fused[0]
        assert f["outputs"] == [out_name]
        assert f["act"] == {"ReLU6": "relu6", "ReLU": "relu", None: None}[act]
        assert (f["quant"] or {}).get("op") == qop
        assert f["inputs"] == ["x", "w", "b", "beta", "gamma", "mean", "var"]


def test_pointwise_patterns_that_must_not_fuse():
    ops_of = lambda nodes: [n["op"] for n in nodes]
    # a 3x3 kernel, a stride, padding, groups, channel-last, or no shape information: left alone
    for shapes, args in ((dict(PW_SHAPES, w=(16, 8, 3, 3)), {}), (PW_SHAPES, {"stride": (2, 2)}), (PW_SHAPES, {"pad": (1, 1)}),
                         (PW_SHAPES, {"group": 2}), (PW_SHAPES, {"channel_last": True}), (None, {})):
        nodes = _pw_chain(conv_args=args)
        assert ops_of(graph.fuse_pw_bn_quant(nodes, ["y"], shapes)) == ops_of(nodes)
    # MinMaxQuantize stays a node of its own behind the fused convolution + BN + activation
    nodes = _pw_chain("ReLU6", None) + [{"op": "MinMaxQuantize", "inputs": ["a", "q0", "q1", "q2", "q3"], "outputs": ["y"],
                                         "args": {}}]
    assert ops_of(graph.fuse_pw_bn_quant(nodes, ["y"], PW_SHAPES)) == [graph.FUSED_PW, "MinMaxQuantize"]
    # an intermediate with a second consumer (or that is a graph output) ends the fused chain there
    assert ops_of(graph.fuse_pw_bn_quant(_pw_chain(extra_consumer="a"), ["y", "z"], PW_SHAPES)) == \
        [graph.FUSED_PW, "FixedPointQuantize", "FixedPointQuantize"]
    assert ops_of(graph.fuse_pw_bn_quant(_pw_chain(extra_consumer="c"), ["y", "z"], PW_SHAPES)) == ops_of(
        _pw_chain(extra_consumer="c"))
    fused = graph.fuse_pw_bn_quant(_pw_chain(), ["y", "n"], PW_SHAPES)
    assert ops_of(fused) == [graph.FUSED_PW, "ReLU6", "FixedPointQuantize"] and fused[0]["act"] is None
    # batch statistics: not the inference form
    nodes = _pw_chain()
    nodes[1]["args"]["batch_stat"] = True
    assert ops_of(graph.fuse_pw_bn_quant(nodes, ["y"], PW_SHAPES)) == ops_of(nodes)
    # the two passes compose: an inverted residual's expansion, depthwise layer and projection
    block = _pw_chain()
    for n in block:
        n["inputs"] = [("e_" + v) if v != "x" else v for v in n["inputs"]]
        n["outputs"] = ["e_" + v for v in n["outputs"]]
    block += [dict(n, inputs=[("d_" + v) if v != "x" else "e_y" for v in n["inputs"]], outputs=["d_" + v for v in n["outputs"]])
              for n in _chain("FixedPointQuantize")]
    shapes = {"x": (2, 8, 14, 14), "e_w": (16, 8, 1, 1), "d_w": (16, 3, 3)}
    both = graph.fuse_dw_bn_quant(graph.fuse_pw_bn_quant(block, ["d_y"], shapes), ["d_y"], shapes)
    assert ops_of(both) == [graph.FUSED_PW, graph.FUSED]


@pytest.mark.gpu
def test_fused_pointwise_graph_equals_unfused_graph(oracle, cuda_device):
    import torch
    from dwbnq import workloads
    for spec in (workloads.pw1(3)[7], workloads.pw1(2)[26]):  # an expansion on 28x28, a projection on 7x7
        d = workloads.make_pointwise_data(spec)
        qop_args = {"sign": spec.quant["sign"], "n": 8, "delta": spec.quant["delta"]}
        nodes = _pw_chain("ReLU6" if spec.act else None, "FixedPointQuantize", qop_args)
        names = ["x", "w", "b", "beta", "gamma", "mean", "var"]
        fresh = lambda: {k: torch.from_numpy(d[k].copy()).to(cuda_device) for k in names}
        t_unfused = graph.execute(nodes, fresh(), check=True)
        fused = graph.fuse_pw_bn_quant(nodes, ["y"], {k: tuple(d[k].shape) for k in names})
        assert [n["op"] for n in fused] == [graph.FUSED_PW]
        t_fused = graph.execute(fused, fresh(), check=True)
        assert torch.equal(t_unfused["y"].view(torch.int32), t_fused["y"].view(torch.int32)), spec.name
        want = oracle.pw_epilogue(t_unfused["c"].cpu().numpy(), d["beta"], d["gamma"], d["mean"], d["var"], 1e-5, spec.act,
                                  spec.quant)
        assert np.array_equal(t_fused["y"].cpu().numpy().view(np.uint32), want.view(np.uint32)), spec.name
