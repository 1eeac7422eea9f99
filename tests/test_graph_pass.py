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


def test_chain_is_fused_into_one_node():
    for op in ("FixedPointQuantize", "Pow2Quantize", "MinMaxQuantize"):
        fused = graph.fuse_dw_bn_quant(_chain(op), graph_outputs=["y"])
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
    # unrelated nodes pass through untouched and in order
    other = {"op": "ReLU6", "inputs": ["y"], "outputs": ["r"], "args": {}}
    g = graph.fuse_dw_bn_quant(_chain() + [other], ["r"])
    assert [n["op"] for n in g] == [graph.FUSED, "ReLU6"]


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
        fused = graph.fuse_dw_bn_quant(nodes, ["y"])
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
