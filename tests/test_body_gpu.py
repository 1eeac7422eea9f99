"""MobileNetV2's quantized body as one network: the 50 depthwise and pointwise layers chained
(every layer reads the previous layer's output), written as the unfused function list nnabla
would build, rewritten by the two graph passes and run through the library.

  * the passes turn the 166 functions into 17 FusedDwBnQuant + 33 FusedPwBnQuant nodes (CPU);
  * layer by layer, on the input the GPU itself produced for that layer: a depthwise layer equals
    the oracle bit for bit; a pointwise layer lies between the oracle's epilogue of (double sum -
    tolerance) and (double sum + tolerance) - 4e-6 of sum |w||x|, the three-pass TF32 bound - and
    differs from the epilogue of the oracle's own fp32 sum on at most a few outputs per thousand
    (sums that land on a rounding boundary of the quantizer);
  * the fused network, the unfused function list run function by function, and the CUDA-graph
    replay with prepared pointwise parameters give the same bits at every layer output."""
import numpy as np
import pytest
import torch

from dwbnq import graph, ops, workloads


def _fused(n):
    nodes, host, x_in, x_out, layer_outputs = workloads.body_graph(n)
    shapes = {k: v.shape for k, v in host.items()}
    fused = graph.fuse_pw_bn_quant(graph.fuse_dw_bn_quant(nodes, [x_out], shapes), [x_out], shapes)
    return nodes, fused, host, x_in, x_out, layer_outputs


def test_the_passes_fuse_every_layer_of_the_body():
    nodes, fused, host, x_in, x_out, layer_outputs = _fused(0)
    assert len(nodes) == 166 and len(fused) == 50
    order = workloads.mobilenetv2_body(1)
    assert [n["op"] for n in fused] == [graph.FUSED if k == "dw" else graph.FUSED_PW for k, _ in order]
    assert [n["outputs"][0] for n in fused] == layer_outputs and layer_outputs[-1] == x_out
    for n, (kind, spec) in zip(fused, order):
        assert n["quant"]["op"] == "FixedPointQuantize" and n["quant"]["args"]["sign"] == spec.quant["sign"]
        if kind == "pw":
            assert n["act"] == spec.act
    # without shapes a Convolution cannot be told to be pointwise: only the depthwise chains fuse
    only_dw = graph.fuse_pw_bn_quant(graph.fuse_dw_bn_quant(nodes, [x_out]), [x_out])
    assert sum(n["op"] == graph.FUSED for n in only_dw) == 17 and not any(n["op"] == graph.FUSED_PW for n in only_dw)


def test_prepare_walks_the_shapes_from_the_graph_input(monkeypatch):
    """prepare_pointwise needs each pointwise layer's input shape before anything has run: it
    derives them from the graph input and the weights (checked here with the library call
    replaced by a recorder - no device involved)."""
    nodes, fused, host, x_in, x_out, layer_outputs = _fused(2)
    seen = []
    monkeypatch.setattr(ops, "pwconv_prepare", lambda x, w, *a, **k: seen.append((tuple(x.shape), tuple(w.shape))) or "ws")
    out = graph.prepare_pointwise(fused, {k: torch.from_numpy(v) for k, v in host.items()})
    pw = [sp for kind, sp in workloads.mobilenetv2_body(2) if kind == "pw"]
    assert [sx for sx, _ in seen] == [(2, sp.c_in, sp.h, sp.h) for sp in pw]
    assert [sw for _, sw in seen] == [(sp.c_out, sp.c_in, 1, 1) for sp in pw]
    assert sum(nd.get("prepared_ws") == "ws" for nd in out) == 33 and not any("prepared_ws" in nd for nd in fused)


@pytest.mark.gpu
def test_body_layer_by_layer_against_the_oracle(oracle, cuda_device):
    n = 2
    nodes, fused, host, x_in, x_out, layer_outputs = _fused(n)
    t = {k: torch.from_numpy(v).to(cuda_device) for k, v in host.items()}
    graph.execute(fused, t, check=True)
    nt = oracle.max_threads()
    x = host[x_in]
    flips = 0
    for li, ((kind, spec), node) in enumerate(zip(workloads.mobilenetv2_body(n), fused)):
        p = "L%02d." % li
        got = t[node["outputs"][0]].cpu().numpy()
        prm = [host[p + k] for k in ("beta", "gamma", "mean", "var")]
        if kind == "dw":
            want = oracle.fused_layer(x, host[p + "w"], host[p + "b"], *prm, spec.bn_eps, (spec.stride,) * 2,
                                      (spec.pad,) * 2, workloads.quant_for_ops(spec), nthreads=nt)
            assert got.shape == want.shape
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "layer %d (%s)" % (li, spec.name)
        else:
            acc32, acc64, mag = oracle.pwconv(x, host[p + "w"], host[p + "b"], nthreads=nt)
            tol = (4e-6 * mag).astype(np.float32) + 1e-30
            lo = oracle.pw_epilogue(acc64 - tol, *prm, spec.bn_eps, spec.act, spec.quant, nthreads=nt)
            hi = oracle.pw_epilogue(acc64 + tol, *prm, spec.bn_eps, spec.act, spec.quant, nthreads=nt)
            lo, hi = np.minimum(lo, hi), np.maximum(lo, hi)
            assert got.shape == lo.shape
            assert ((got >= lo) & (got <= hi)).all(), "layer %d (%s) leaves the bracket" % (li, spec.name)
            want = oracle.pw_epilogue(acc32, *prm, spec.bn_eps, spec.act, spec.quant, nthreads=nt)
            differ = int((got != want).sum())
            assert differ <= 2e-3 * got.size + 2, "layer %d (%s): %d of %d outputs" % (li, spec.name, differ, got.size)
            flips += differ
        assert len(np.unique(got)) > 8, "layer %d collapsed" % li  # the network stays alive to its end
        x = got  # the next layer is checked on what the GPU really fed it
    assert tuple(x.shape) == (n, 320, 7, 7)


@pytest.mark.gpu
def test_fused_unfused_and_replayed_body_agree_bit_for_bit(cuda_device):
    n = 3
    nodes, fused, host, x_in, x_out, layer_outputs = _fused(n)
    a = {k: torch.from_numpy(v).to(cuda_device) for k, v in host.items()}
    b = {k: v.clone() for k, v in a.items()}
    c = {k: v.clone() for k, v in a.items()}
    graph.execute(fused, a, check=True)
    graph.execute(nodes, b, check=True)       # 166 functions, one kernel (or more) each
    runner = graph.GraphRunner(fused, c)       # pointwise parameters prepared once, 50 launches in a CUDA graph
    assert sum("prepared_ws" in nd for nd in runner.nodes) == 33
    c[x_in].copy_(a[x_in])
    runner.replay()
    runner.replay()
    runner.synchronize()
    for name in layer_outputs:
        assert torch.equal(a[name], b[name]), "fused and unfused differ at " + name
        assert torch.equal(a[name], c[name]), "replay differs at " + name
