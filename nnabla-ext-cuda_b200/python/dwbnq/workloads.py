"""The benchmark / parity workloads and their seeded synthetic inputs.

No dataset is involved: activations, weights and BN statistics are drawn from the
distributions the workload definitions state, all in float32, with
``numpy.random.default_rng``: the parameters of a layer come first from the layer's
generator (seed), in the order W, b, mean, var, gamma, beta; every image then comes from a
generator of its own (seed, image index), which draws x and, for cfg3, the outlier mask and
values. An image is therefore the same whichever batch shard it is drawn in, which is what
lets the ranks of a sharded job and the single-device oracle see identical data.
``N(mu, v)`` below means variance ``v``.

Workloads (ids follow the benchmark's config list):
  cfg0  single layer  x[32,64,56,56]~N(0,1), 3x3 s1 p1, BN, FixedPointQuantize(sign, n=8, delta=2^-4)
  cfg1  the 17 depthwise layers of MobileNetV2 at 224x224, batch 256, each with its own
        input x~ReLU6(N(0,1)), BN, FixedPointQuantize(unsigned, n=8, delta=2^-3)
  cfg2  x[128,144,56,56]~N(0,1), 5x5 s1 p2, BN, Pow2Quantize(sign, with_zero, n=8, m=1)
  cfg3  x[512,192,28,28]~N(0,2) with 0.1% outliers~U(-20,20), 3x3 s2 p1, BN,
        MinMaxQuantize(per-channel over axes (0,2,3), ql=[0,255], x_min_max, no ema)
  cfg4  cfg1 cast to float16
  pw1   the 33 pointwise (1x1) convolutions that sit either side of cfg1's depthwise layers in
        MobileNetV2: 16 expansions (BN, ReLU6, unsigned FixedPointQuantize as in cfg1; input
        x~N(0,1), the signed output of a projection) and 17 linear projections (BN, signed
        FixedPointQuantize n=8, delta=2^-4; input x~ReLU6(N(0,1)) like cfg1's), W~N(0,1/c_in)
"""
import os
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field

import numpy as np

# (channels, input height = width, stride) of the 17 depthwise 3x3 layers of MobileNetV2.
MOBILENETV2_DW = ([(32, 112, 1), (96, 112, 2), (144, 56, 1), (144, 56, 2)] + [(192, 28, 1)] * 2 +
                  [(192, 28, 2)] + [(384, 14, 1)] * 4 + [(576, 14, 1)] * 2 + [(576, 14, 2)] +
                  [(960, 7, 1)] * 3)

# (c_in, c_out, height = width, kind) of the pointwise layers around them: block i expands
# c_in -> 6 c_in at the block's input resolution (the first block has no expansion) and
# projects 6 c_in -> c_out at the depthwise layer's output resolution.
_MBV2_BLOCK_IO = ([(32, 16), (16, 24), (24, 24), (24, 32), (32, 32), (32, 32), (32, 64)] + [(64, 64)] * 3 + [(64, 96)] +
                  [(96, 96)] * 2 + [(96, 160)] + [(160, 160)] * 2 + [(160, 320)])


def mobilenetv2_pointwise():
    out = []
    for (cin, cout), (cdw, h, stride) in zip(_MBV2_BLOCK_IO, MOBILENETV2_DW):
        if cdw != cin:
            out.append((cin, cdw, h, "expand"))
        out.append((cdw, cout, h // stride, "project"))
    return out


FPQ_CFG0 = {"kind": "fpq", "sign": True, "n": 8, "delta": 2.0 ** -4}
FPQ_CFG1 = {"kind": "fpq", "sign": False, "n": 8, "delta": 2.0 ** -3}
POW2_CFG2 = {"kind": "pow2", "sign": True, "with_zero": True, "n": 8, "m": 1}
MINMAX_CFG3 = {"kind": "minmax", "decay": 0.999, "x_min_max": True, "ema": False, "eps": 0.01,
               "ql_min": 0.0, "ql_max": 255.0}


@dataclass
class LayerSpec:
    name: str
    n: int
    c: int
    h: int
    w: int
    k: int = 3
    stride: int = 1
    pad: int = 1
    quant: dict = field(default_factory=lambda: dict(FPQ_CFG1))
    seed: int = 0
    x_dist: str = "normal"  # "normal" | "relu6" | "normal2_outliers"
    bn_eps: float = 1e-5

    @property
    def ho(self):
        return (self.h + 2 * self.pad - (self.k - 1) - 1) // self.stride + 1

    @property
    def wo(self):
        return (self.w + 2 * self.pad - (self.k - 1) - 1) // self.stride + 1

    def elems_in(self, n=None):
        return (self.n if n is None else n) * self.c * self.h * self.w

    def elems_out(self, n=None):
        return (self.n if n is None else n) * self.c * self.ho * self.wo

    def algorithmic_bytes(self, itemsize=4, n=None):
        """Read x once, write the quantized y once (parameter vectors are < 0.01 %)."""
        return itemsize * (self.elems_in(n) + self.elems_out(n))


def cfg0(n=32):
    return [LayerSpec("cfg0", n, 64, 56, 56, 3, 1, 1, dict(FPQ_CFG0), seed=0)]


def cfg1(n=256):
    return [LayerSpec("cfg1.l%02d" % i, n, c, hw, hw, 3, s, 1, dict(FPQ_CFG1), seed=i, x_dist="relu6")
            for i, (c, hw, s) in enumerate(MOBILENETV2_DW)]


def cfg2(n=128):
    return [LayerSpec("cfg2", n, 144, 56, 56, 5, 1, 2, dict(POW2_CFG2), seed=0)]


def cfg3(n=512):
    return [LayerSpec("cfg3", n, 192, 28, 28, 3, 2, 1, dict(MINMAX_CFG3), seed=0, x_dist="normal2_outliers")]


def workload(name, n=None):
    table = {"cfg0": cfg0, "cfg1": cfg1, "cfg2": cfg2, "cfg3": cfg3, "cfg4": cfg1, "cfg1q8": cfg1}
    return table[name]() if n is None else table[name](n)


def _normal(rng, shape, var):
    a = rng.standard_normal(shape, dtype=np.float32)
    if var != 1.0:
        a *= np.float32(np.sqrt(var))
    return a


def _uniform(rng, shape, lo, hi):
    return (rng.random(shape, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def make_layer_data(spec, n=None, first_image=0, dtype=np.float32):
    """Seeded tensors of one layer: dict with x, w, b, mean, var, gamma, beta (and, for
    MinMax, qr_min, qr_max, ql_min, ql_max). ``n`` / ``first_image`` select a batch shard:
    image i of the full batch is the same whatever shard it is drawn in (one generator per
    image), so ranks of a sharded job and the single-device oracle see identical data."""
    n = spec.n if n is None else n
    rng = np.random.default_rng(spec.seed)
    # Parameters first from the layer generator so they do not depend on the shard.
    k = spec.k
    d = {}
    d["w"] = _normal(rng, (spec.c, k, k), 1.0 / (k * k))
    d["b"] = _normal(rng, (spec.c,), 0.1)
    d["mean"] = _normal(rng, (spec.c,), 0.1)
    d["var"] = _uniform(rng, (spec.c,), 0.5, 1.5)
    d["gamma"] = _uniform(rng, (spec.c,), 0.8, 1.2)
    d["beta"] = _normal(rng, (spec.c,), 0.1)
    x = np.empty((n, spec.c, spec.h, spec.w), dtype=np.float32)

    def one_image(i):
        irng = np.random.default_rng([spec.seed, 1 + first_image + i])
        if spec.x_dist == "normal":
            x[i] = irng.standard_normal((spec.c, spec.h, spec.w), dtype=np.float32)
        elif spec.x_dist == "relu6":
            xi = irng.standard_normal((spec.c, spec.h, spec.w), dtype=np.float32)
            np.clip(xi, 0.0, 6.0, out=xi)
            x[i] = xi
        elif spec.x_dist == "normal2_outliers":
            xi = _normal(irng, (spec.c, spec.h, spec.w), 2.0)
            mask = irng.random((spec.c, spec.h, spec.w), dtype=np.float32) < np.float32(0.001)
            out = _uniform(irng, (spec.c, spec.h, spec.w), -20.0, 20.0)
            xi[mask] = out[mask]
            x[i] = xi
        else:
            raise ValueError(spec.x_dist)

    workers = min(16, os.cpu_count() or 1)
    if n >= 8 and workers > 1:
        with ThreadPoolExecutor(workers) as pool:
            list(pool.map(one_image, range(n)))
    else:
        for i in range(n):
            one_image(i)
    d["x"] = x
    if spec.quant["kind"] == "minmax":
        d["qr_min"] = np.zeros(spec.c, np.float32)
        d["qr_max"] = np.ones(spec.c, np.float32)
        d["ql_min"] = np.full(spec.c, spec.quant["ql_min"], np.float32)
        d["ql_max"] = np.full(spec.c, spec.quant["ql_max"], np.float32)
    if dtype != np.float32:
        d = {k_: v.astype(dtype) for k_, v in d.items()}
    return d


def quant_for_ops(spec, tensors=None):
    """The quantizer dict in the form dwbnq.ops / the oracle take (MinMax: with tensors)."""
    q = {k_: v for k_, v in spec.quant.items() if k_ not in ("ql_min", "ql_max")}
    if q["kind"] == "minmax" and tensors is not None:
        for k_ in ("qr_min", "qr_max", "ql_min", "ql_max"):
            q[k_] = tensors[k_]
    return q


@dataclass
class PointwiseSpec:
    name: str
    n: int
    c_in: int
    c_out: int
    h: int
    kind: str  # "expand": BN, ReLU6, unsigned FPQ; "project": BN, signed FPQ
    seed: int = 0
    bn_eps: float = 1e-5

    @property
    def act(self):
        return "relu6" if self.kind == "expand" else None

    @property
    def quant(self):
        return dict(FPQ_CFG1) if self.kind == "expand" else dict(FPQ_CFG0)

    def algorithmic_bytes(self, itemsize=4, n=None):
        n = self.n if n is None else n
        return itemsize * (n * (self.c_in + self.c_out) * self.h * self.h + self.c_in * self.c_out + 5 * self.c_out)

    def flops(self, n=None):
        n = self.n if n is None else n
        return 2.0 * n * self.h * self.h * self.c_in * self.c_out


def pw1(n=256):
    return [PointwiseSpec("pw1.l%02d.%s" % (i, kind), n, ci, co, h, kind, seed=100 + i)
            for i, (ci, co, h, kind) in enumerate(mobilenetv2_pointwise())]


def make_pointwise_data(spec, n=None, dtype=np.float32):
    """Parameters from the layer's generator in the order W, b, mean, var, gamma, beta, then x."""
    n = spec.n if n is None else n
    rng = np.random.default_rng(spec.seed)
    co, ci = spec.c_out, spec.c_in
    d = {
        "w": _normal(rng, (co, ci, 1, 1), 1.0 / ci),
        "b": _normal(rng, (co,), 0.1),
        "mean": _normal(rng, (co,), 0.1),
        "var": _uniform(rng, (co,), 0.5, 1.5),
        "gamma": _uniform(rng, (co,), 0.8, 1.2),
        "beta": _normal(rng, (co,), 0.1),
    }
    x = rng.standard_normal((n, ci, spec.h, spec.h), dtype=np.float32)
    if spec.kind == "project":
        x = np.minimum(np.maximum(x, 0.0), 6.0)
    d["x"] = x
    return {k: np.ascontiguousarray(v, dtype=dtype) for k, v in d.items()}


def mobilenetv2_body(n=256):
    """The 50 convolution layers of MobileNetV2's inverted-residual stack in network order:
    [("dw", LayerSpec) | ("pw", PointwiseSpec), ...] - cfg1's depthwise layers with pw1's
    projections and expansions between them (residual additions left out: each layer feeds the
    next). The input is [n, 32, 112, 112], the output [n, 320, 7, 7]."""
    dws, pws = cfg1(n), pw1(n)
    order, p = [("dw", dws[0]), ("pw", pws[0])], 1
    for dw in dws[1:]:
        order += [("pw", pws[p]), ("dw", dw), ("pw", pws[p + 1])]
        p += 2
    assert p == len(pws)
    for (_, a), (_, b) in zip(order, order[1:]):
        a_out = (a.c, a.ho) if isinstance(a, LayerSpec) else (a.c_out, a.h)
        b_in = (b.c, b.h) if isinstance(b, LayerSpec) else (b.c_in, b.h)
        assert a_out == b_in, (a.name, b.name)
    return order


def body_graph(n=256, dtype=np.float32):
    """The body as the unfused function list nnabla would build (DepthwiseConvolution |
    Convolution -> BatchNormalization(batch_stat=False) -> [ReLU6] -> FixedPointQuantize per
    layer, 166 functions), with its seeded parameters. Returns (nodes, tensors, input name,
    output name, [name of each layer's output]); ``tensors`` holds the parameters of every
    layer and the input "x0" (cfg1's first-layer input) as numpy arrays."""
    nodes, tensors, layer_outputs = [], {}, []
    order = mobilenetv2_body(n)
    cur = "x0"
    tensors[cur] = make_layer_data(order[0][1], n, dtype=dtype)["x"]
    for li, (kind, spec) in enumerate(order):
        p = "L%02d" % li
        data = (make_layer_data(LayerSpec(**dict(spec.__dict__, n=0)), 0, dtype=dtype) if kind == "dw"
                else make_pointwise_data(PointwiseSpec(**dict(spec.__dict__, n=0)), 0, dtype=dtype))
        for k_ in ("w", "b", "beta", "gamma", "mean", "var"):
            tensors["%s.%s" % (p, k_)] = data[k_]
        if kind == "dw":
            nodes.append({"op": "DepthwiseConvolution", "inputs": [cur, p + ".w", p + ".b"], "outputs": [p + ".c"],
                          "args": {"base_axis": 1, "pad": (spec.pad, spec.pad), "stride": (spec.stride, spec.stride),
                                   "dilation": (1, 1), "multiplier": 1}})
        else:
            nodes.append({"op": "Convolution", "inputs": [cur, p + ".w", p + ".b"], "outputs": [p + ".c"],
                          "args": {"base_axis": 1, "pad": (0, 0), "stride": (1, 1), "dilation": (1, 1), "group": 1}})
        nodes.append({"op": "BatchNormalization", "inputs": [p + ".c", p + ".beta", p + ".gamma", p + ".mean", p + ".var"],
                      "outputs": [p + ".bn"], "args": {"axes": [1], "decay_rate": 0.9, "eps": spec.bn_eps,
                                                       "batch_stat": False}})
        last = p + ".bn"
        if kind == "pw" and spec.act == "relu6":
            nodes.append({"op": "ReLU6", "inputs": [last], "outputs": [p + ".a"], "args": {}})
            last = p + ".a"
        q = spec.quant
        nodes.append({"op": "FixedPointQuantize", "inputs": [last], "outputs": [p + ".q"],
                      "args": {"sign": q["sign"], "n": q["n"], "delta": q["delta"]}})
        cur = p + ".q"
        layer_outputs.append(cur)
    return nodes, tensors, "x0", cur, layer_outputs
