"""Graph passes: DepthwiseConvolution -> BatchNormalization(batch_stat=False) -> quantizer
becomes one fused node, so does pointwise Convolution -> BatchNormalization -> [ReLU | ReLU6] ->
quantizer (``fuse_pw_bn_quant``); and a small executor that runs such graphs through libdwbnq.

nnabla's graph converters (``nnabla.experimental.graph_converters``, e.g.
BatchNormalizationFolding) walk a function list and rewrite conv -> BN chains whose
intermediate variable has a single consumer. This pass matches the same shape of pattern
one function further (the quantizer) but, unlike BN folding, keeps the BN parameters as
they are: folding them into the weights changes the rounding of every output, while the
fused kernel reproduces the three-function chain bit for bit.

The IR is a plain list of nodes in topological order:
    {"op": "DepthwiseConvolution", "inputs": ["x", "w", "b"], "outputs": ["c"],
     "args": {"base_axis": 1, "pad": (1, 1), "stride": (1, 1), "dilation": (1, 1), "multiplier": 1}}
with the function names and argument names of nnabla's functions.yaml. ``from_nnabla``
builds it from a real nnabla graph when nnabla is importable.
"""
from collections import Counter

QUANTIZERS = ("FixedPointQuantize", "Pow2Quantize", "MinMaxQuantize")
FUSED = "FusedDwBnQuant"
FUSED_PW = "FusedPwBnQuant"
ACTIVATIONS = {"ReLU": "relu", "ReLU6": "relu6"}


def _consumers(nodes):
    c = Counter()
    for n in nodes:
        for v in n["inputs"]:
            c[v] += 1
    return c


def _bn_is_fusable(bn, channel_axis):
    a = bn["args"]
    axes = list(a.get("axes", [1]))
    return (not a.get("batch_stat", True)) and axes == [channel_axis] and len(bn["outputs"]) == 1


def fuse_dw_bn_quant(nodes, graph_outputs=(), shapes=None):
    """Returns a new node list where every dw-conv -> BN(inference) -> quantizer chain whose
    intermediates have no other consumer (and are not graph outputs) is one FusedDwBnQuant
    node. A dw-conv -> BN chain without a quantizer is fused too (quantizer "none").

    ``shapes`` maps variable names to shapes (``from_nnabla`` returns it). A MinMaxQuantize
    is absorbed only when its range tensors are known to be per-channel along the
    convolution's channel axis ([1, C*multiplier, 1, 1]); with per-tensor ranges, or without
    shape information, it stays a node of its own behind the fused conv + BN."""
    nodes = list(nodes)
    uses = _consumers(nodes)
    keep = set(graph_outputs)
    producer = {}
    for i, n in enumerate(nodes):
        for v in n["outputs"]:
            producer[v] = i
    consumer_of = {}
    for i, n in enumerate(nodes):
        for v in n["inputs"]:
            consumer_of.setdefault(v, []).append(i)

    def sole_consumer(var):
        if var in keep or uses[var] != 1:
            return None
        return consumer_of[var][0]

    removed = set()
    out = []
    for i, conv in enumerate(nodes):
        if i in removed:
            continue
        if conv["op"] != "DepthwiseConvolution":
            out.append(conv)
            continue
        j = sole_consumer(conv["outputs"][0])
        base_axis = conv["args"].get("base_axis", 1)
        if j is None or nodes[j]["op"] != "BatchNormalization" or nodes[j]["inputs"][0] != conv["outputs"][0] \
                or not _bn_is_fusable(nodes[j], base_axis):
            out.append(conv)
            continue
        bn = nodes[j]
        fused = {"op": FUSED, "conv_args": dict(conv["args"]), "bn_args": dict(bn["args"]), "quant": None,
                 "inputs": list(conv["inputs"]) + list(bn["inputs"][1:]), "n_conv_inputs": len(conv["inputs"]),
                 "outputs": list(bn["outputs"])}
        removed.add(j)
        k = sole_consumer(bn["outputs"][0])
        if k is not None and nodes[k]["op"] in QUANTIZERS and nodes[k]["inputs"][0] == bn["outputs"][0]:
            qn = nodes[k]
            if qn["op"] != "MinMaxQuantize" or _minmax_is_per_channel(qn, conv, shapes):
                fused["quant"] = {"op": qn["op"], "args": dict(qn["args"])}
                fused["inputs"] += list(qn["inputs"][1:])
                fused["outputs"] = list(qn["outputs"])
                removed.add(k)
        out.append(fused)
    # keep topological order: a fused node sits where its convolution was; everything it
    # needs (parameters) is a graph input or was produced earlier
    return out


def _is_pointwise(conv, shapes):
    """Convolution with a 1x1 kernel, pad 0, stride 1, dilation 1, group 1, NCHW: the weight's
    shape (``shapes``) decides the kernel size; without it the node is left alone."""
    a = conv["args"]
    if a.get("group", 1) != 1 or a.get("channel_last", False) or not shapes or len(conv["inputs"]) < 2:
        return False
    w = shapes.get(conv["inputs"][1])
    if w is None or len(w) != 4 or tuple(int(v) for v in w[2:]) != (1, 1):
        return False
    one = lambda v, d: all(int(e) == d for e in (v if v is not None else (d, d)))
    return one(a.get("pad"), 0) and one(a.get("stride"), 1) and one(a.get("dilation"), 1)


def fuse_pw_bn_quant(nodes, graph_outputs=(), shapes=None):
    """Every pointwise Convolution -> BN(inference) -> [ReLU | ReLU6] -> FixedPointQuantize |
    Pow2Quantize chain whose intermediates have no other consumer becomes one FusedPwBnQuant
    node (activation and quantizer are optional; a MinMaxQuantize is never absorbed: it needs the
    whole tensor's range first). Run it after or before ``fuse_dw_bn_quant``: the two passes
    match disjoint operators."""
    nodes = list(nodes)
    uses = _consumers(nodes)
    keep = set(graph_outputs)
    consumer_of = {}
    for i, n in enumerate(nodes):
        for v in n["inputs"]:
            consumer_of.setdefault(v, []).append(i)

    def sole_consumer(var):
        if var in keep or uses[var] != 1:
            return None
        return consumer_of[var][0]

    removed, out = set(), []
    for i, conv in enumerate(nodes):
        if i in removed:
            continue
        if conv["op"] != "Convolution" or not _is_pointwise(conv, shapes):
            out.append(conv)
            continue
        base_axis = conv["args"].get("base_axis", 1)
        j = sole_consumer(conv["outputs"][0])
        if j is None or nodes[j]["op"] != "BatchNormalization" or nodes[j]["inputs"][0] != conv["outputs"][0] \
                or not _bn_is_fusable(nodes[j], base_axis):
            out.append(conv)
            continue
        bn = nodes[j]
        fused = {"op": FUSED_PW, "conv_args": dict(conv["args"]), "bn_args": dict(bn["args"]), "act": None, "quant": None,
                 "inputs": list(conv["inputs"]) + list(bn["inputs"][1:]), "n_conv_inputs": len(conv["inputs"]),
                 "outputs": list(bn["outputs"])}
        removed.add(j)
        k = sole_consumer(fused["outputs"][0])
        if k is not None and nodes[k]["op"] in ACTIVATIONS and nodes[k]["inputs"][0] == fused["outputs"][0]:
            fused["act"] = ACTIVATIONS[nodes[k]["op"]]
            fused["outputs"] = list(nodes[k]["outputs"])
            removed.add(k)
            k = sole_consumer(fused["outputs"][0])
        if k is not None and nodes[k]["op"] in ("FixedPointQuantize", "Pow2Quantize") \
                and nodes[k]["inputs"][0] == fused["outputs"][0]:
            fused["quant"] = {"op": nodes[k]["op"], "args": dict(nodes[k]["args"])}
            fused["outputs"] = list(nodes[k]["outputs"])
            removed.add(k)
        out.append(fused)
    return out


def _minmax_is_per_channel(qn, conv, shapes):
    """MinMaxQuantize has no axis argument (decay, x_min_max, ema, ste_fine_grained, eps):
    whether it is per-channel or per-tensor is decided by the shape of its range inputs."""
    if not shapes or len(qn["inputs"]) < 5 or len(conv["inputs"]) < 2:
        return False
    w_shape = shapes.get(conv["inputs"][1])
    if not w_shape:
        return False
    oc = int(w_shape[0])
    axis = conv["args"].get("base_axis", 1)
    for name in qn["inputs"][1:5]:
        shp = shapes.get(name)
        if shp is None:
            return False
        shp = tuple(int(v) for v in shp)
        if len(shp) == 1:  # a bare [C] vector is accepted as per-channel too
            if shp[0] != oc:
                return False
            continue
        if axis >= len(shp) or shp[axis] != oc or any(v != 1 for i, v in enumerate(shp) if i != axis):
            return False
    return True


def execute(nodes, tensors, comm=None, check=False):
    """Runs the node list on torch CUDA tensors (dict name -> tensor, updated in place with
    every produced variable). Only the operators of this library are known. ``check=True``
    synchronises at the end and raises if a kernel gave up one of its bounded waits (its
    output tile would then be stale)."""
    from . import ops

    t = tensors
    for n in nodes:
        a = n.get("args", {})
        i = [t[v] if v is not None else None for v in n["inputs"]]
        if n["op"] == "DepthwiseConvolution":
            b = i[2] if len(i) > 2 else None
            y = ops.depthwise_convolution(i[0], i[1], b, a.get("base_axis", 1), a.get("pad"), a.get("stride"),
                                          a.get("dilation"), a.get("multiplier", 1))
        elif n["op"] == "BatchNormalization":
            beta, gamma, mean, var = _bn_inputs(i[1:], a)
            y = ops.batch_normalization(i[0], beta, gamma, mean, var, a.get("axes", [1]), a.get("decay_rate", 0.9),
                                        a.get("eps", 1e-5), a.get("batch_stat", True))
        elif n["op"] == "FixedPointQuantize":
            y = ops.fixed_point_quantize(i[0], a.get("sign", True), a.get("n", 8), a.get("delta", 2.0 ** -4))
        elif n["op"] == "Pow2Quantize":
            y = ops.pow2_quantize(i[0], a.get("sign", True), a.get("with_zero", True), a.get("n", 8), a.get("m", 1))
        elif n["op"] == "MinMaxQuantize":
            y = ops.min_max_quantize(i[0], i[1], i[2], i[3], i[4], a.get("decay", 0.999), a.get("x_min_max", False),
                                     a.get("ema", False), True, a.get("eps", 0.01), comm=comm)
        elif n["op"] == FUSED:
            nc = n["n_conv_inputs"]
            ca, ba = n["conv_args"], n["bn_args"]
            b = i[2] if nc > 2 else None
            n_bn = 4 - int(ba.get("no_bias", False)) - int(ba.get("no_scale", False))
            beta, gamma, mean, var = _bn_inputs(i[nc:nc + n_bn], ba)
            quant = None
            if n["quant"]:
                qa = n["quant"]["args"]
                qi = i[nc + n_bn:]
                if n["quant"]["op"] == "FixedPointQuantize":
                    quant = {"kind": "fpq", "sign": qa.get("sign", True), "n": qa.get("n", 8),
                             "delta": qa.get("delta", 2.0 ** -4)}
                elif n["quant"]["op"] == "Pow2Quantize":
                    quant = {"kind": "pow2", "sign": qa.get("sign", True), "with_zero": qa.get("with_zero", True),
                             "n": qa.get("n", 8), "m": qa.get("m", 1)}
                else:
                    quant = {"kind": "minmax", "decay": qa.get("decay", 0.999), "x_min_max": qa.get("x_min_max", False),
                             "ema": qa.get("ema", False), "eps": qa.get("eps", 0.01), "qr_min": qi[0], "qr_max": qi[1],
                             "ql_min": qi[2], "ql_max": qi[3]}
            y = ops.fused_dw_bn_quant(i[0], i[1], b, beta, gamma, mean, var, ba.get("eps", 1e-5), ca.get("pad"),
                                      ca.get("stride"), ca.get("dilation"), ca.get("multiplier", 1), quant,
                                      ca.get("base_axis", 1), comm=comm)
        elif n["op"] in ACTIVATIONS:
            y = i[0].clamp(min=0.0) if n["op"] == "ReLU" else i[0].clamp(0.0, 6.0)
        elif n["op"] == "Convolution":
            b = i[2] if len(i) > 2 else None
            y = ops.pointwise_convolution(i[0], i[1], b, a.get("base_axis", 1))
        elif n["op"] == FUSED_PW:
            nc = n["n_conv_inputs"]
            ca, ba = n["conv_args"], n["bn_args"]
            b = i[2] if nc > 2 else None
            n_bn = 4 - int(ba.get("no_bias", False)) - int(ba.get("no_scale", False))
            beta, gamma, mean, var = _bn_inputs(i[nc:nc + n_bn], ba)
            quant = None
            if n["quant"]:
                qa = n["quant"]["args"]
                if n["quant"]["op"] == "FixedPointQuantize":
                    quant = {"kind": "fpq", "sign": qa.get("sign", True), "n": qa.get("n", 8),
                             "delta": qa.get("delta", 2.0 ** -4)}
                else:
                    quant = {"kind": "pow2", "sign": qa.get("sign", True), "with_zero": qa.get("with_zero", True),
                             "n": qa.get("n", 8), "m": qa.get("m", 1)}
            if n.get("prepared_ws") is not None:  # parameters already in the workspace: one launch
                y = ops.fused_pw_bn_quant_prepared(i[0], i[1], n["prepared_ws"], True, quant, n["act"], ca.get("base_axis", 1))
            else:
                y = ops.fused_pw_bn_quant(i[0], i[1], b, beta, gamma, mean, var, ba.get("eps", 1e-5), quant, n["act"],
                                          ca.get("base_axis", 1))
        else:
            raise NotImplementedError("operator %r is outside the dwbnq path" % (n["op"],))
        t[n["outputs"][0]] = y
    if check:
        ops.check_device_flag()
    return t


def prepare_pointwise(nodes, tensors):
    """For parameters that stay as they are between runs (inference): returns a copy of the node
    list in which every FusedPwBnQuant node owns a workspace already filled from its weights,
    bias and BN vectors (``dwbnq_pwconv_prepare``), so that ``execute`` launches one kernel per
    such node instead of two. The nodes' inputs must have reached ``tensors`` with their run-time
    shapes: the graph input and the parameters are enough, shapes follow from the weights."""
    from . import ops
    import torch

    out, shape_of = [], {k: tuple(v.shape) for k, v in tensors.items() if v is not None}
    for n in nodes:
        n = dict(n)
        if n["op"] == FUSED_PW:
            nc, ba, ca = n["n_conv_inputs"], n["bn_args"], n["conv_args"]
            i = [None] + [tensors[v] if v is not None else None for v in n["inputs"][1:]]  # x: only its shape
            n_bn = 4 - int(ba.get("no_bias", False)) - int(ba.get("no_scale", False))
            beta, gamma, mean, var = _bn_inputs(i[nc:nc + n_bn], ba)
            x_shape = shape_of[n["inputs"][0]]
            x_like = torch.empty(x_shape, dtype=i[1].dtype, device="meta")
            n["prepared_ws"] = ops.pwconv_prepare(x_like, i[1], i[2] if nc > 2 else None, beta, gamma, mean, var,
                                                  ba.get("eps", 1e-5), n["act"], ca.get("base_axis", 1))
        # output shapes of the operators this library knows, for the nodes further down
        src = shape_of.get(n["inputs"][0])
        if src is not None:
            if n["op"] in (FUSED_PW, "Convolution"):
                w = shape_of[n["inputs"][1]]
                a = n.get("conv_args", n.get("args", {}))
                ax = a.get("base_axis", 1)
                shape_of[n["outputs"][0]] = src[:ax] + (w[0],) + src[ax + 1:]
            elif n["op"] in (FUSED, "DepthwiseConvolution"):
                w = shape_of[n["inputs"][1]]
                a = n.get("conv_args", n.get("args", {}))
                ax = a.get("base_axis", 1)
                pad, stride, dil = (a.get(k) or d for k, d in (("pad", (0, 0)), ("stride", (1, 1)), ("dilation", (1, 1))))
                sp = tuple((src[ax + 1 + j] + 2 * pad[j] - dil[j] * (w[-len(pad) + j] - 1) - 1) // stride[j] + 1
                           for j in range(len(pad)))
                shape_of[n["outputs"][0]] = src[:ax] + (src[ax] * a.get("multiplier", 1),) + sp
            else:
                shape_of[n["outputs"][0]] = src
        out.append(n)
    return out


class GraphRunner:
    """A node list captured once into a CUDA graph and replayed: the host launches one graph
    instead of one kernel per node (what matters at small batches, where the kernels are
    shorter than their launches). The tensors dict passed in is the graph's memory: write new
    inputs into its tensors in place (``copy_``), call ``replay()``, read the outputs from it.
    Parameters are taken as constant (``prepare_pointwise``) unless ``prepare=False``.
    Nodes that need a communicator are not captured (run them with ``execute``)."""

    def __init__(self, nodes, tensors, warmup=2, prepare=True):
        import torch
        self.nodes, self.tensors = (prepare_pointwise(nodes, tensors) if prepare else list(nodes)), tensors
        dev = next(t.device for t in tensors.values() if t is not None)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):  # first-call set-up (tables, symbol look-ups) and allocations
                execute(self.nodes, self.tensors)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                execute(self.nodes, self.tensors)
        torch.cuda.current_stream(dev).wait_stream(side)

    def replay(self):
        self.graph.replay()
        return self.tensors

    def synchronize(self):
        """Waits for the replays issued so far and raises if a kernel gave up one of its
        bounded waits: call it where the outputs are read."""
        from . import ops
        ops.check_device_flag()
        return self.tensors


def _bn_inputs(rest, args):
    """BatchNormalization inputs after x: [beta, gamma, mean, var] with beta / gamma absent
    when no_bias / no_scale (src/nbla/cuda/function/generic/batch_normalization.cu:120-123)."""
    rest = list(rest)
    beta = None if args.get("no_bias", False) else rest.pop(0)
    gamma = None if args.get("no_scale", False) else rest.pop(0)
    return beta, gamma, rest[0], rest[1]


def from_nnabla(output_variable):
    """Builds the node list from an nnabla graph (needs nnabla; import guarded).

    Returns (nodes, names, shapes): the node list in forward order, the Variable -> name map
    and the name -> shape map ``fuse_dw_bn_quant`` uses to tell a per-channel MinMaxQuantize
    from a per-tensor one. Walks the graph with ``Variable.visit``, reading each function's
    ``info.type_name`` / ``info.args`` and its ``inputs`` / ``outputs``."""
    try:
        import nnabla  # noqa: F401
    except ImportError as e:
        raise ImportError("from_nnabla needs the nnabla package") from e
    nodes, names, shapes = [], {}, {}

    def name(v):
        n = names.setdefault(v, "v%d" % len(names))
        shapes.setdefault(n, tuple(int(d) for d in v.shape))
        return n

    def visit(f):
        nodes.append({"op": f.info.type_name, "args": dict(f.info.args), "inputs": [name(v) for v in f.inputs],
                      "outputs": [name(v) for v in f.outputs]})

    output_variable.visit(visit)
    return nodes, names, shapes
