"""Committed golden vectors (tests/golden/layers_small.npz, produced by make_golden.py from
the CPU oracle): the oracle must keep reproducing them, and the CUDA path must hit them bit
for bit through every kernel family."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402

GOLD = np.load(os.path.join(HERE, "golden", "layers_small.npz"))


@pytest.mark.parametrize("name", list(make_golden.CASES))
def test_oracle_reproduces_golden(oracle, name):
    _, r = make_golden.compute(make_golden.CASES[name])
    for k, v in r.items():
        want = GOLD["%s.%s" % (name, k)]
        assert v.shape == want.shape and np.array_equal(v.view(np.uint32), want.view(np.uint32)), (name, k)


@pytest.mark.gpu
@pytest.mark.parametrize("path", [-1, 0, 1, 3], ids=["auto", "generic", "coop", "raw"])
@pytest.mark.parametrize("name", list(make_golden.CASES))
def test_cuda_path_hits_golden(cuda_device, name, path):
    import torch
    from dwbnq import ops, workloads
    spec = make_golden.CASES[name]
    d = workloads.make_layer_data(spec)
    t = {k: torch.from_numpy(v).to(cuda_device) for k, v in d.items()}
    q = workloads.quant_for_ops(spec, t)
    ops.set_forced_path(path)
    try:
        y = ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], spec.bn_eps,
                                  (spec.pad,) * 2, (spec.stride,) * 2, quant=q)
        pre = ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], spec.bn_eps,
                                    (spec.pad,) * 2, (spec.stride,) * 2, quant=None)
    finally:
        ops.set_forced_path(-1)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), GOLD[name + ".y"].view(np.uint32))
    assert np.array_equal(pre.cpu().numpy().view(np.uint32), GOLD[name + ".pre"].view(np.uint32))
    if spec.quant["kind"] == "minmax":
        np.testing.assert_array_equal(t["qr_min"].cpu().numpy(), GOLD[name + ".qr_min"])
        np.testing.assert_array_equal(t["qr_max"].cpu().numpy(), GOLD[name + ".qr_max"])


@pytest.mark.parametrize("name", list(make_golden.PW_CASES))
def test_oracle_reproduces_pointwise_golden(oracle, name):
    _, r = make_golden.compute_pw(name)
    for k, v in r.items():
        want = GOLD["%s.%s" % (name, k)]
        assert v.shape == want.shape and np.array_equal(v.view(np.uint32), want.view(np.uint32)), (name, k)
    # exactly summable: the double-precision sum, rounded once, is the same array
    d, _, _ = make_golden.pw_data(name)
    exact = np.einsum("nchw,oc->nohw", d["x"].astype(np.float64), d["w"][:, :, 0, 0].astype(np.float64)) + \
        d["b"].astype(np.float64)[None, :, None, None]
    assert np.array_equal(exact.astype(np.float32), GOLD[name + ".conv"]) and np.array_equal(exact, GOLD[name + ".conv"])


@pytest.mark.gpu
@pytest.mark.parametrize("math", ["fp32", "tf32"])
@pytest.mark.parametrize("name", list(make_golden.PW_CASES))
def test_pointwise_cuda_path_hits_golden_bit_for_bit(cuda_device, name, math):
    """Sums that are exact in binary32 leave no room for a tolerance: the tcgen05 kernel (three TF32
    passes or one - factors of at most 11 significant bits are exact in TF32), the FMA kernel, the
    fused and the prepared forms all return the golden bits."""
    import torch
    from dwbnq import ops
    d, act, quant = make_golden.pw_data(name)
    t = {k: torch.from_numpy(v).to(cuda_device) for k, v in d.items()}
    conv = ops.pointwise_convolution(t["x"], t["w"], t["b"], math=math)
    y = ops.fused_pw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, quant, act, math=math)
    ws = ops.pwconv_prepare(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"], 1e-5, act=act, math=math)
    y2 = ops.fused_pw_bn_quant_prepared(t["x"], t["w"], ws, True, quant, act, math=math)
    torch.cuda.synchronize()
    ops.check_device_flag()
    assert np.array_equal(conv.cpu().numpy().view(np.uint32), GOLD[name + ".conv"].view(np.uint32))
    assert np.array_equal(y.cpu().numpy().view(np.uint32), GOLD[name + ".y"].view(np.uint32))
    assert np.array_equal(y2.cpu().numpy().view(np.uint32), GOLD[name + ".y"].view(np.uint32))
    # binary16 tensors: the same values are exact in binary16 too (the result is rounded once to binary16)
    th = {k: v.half() for k, v in t.items()}
    yh = ops.fused_pw_bn_quant(th["x"], th["w"], th["b"], th["beta"], th["gamma"], th["mean"], th["var"], 1e-5, quant, act)
    convh = ops.pointwise_convolution(th["x"], th["w"], th["b"])
    want = GOLD[name + ".conv"].astype(np.float16)
    assert np.array_equal(convh.cpu().numpy().view(np.uint16), want.view(np.uint16))
    assert yh.dtype == torch.float16
