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
