"""Writes tests/golden/layers_small.npz: outputs of the CPU oracle on small seeded layers (depthwise
layers, and pointwise layers with exactly summable inputs).

These vectors freeze the oracle's behaviour (a regression anchor for the oracle and a fixed
target for the CUDA path); they are NOT reference-generated - nnabla core, whose CPU classes
they restate, is not installed in this environment. The vectors derived by hand from the
reference sources are in known_answers.json.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
for p in (ROOT, os.path.join(ROOT, "nnabla-ext-cuda_b200", "python")):
    if p not in sys.path:
        sys.path.insert(0, p)

from dwbnq import workloads  # noqa: E402
from oracle import oracle  # noqa: E402

CASES = {
    "fpq_3x3_s1": workloads.LayerSpec("g0", 2, 5, 9, 11, 3, 1, 1, dict(workloads.FPQ_CFG0), seed=11),
    "fpq_3x3_s2": workloads.LayerSpec("g1", 2, 4, 14, 14, 3, 2, 1, dict(workloads.FPQ_CFG1), seed=12, x_dist="relu6"),
    "pow2_5x5_s1": workloads.LayerSpec("g2", 1, 3, 12, 10, 5, 1, 2, dict(workloads.POW2_CFG2), seed=13),
    "minmax_3x3_s2": workloads.LayerSpec("g3", 3, 6, 8, 8, 3, 2, 1, dict(workloads.MINMAX_CFG3), seed=14,
                                         x_dist="normal2_outliers"),
}


# Pointwise layers whose sums are exact in binary32 whatever their order: activations k / 8 and
# weights m / 16 with small integers k, m (what a quantized network carries), so every product has
# at most 12 significant bits and every sum at most 22. The golden convolution is therefore THE
# result, and a CUDA path that splits factors (TF32 halves) or reorders the sum must still hit it
# bit for bit; the epilogue behind it is exact arithmetic anyway.
#   name: (n, c_in, c_out, h, w, activation, quantizer)
PW_CASES = {
    "pw_expand_16_96": (3, 16, 96, 12, 12, "relu6", dict(workloads.FPQ_CFG1)),
    "pw_project_384_64": (2, 384, 64, 7, 7, None, dict(workloads.FPQ_CFG0)),
    "pw_odd_30_50": (2, 30, 50, 5, 9, "relu", dict(workloads.POW2_CFG2)),  # c_in not a multiple of 4: the FMA kernel
}


def pw_data(name):
    n, ci, co, h, w, act, quant = PW_CASES[name]
    rng = np.random.default_rng(sum(map(ord, name)))
    d = {"x": (rng.integers(-40, 56, (n, ci, h, w)) / 8.0).astype(np.float32),
         "w": (rng.integers(-31, 32, (co, ci, 1, 1)) / 16.0).astype(np.float32),
         "b": (rng.integers(-24, 25, co) / 8.0).astype(np.float32),
         "mean": rng.standard_normal(co).astype(np.float32), "var": (rng.random(co) * 20 + 5).astype(np.float32),
         "gamma": (rng.random(co) + 0.5).astype(np.float32), "beta": rng.standard_normal(co).astype(np.float32)}
    return d, act, quant


def compute_pw(name):
    d, act, quant = pw_data(name)
    acc32, acc64, _ = oracle.pwconv(d["x"], d["w"], d["b"])
    assert np.array_equal(acc32, acc64.astype(np.float32)), "the sums of this case are meant to be exact"
    y = oracle.pw_epilogue(acc32, d["beta"], d["gamma"], d["mean"], d["var"], 1e-5, act, quant)
    return d, {"conv": acc32, "y": y}


def compute(spec):
    d = workloads.make_layer_data(spec)
    q = workloads.quant_for_ops(spec, d)
    out = oracle.fused_layer(d["x"], d["w"], d["b"], d["beta"], d["gamma"], d["mean"], d["var"], spec.bn_eps,
                             (spec.stride,) * 2, (spec.pad,) * 2, q, return_prequant=True)
    res, pre = out
    r = {"pre": pre}
    if spec.quant["kind"] == "minmax":
        r["y"], r["qr_min"], r["qr_max"] = res
    else:
        r["y"] = res
    return d, r


def main():
    blob = {}
    for name, spec in CASES.items():
        _, r = compute(spec)
        for k, v in r.items():
            blob["%s.%s" % (name, k)] = v
    for name in PW_CASES:
        _, r = compute_pw(name)
        for k, v in r.items():
            blob["%s.%s" % (name, k)] = v
    np.savez_compressed(os.path.join(HERE, "layers_small.npz"), **blob)
    print("wrote", len(blob), "arrays")


if __name__ == "__main__":
    main()
