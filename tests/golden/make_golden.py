"""Writes tests/golden/layers_small.npz: outputs of the CPU oracle on small seeded layers.

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
    np.savez_compressed(os.path.join(HERE, "layers_small.npz"), **blob)
    print("wrote", len(blob), "arrays")


if __name__ == "__main__":
    main()
