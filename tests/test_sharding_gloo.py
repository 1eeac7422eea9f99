"""The multi-GPU scheme on CPU: two gloo ranks shard a batch by image with the library's
shard_range, exchange the per-channel [max, -min] vector with an all-reduce(max) (what the
library does over NCCL between MinMaxQuantize's two passes) and quantize their shards; the
concatenation must be bit-identical to the single-process oracle on the full batch - also when
the batch has fewer images than ranks and a rank's shard is empty (its identities are neutral
under max). The arithmetic here is the oracle's: this checks the scheme and the sharding
function; the library's own collective is covered on GPUs by tests/test_multi_gpu.py and on
the host by tests/test_comm_failures.py."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, ".."))


def _worker(rank, world, port, n_total, out_dir):
    for p in (ROOT, os.path.join(ROOT, "nnabla-ext-cuda_b200", "python")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from dwbnq import workloads
    from dwbnq.comm import shard_range
    from oracle import oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = workloads.LayerSpec("shard", n_total, 12, 14, 14, 3, 2, 1, dict(workloads.MINMAX_CFG3), seed=4,
                               x_dist="normal2_outliers")
    first, count = shard_range(n_total, rank, world)
    d = workloads.make_layer_data(spec, n=count, first_image=first)
    pre = oracle.bn_infer(oracle.dwconv(d["x"], d["w"], d["b"], (2, 2), (1, 1)), d["beta"], d["gamma"], d["mean"],
                          d["var"], 1e-5)
    mn, mx = oracle.minmax_reduce(pre)
    packed = torch.from_numpy(np.concatenate([mx, -mn]))
    dist.all_reduce(packed, op=dist.ReduceOp.MAX)
    c = spec.c
    gmax, gmin = packed[:c].numpy(), -packed[c:].numpy()
    y, _, _ = oracle.minmaxq_from_ranges(pre, gmin, gmax, d["ql_min"], d["ql_max"], eps=0.01)
    np.save(os.path.join(out_dir, "y%d.npy" % rank), y)
    np.save(os.path.join(out_dir, "r%d.npy" % rank), np.stack([gmin, gmax]))
    dist.destroy_process_group()


def test_shard_range_covers_the_batch():
    for p in (ROOT, os.path.join(ROOT, "nnabla-ext-cuda_b200", "python")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from dwbnq.comm import shard_range
    for n, w in ((512, 8), (10, 4), (3, 8), (256, 1), (7, 2)):
        spans = [shard_range(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and sum(c for _, c in spans) == n
        for (f0, c0), (f1, _) in zip(spans, spans[1:]):
            assert f0 + c0 == f1
        assert max(c for _, c in spans) - min(c for _, c in spans) <= 1


@pytest.mark.timeout(180)
@pytest.mark.parametrize("n_total", [5, 1], ids=["uneven_3+2", "one_image_two_ranks"])
def test_two_ranks_reproduce_the_single_process_result(tmp_path, oracle, n_total):
    from dwbnq import workloads
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, n_total, str(tmp_path)), nprocs=world, join=True)
    spec = workloads.LayerSpec("shard", n_total, 12, 14, 14, 3, 2, 1, dict(workloads.MINMAX_CFG3), seed=4,
                               x_dist="normal2_outliers")
    d = workloads.make_layer_data(spec)
    q = workloads.quant_for_ops(spec, d)
    want, qmin, qmax = oracle.fused_layer(d["x"], d["w"], d["b"], d["beta"], d["gamma"], d["mean"], d["var"], 1e-5,
                                          (2, 2), (1, 1), q)
    got = np.concatenate([np.load(tmp_path / ("y%d.npy" % r)) for r in range(world)])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    for r in range(world):
        rr = np.load(tmp_path / ("r%d.npy" % r))
        np.testing.assert_array_equal(rr[0], qmin)
        np.testing.assert_array_equal(rr[1], qmax)
