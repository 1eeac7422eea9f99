"""Every GPU of the box (2 to 8), one process each: the batch of a MinMaxQuantize layer is
sharded by image, the library's NCCL communicator all-reduces the per-channel [max, -min]
vector between the two passes, and the concatenated result must be bit-identical to the
single-process oracle on the full batch - for an uneven split and for a batch with fewer
images than ranks (the ranks with an empty shard still join the collective and derive the
same ranges). Skipped on a box with one GPU (the gloo test covers the host logic there)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, ".."))
SHAPES = [(14, 2), (28, 1), (56, 2)]  # plane kernels and the tiled family


def _batches(world):
    return [2 * world + 1, max(1, world - 1)]  # uneven split; fewer images than ranks


def _worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "nnabla-ext-cuda_b200", "python")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from dwbnq import ops, workloads
    from dwbnq.comm import Communicator, shard_range

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    comm = Communicator.from_torch_distributed(device)
    for n_total in _batches(world):
        for hw, stride in SHAPES:
            spec = workloads.LayerSpec("shard", n_total, 24, hw, hw, 3, stride, 1, dict(workloads.MINMAX_CFG3),
                                       seed=4, x_dist="normal2_outliers")
            first, count = shard_range(n_total, rank, world)
            d = workloads.make_layer_data(spec, n=count, first_image=first)
            t = {k: torch.from_numpy(v).to(device) for k, v in d.items()}
            q = workloads.quant_for_ops(spec, t)
            y = ops.fused_dw_bn_quant(t["x"], t["w"], t["b"], t["beta"], t["gamma"], t["mean"], t["var"],
                                      spec.bn_eps, pad=(1, 1), stride=(stride, stride), quant=q, comm=comm)
            torch.cuda.synchronize()
            ops.check_device_flag()
            tag = "%d_%d_%d_%d" % (n_total, hw, stride, rank)
            np.save(os.path.join(out_dir, "y_%s.npy" % tag), y.cpu().numpy())
            np.save(os.path.join(out_dir, "r_%s.npy" % tag),
                    np.stack([t["qr_min"].cpu().numpy(), t["qr_max"].cpu().numpy()]))
    comm.destroy()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_all_gpus_reproduce_the_single_process_result(tmp_path, oracle):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs two GPUs")
    from dwbnq import workloads
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for n_total in _batches(world):
        for hw, stride in SHAPES:
            spec = workloads.LayerSpec("shard", n_total, 24, hw, hw, 3, stride, 1, dict(workloads.MINMAX_CFG3),
                                       seed=4, x_dist="normal2_outliers")
            d = workloads.make_layer_data(spec)
            q = workloads.quant_for_ops(spec, d)
            want, qmin, qmax = oracle.fused_layer(d["x"], d["w"], d["b"], d["beta"], d["gamma"], d["mean"], d["var"],
                                                  1e-5, (stride, stride), (1, 1), q)
            got = np.concatenate([np.load(tmp_path / ("y_%d_%d_%d_%d.npy" % (n_total, hw, stride, r)))
                                  for r in range(world)])
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (world, n_total, hw, stride)
            for r in range(world):  # every rank, the empty ones included, holds the global ranges
                rr = np.load(tmp_path / ("r_%d_%d_%d_%d.npy" % (n_total, hw, stride, r)))
                np.testing.assert_array_equal(rr[0], qmin)
                np.testing.assert_array_equal(rr[1], qmax)
