"""Communicator for the one exchange of the path: the all-reduce(max) of MinMaxQuantize's
per-channel [max, -min] vector when the reduced batch is sharded over GPUs.

The NCCL communicator lives inside libdwbnq (created from a 128-byte unique id);
torch.distributed is only the out-of-band channel that carries the id from rank 0 to the
other ranks, the role MPI_Bcast plays in the reference
(src/nbla/cuda/communicator/multi_process_data_parallel_communicator.cu:415-421).
"""
import ctypes

import torch

from . import _lib as L


class Communicator:
    def __init__(self, handle, rank, nranks, device):
        self.handle = ctypes.c_void_p(handle)
        self.rank, self.nranks, self.device = rank, nranks, device

    @classmethod
    def from_torch_distributed(cls, device):
        """Call on every rank of an initialised torch.distributed job (one GPU per rank)."""
        import torch.distributed as dist
        rank, nranks = dist.get_rank(), dist.get_world_size()
        buf = (ctypes.c_ubyte * L.UNIQUE_ID_BYTES)()
        if rank == 0:
            L.check(L.lib().dwbnq_comm_get_unique_id(buf))
        idt = torch.tensor(list(buf), dtype=torch.uint8)
        if dist.get_backend() == "nccl":
            idt = idt.to(device)
        dist.broadcast(idt, src=0)
        raw = bytes(idt.cpu().tolist())
        out = ctypes.c_void_p()
        L.check(L.lib().dwbnq_comm_create(raw, nranks, rank, device.index, ctypes.byref(out)))
        return cls(out.value, rank, nranks, device)

    def allreduce_max_(self, t, timeout_ms=0):
        """In-place all-reduce(max) of a float32 CUDA tensor on the current stream."""
        assert t.dtype == torch.float32 and t.is_cuda and t.is_contiguous()
        stream = ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
        L.check(L.lib().dwbnq_comm_allreduce_max_f32(self.handle, ctypes.c_void_p(t.data_ptr()), t.numel(), stream,
                                                     int(timeout_ms)))
        return t

    def destroy(self):
        if self.handle:
            L.check(L.lib().dwbnq_comm_destroy(self.handle))
            self.handle = ctypes.c_void_p()


def shard_range(n_total, rank, nranks):
    """Contiguous batch slice [first, first + count) of rank `rank`: NCHW makes it one
    contiguous byte range. The first n_total % nranks ranks take one extra image."""
    base, extra = divmod(n_total, nranks)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count
