"""Collectives used by the parallel engines.

Mode (``KERAS_B200_COMM``):

* ``p2p`` (default on CUDA): this package's kernels over IPC-mapped peer memory (two-shot all-reduce in place);
* ``nccl``: ``torch.distributed`` on the NCCL group (also the path for CPU/gloo jobs, where it is the only one).

Replaces the per-bucket NCCL all-reduce of DistributedDataParallel and the one-all-reduce-per-metric-variable loop
of the reference (keras/src/backend/torch/trainer.py:83-92,207-244).
"""

import ctypes
import os

import torch
import torch.distributed as dist

from keras_b200.core import config
from keras_b200.parallel import process_groups


def comm_timeout_ms():
    return int(os.environ.get("KERAS_B200_COMM_TIMEOUT_MS", "20000"))


class CommError(RuntimeError):
    """A bounded wait inside a communication kernel ran out (a peer did not arrive)."""


class P2PAllReducer:
    """In-place sum (or mean) all-reduce of a symmetric fp32 arena with this package's kernel.

    ``arena`` is a ``SymmetricBuffer``-backed flat fp32 tensor allocated by ``allocate``.  Each call takes
    one kernel pair on the current stream; completion is ordered by the stream, no host synchronisation.
    """

    def __init__(self, numel, group=None, ranks=None):
        from keras_b200.parallel.symmetric import SymmetricBuffer

        self.numel = (int(numel) + 3) // 4 * 4
        self.buffer = SymmetricBuffer(max(self.numel, 4) * 4, group, ranks)
        self.signals = SymmetricBuffer(256, group, ranks)
        self.flat = self.buffer.tensor(torch.float32)
        self.rank, self.world = self.buffer.rank, self.buffer.world
        self.epoch = 0  # host-side count of calls issued (bookkeeping); the epoch the kernels use lives in `epoch_ctr`
        self.epoch_ctr = torch.zeros(1, dtype=torch.int32, device=self.flat.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.flat.device)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_event = None

    def _collective(self, mode, offset, numel, scale=1.0, root=0):
        from keras_b200.kernels import ops as kops

        lib = kops._lib()
        n = self.numel - offset if numel is None else int(numel)
        recording = torch.cuda.is_current_stream_capturing()
        if not recording:
            self.check()
        self.epoch += 1
        # epoch argument 1 + device counter: identical launch arguments for every call, so a recorded step can be replayed
        kops._check(lib.kb200_collective_p2p(self.buffer.ptr_array, self.signals.ptr_array, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                             ctypes.c_longlong(offset), ctypes.c_longlong(n), ctypes.c_float(scale), ctypes.c_uint(1),
                                             ctypes.c_void_p(self.epoch_ctr.data_ptr()), ctypes.c_longlong(comm_timeout_ms()),
                                             ctypes.c_void_p(self.status.data_ptr()), ctypes.c_int(mode), ctypes.c_int(root), kops._stream()),
                    "collective_p2p")
        if not recording:
            self.post_status()

    def post_status(self):
        """Queue a copy of the device status word to the host (read by ``check`` once it has landed).  A replayed recording
        of collectives calls this after each replay: events cannot be recorded for later queries inside a recording."""
        self._status_host.copy_(self.status, non_blocking=True)
        self._status_event = torch.cuda.Event()
        self._status_event.record()

    def all_reduce(self, offset=0, numel=None, scale=1.0):
        """Region := scale * sum over ranks, in every arena."""
        self._collective(0, offset, numel, scale)

    def reduce_scatter(self, offset=0, numel=None, scale=1.0):
        """Slice ``rank`` of the region (``ceil(numel / 4 / world)`` float4 vectors per slice) := scale * sum over ranks; the other
        slices of this arena keep their local values."""
        self._collective(1, offset, numel, scale)

    def all_gather(self, offset=0, numel=None):
        """Every rank's slice ``rank`` of the region is copied into the same slice of every arena."""
        self._collective(2, offset, numel)

    def broadcast(self, root=0, offset=0, numel=None):
        """The region of rank ``root`` is copied into every arena."""
        self._collective(3, offset, numel, root=root)

    def check(self, wait=False):
        """Raise if an earlier call timed out.  Without ``wait`` only completed status copies are inspected."""
        ev = self._status_event
        if ev is None:
            return
        if wait:
            ev.synchronize()
        if ev.query():
            code = int(self._status_host[0])
            if code != 0:
                raise CommError(f"all-reduce kernel gave up waiting (phase {code // 256}, peer index {code % 256 - 1}); a rank is missing or stalled")

    def close(self):
        self.buffer.close()
        self.signals.close()


def use_p2p(device):
    return device.type == "cuda" and config.comm_mode() in ("p2p", "nvls") and process_groups.world_size() > 1


def all_reduce(tensor, group=None, average=False):
    """Library all-reduce (NCCL on CUDA tensors, gloo on CPU tensors), in place."""
    if not process_groups.is_initialized() or dist.get_world_size(group) == 1:
        return tensor
    if tensor.is_cuda or dist.get_backend(group) == "gloo":
        try:
            dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group)
        except RuntimeError as e:
            from keras_b200.parallel import watchdog

            watchdog.explain_collective_error(e)  # raises RankFailure when a peer is known to be lost
            raise
    else:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=process_groups.host_group())
    if average:
        tensor.div_(dist.get_world_size(group))
    return tensor


def broadcast(tensor, src=0, group=None):
    if process_groups.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(tensor, src=src, group=group)
    return tensor


def all_gather(tensor, group=None, dim=0):
    if not process_groups.is_initialized() or dist.get_world_size(group) == 1:
        return tensor
    parts = [torch.empty_like(tensor) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, tensor.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


def reduce_scatter(tensor, group=None, dim=0):
    if not process_groups.is_initialized() or dist.get_world_size(group) == 1:
        return tensor
    n = dist.get_world_size(group)
    chunks = [c.contiguous() for c in tensor.chunk(n, dim=dim)]
    out = torch.empty_like(chunks[0])
    if tensor.is_cuda:
        dist.reduce_scatter(out, chunks, group=group)
    else:
        dist.all_reduce(tensor, group=group)
        out = tensor.chunk(n, dim=dim)[dist.get_rank(group)].contiguous()
    return out


def barrier():
    if process_groups.is_initialized():
        dist.barrier(group=process_groups.host_group())
