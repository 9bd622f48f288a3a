"""Host-to-device staging of batches on a copy stream.

The reference moves every batch inside the step, synchronously (``convert_to_tensor`` in
keras/src/trainers/data_adapters/array_data_adapter.py:289-303, called from the hot loop of
keras/src/backend/torch/trainer.py:356-416).  Here a batch is copied as soon as it is pulled from the data adapter,
on a stream of its own, from pinned memory; the step that consumes it only makes its compute stream wait for the
copy's event.  With the trainers' look-ahead loop the copy of batch i+1 runs while batch i is computing.
"""

import numpy as np
import torch

from keras_b200 import tree
from keras_b200.core.tensor import convert_to_tensor, get_device


class Staged:
    """A batch whose tensors are (being) copied to the device; ``event`` completes when they have arrived."""

    __slots__ = ("data", "event")

    def __init__(self, data, event):
        self.data, self.event = data, event


def _host_tensor(x):
    """numpy array → CPU tensor with the dtypes the kernels accept (float64 → float32, unsigned → signed)."""
    if x.dtype == np.float64:
        x = x.astype(np.float32)
    elif x.dtype == np.uint16:
        x = x.astype(np.int32)
    elif x.dtype in (np.uint32, np.uint64):
        x = x.astype(np.int64)
    return torch.from_numpy(np.ascontiguousarray(x))


class DeviceStager:
    """``stage(batch)`` starts the copies, ``acquire(staged)`` hands the device batch to the current stream."""

    def __init__(self, device=None):
        self.device = device if device is not None else get_device()
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    @property
    def active(self):
        return self.stream is not None

    def _move(self, x):
        if x is None or isinstance(x, (int, float, bool, str)):
            return x
        if isinstance(x, np.ndarray):
            if x.dtype.kind in "OUS":
                return x
            t = _host_tensor(x)
            return t.pin_memory().to(self.device, non_blocking=True) if self.stream is not None else t
        if isinstance(x, torch.Tensor):
            if x.device != self.device:
                return x.to(self.device, non_blocking=True)
            return x
        return convert_to_tensor(x)

    def stage(self, batch):
        if isinstance(batch, Staged):
            return batch
        if self.stream is None:
            return Staged(tree.map_structure(self._move, batch), None)
        with torch.cuda.stream(self.stream):
            moved = tree.map_structure(self._move, batch)
            event = torch.cuda.Event()
            event.record(self.stream)
        return Staged(moved, event)

    def acquire(self, staged):
        """Device batch of ``staged``, safe to use on the current stream."""
        if not isinstance(staged, Staged):
            staged = self.stage(staged)
        if staged.event is not None:
            current = torch.cuda.current_stream(self.device)
            current.wait_event(staged.event)
            for t in tree.flatten(staged.data):
                if isinstance(t, torch.Tensor) and t.is_cuda:
                    t.record_stream(current)  # the copy stream allocated it; the compute stream uses it
        return staged.data
