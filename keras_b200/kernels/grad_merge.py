"""One gradient buffer for an activation with two consumers.

In a residual block the block input feeds a convolution and, further on, the add of the skip connection (or a second,
projecting convolution).  Autograd would produce one gradient tensor per consumer and add them with an elementwise
kernel: three passes over an activation-sized tensor.  Here the activation carries a ``MergeSlot``; the consumer whose
backward runs first leaves its gradient tensor in the slot and returns it as usual, the other one adds its own result
into that very buffer (the convolution's data-gradient kernel stores with a TMA reduce-add) and returns nothing.  The
autograd engine hands the producer of the activation the one buffer once both consumers are done, as it would have
handed it the sum.  Only inside the trainer's backward pass (``shadow.arena_backward``); anywhere else every consumer
returns its own gradient.
"""

import os

import torch

from keras_b200.kernels import shadow

_ENABLED = os.environ.get("KERAS_B200_GRAD_MERGE", "1") != "0"


class MergeSlot:
    __slots__ = ("buffer",)

    def __init__(self):
        self.buffer = None


def mark(tensor):
    """Give ``tensor`` a slot (when gradients will flow through it)."""
    if _ENABLED and isinstance(tensor, torch.Tensor) and tensor.requires_grad and torch.is_grad_enabled():
        tensor._kb_merge = MergeSlot()
    return tensor


def slot_of(tensor):
    return getattr(tensor, "_kb_merge", None) if isinstance(tensor, torch.Tensor) else None


def target(slot, shape, dtype):
    """The buffer to add into, when another consumer has already left a matching one."""
    if slot is None or not shadow.in_arena_backward():
        return None
    buf = slot.buffer
    if buf is None or tuple(buf.shape) != tuple(shape) or buf.dtype != dtype or not buf.is_contiguous() or buf.data_ptr() % 16:
        return None
    return buf


def offer(slot, grad):
    """Leave ``grad`` (this consumer's gradient tensor, returned to autograd as it is) for the other consumer to add into."""
    if slot is not None and shadow.in_arena_backward() and slot.buffer is None and grad is not None and grad.is_contiguous():
        slot.buffer = grad
