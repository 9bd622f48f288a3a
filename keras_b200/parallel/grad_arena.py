"""Flat gradient storage shared by the optimizer and the data-parallel reducer.

Gradients of all trainable variables live in one buffer per dtype, in reverse creation order (the
order in which backward produces them), each padded to 128 bytes.  ``param.grad`` is a view into
the buffer, so autograd accumulates in place and every pointer is stable across steps.
"""

import torch


class GradArena:
    ALIGN = 32  # elements (128 bytes for fp32)

    @classmethod
    def required_numel(cls, variables):
        return sum((v._value.numel() + cls.ALIGN - 1) // cls.ALIGN * cls.ALIGN for v in variables)

    def __init__(self, variables, flat=None):
        self.signature = tuple(id(v) for v in variables)
        self.variables = list(variables)
        params = [v._value for v in variables]
        dev = params[0].device
        self.offsets = {}
        total = 0
        # reverse order: the last layers' gradients are ready first and sit at the front
        for idx in range(len(params) - 1, -1, -1):
            p = params[idx]
            self.offsets[idx] = total
            n = p.numel()
            total += (n + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.total = total
        if flat is not None:
            if flat.numel() < total or flat.dtype != torch.float32:
                raise ValueError("external gradient storage is too small")
            flat.zero_()
            self.flat = flat
        else:
            self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        self.views = []
        for idx, p in enumerate(params):
            off = self.offsets[idx]
            if p.dtype == torch.float32:
                self.views.append(self.flat[off:off + p.numel()].view(p.shape))
            else:
                self.views.append(None)

        # indices of variables that the first backward pass did not reach (``None`` until ``adopt`` has looked): they get no
        # gradient, so the optimizer skips them as it would skip a ``None`` gradient (no decay, no moment update)
        self.unused = None

    def bind(self):
        for v, view in zip(self.variables, self.views):
            p = v._value
            if view is not None and p.grad is not view:
                p.grad = view

    def unbind(self):
        """Detach every ``.grad`` so that the next backward pass shows which variables it reaches."""
        for v in self.variables:
            v._value.grad = None

    def adopt(self):
        """After a backward pass that ran unbound: note the variables without a gradient, move the gradients that exist into
        the arena and bind."""
        self.unused = set()
        with torch.no_grad():
            for idx, (v, view) in enumerate(zip(self.variables, self.views)):
                g = v._value.grad
                if g is None:
                    if getattr(v, "_gradient_is_zero_when_absent", False) and view is not None:
                        continue  # known to be zero (a bias folded into a batch normalization): its zeroed slot is its gradient
                    self.unused.add(idx)
                elif view is not None:
                    view.copy_(g)
        self.bind()

    def gradients(self):
        """Per variable: its gradient view, or ``None`` for a variable the model does not use."""
        unused = self.unused or ()
        return [None if idx in unused else v._value.grad for idx, v in enumerate(self.variables)]

    def zero(self):
        self.flat.zero_()
