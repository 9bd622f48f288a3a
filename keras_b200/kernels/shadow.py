"""bf16 shadow copies of fp32 variables.

Under ``mixed_bfloat16`` every layer reads its fp32 variables in bf16.  Instead of one cast kernel
per variable per step, the fused optimizer writes a bf16 copy of each parameter as part of its
update; reads return that copy through an autograd function whose backward hands the gradient to
the fp32 parameter.
"""

import torch

_arena_backward_depth = 0


class arena_backward:
    """Scope of a backward pass whose parameter gradients live in persistent fp32 storage bound to ``.grad`` (the
    gradient arena).  Inside it, kernels that produce a weight gradient may add it into ``param.grad`` themselves and
    send nothing back through autograd; outside it (``torch.autograd.grad`` in user code, say) they return gradients."""

    def __enter__(self):
        global _arena_backward_depth
        _arena_backward_depth += 1
        return self

    def __exit__(self, *exc):
        global _arena_backward_depth
        _arena_backward_depth -= 1
        return False


def in_arena_backward():
    return _arena_backward_depth > 0


_slot_observer = None


def set_slot_observer(fn):
    """``fn(param)`` is called whenever ``grad_slot`` hands out a parameter's gradient storage, that is, just before a kernel
    adds a contribution to it (the data-parallel engine counts these to know when a gradient is complete).  ``None`` clears."""
    global _slot_observer
    _slot_observer = fn


def grad_slot(param, shape=None):
    """``param.grad`` when a kernel may accumulate into it: inside ``arena_backward``, fp32, contiguous, 16-byte aligned."""
    if _arena_backward_depth <= 0 or param is None:
        return None
    g = param.grad
    if g is None or g.dtype != torch.float32 or g.requires_grad or not g.is_contiguous() or g.data_ptr() % 16:
        return None
    if shape is not None and g.numel() != _numel(shape):
        return None
    if _slot_observer is not None:
        _slot_observer(param)
    return g


def _numel(shape):
    n = 1
    for d in shape:
        n *= int(d)
    return n


def shadows_for(variables):
    """List of bf16 shadow tensors (or ``None``) aligned with ``variables``."""
    out = []
    any_shadow = False
    for v in variables:
        sh = getattr(v, "_shadow_tensor", None)
        out.append(sh)
        any_shadow = any_shadow or sh is not None
    return out if any_shadow else None


class _ShadowRead(torch.autograd.Function):
    """Reads the bf16 shadow; backward hands the gradient to the fp32 parameter.  When the parameter's ``.grad`` is bound
    to persistent fp32 storage (the gradient arena), the bf16 gradient is added into it directly: one kernel instead of
    a cast to fp32 followed by autograd's accumulation."""

    @staticmethod
    def forward(ctx, param, shadow):
        ctx.param = param
        # a consumer that already added its gradient into the parameter's fp32 storage sends nothing back
        ctx.set_materialize_grads(False)
        return shadow.view_as(shadow)

    @staticmethod
    def backward(ctx, grad):
        if grad is None:
            return None, None
        g = grad_slot(ctx.param, grad.shape)
        if g is not None:
            g.view(grad.shape).add_(grad)
            return None, None
        return grad.float(), None


def attach(variables):
    """Create shadows for fp32 CUDA variables that are read with autocast.

    A shadow remembers the version counter of its parameter: any in-place torch update of the parameter (an unfused
    optimizer, ``assign``, weight loading) is noticed at the next read and the shadow is refreshed with one cast; the
    fused optimizer kernels write parameter and shadow together through raw pointers and leave the counter alone."""
    from keras_b200.kernels import ops

    for v in variables:
        p = v._value
        if p is None or not p.is_cuda or p.dtype != torch.float32 or not v._autocast or getattr(v, "_shadow_tensor", None) is not None:
            continue
        sh = torch.empty_like(p, dtype=torch.bfloat16)
        ops.cast_f32_to_bf16(p.detach().reshape(-1), sh.reshape(-1))
        v._shadow_tensor = sh
        state = {"version": p._version, "ptr": p.data_ptr()}

        def read(value, _v=v, _sh=sh, _state=state):
            p_now = _v._value
            if p_now._version != _state["version"] or p_now.data_ptr() != _state["ptr"]:
                if p_now.shape != _sh.shape or not p_now.is_cuda:
                    return value.to(torch.bfloat16)
                ops.cast_f32_to_bf16(p_now.detach().reshape(-1), _sh.reshape(-1))
                _state["version"], _state["ptr"] = p_now._version, p_now.data_ptr()
            if value.requires_grad and torch.is_grad_enabled():
                return _ShadowRead.apply(value, _sh)
            return _sh

        def invalidate(_v=v, _sh=sh, _state=state):
            """The parameter was assigned (``assign``, weight loading): refresh the shadow now.  A recorded training step reads
            the shadow without coming back to Python, so "at the next read" would be one step too late."""
            p_now = _v._value
            if p_now is not None and p_now.is_cuda and p_now.shape == _sh.shape and p_now.dtype == torch.float32:
                ops.cast_f32_to_bf16(p_now.detach().reshape(-1), _sh.reshape(-1))
                _state["version"], _state["ptr"] = p_now._version, p_now.data_ptr()
            else:
                _state["version"] = -1

        v._shadow = (torch.bfloat16, read, invalidate)


def attach_for_model(model, variables):
    """Attach shadows when ``model`` computes in bfloat16 on fp32 variables (``mixed_bfloat16``); switch off with
    ``KERAS_B200_SHADOW_WEIGHTS=0``."""
    import os

    if os.environ.get("KERAS_B200_SHADOW_WEIGHTS", "1") == "0" or not variables:
        return
    if getattr(model, "_shadows_checked", None) == tuple(id(v) for v in variables):
        return
    model._shadows_checked = tuple(id(v) for v in variables)
    try:
        mixed = any(getattr(layer, "compute_dtype", None) == "bfloat16" and getattr(layer, "variable_dtype", None) == "float32"
                    for layer in model._flatten_layers())
    except Exception:
        mixed = False
    if mixed:
        attach(variables)


def detach(variables):
    for v in variables:
        v._shadow = None
        v._shadow_tensor = None
