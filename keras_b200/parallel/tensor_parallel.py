"""Sharded variables for ``ModelParallel`` (the reference realises this only through JAX/GSPMD,
keras/src/backend/jax/distribution_lib.py:32-106; its torch backend converts layouts to DTensor placements but
never applies them to variables, keras/src/backend/torch/distribution_lib.py:186-310).

A variable whose ``TensorLayout`` names mesh axes on some dimensions stores only this rank's shard
(``Variable._value``); ``Variable.shape`` stays the logical (global) shape.  Reading ``variable.value`` outside
a shard-aware layer all-gathers the shards with an autograd-aware collective (backward keeps this rank's slice of
the gradient), which is always correct; layers that recognise the column/row pattern read the shard directly and
communicate activations instead.

Initialisation draws the full value from the seeded initializer on every rank (identical by construction, the
global seed is agreed at ``initialize``) and keeps the local slice, so a sharded model starts from exactly the
values of the unsharded one.
"""

import contextlib

import numpy as np
import torch
import torch.distributed as dist

from keras_b200.core import global_state
from keras_b200.parallel import process_groups


def _axis_info(layout, mesh_groups):
    """[(dim, parts, index, group)] for every sharded dimension of ``layout`` on this rank."""
    out = []
    mesh = layout.device_mesh
    for dim, axis in enumerate(layout.axes):
        if axis is None:
            continue
        size = mesh.shape[mesh.axis_names.index(axis)]
        if size <= 1:
            continue
        out.append((dim, size, mesh_groups.index(axis), mesh_groups.get_group(axis)))
    return out


def shard_slices(shape, layout):
    """Index tuple selecting this rank's shard of a tensor of ``shape`` laid out as ``layout`` (None: replicated)."""
    if layout is None or layout.device_mesh is None or not process_groups.is_initialized():
        return None
    info = _axis_info(layout, layout.device_mesh.backend_mesh)
    if not info:
        return None
    idx = [slice(None)] * len(shape)
    for dim, parts, index, _ in info:
        if shape[dim] % parts != 0:
            raise ValueError(f"Dimension {dim} of shape {tuple(shape)} is not divisible by the {parts} shards of mesh axis {layout.axes[dim]!r}.")
        step = shape[dim] // parts
        idx[dim] = slice(index * step, (index + 1) * step)
    return tuple(idx)


def distribute_tensor(tensor, layout):
    """This rank's shard of a full tensor (a view; replicated layouts return the tensor itself)."""
    sl = shard_slices(tuple(tensor.shape), layout)
    if sl is None:
        return tensor
    return tensor[sl]


def shard_variable_init(distribution, variable, initializer):
    layout = variable._layout
    sl = shard_slices(tuple(variable._shape), layout)
    if sl is None:
        return None
    from keras_b200.core.tensor import convert_to_tensor

    full = convert_to_tensor(initializer(variable._shape, dtype=variable._dtype), dtype=variable._torch_dtype)
    variable._global_shape = tuple(variable._shape)
    variable._shard_slices = sl
    return full[sl].clone()


class _GatherShards(torch.autograd.Function):
    """Forward: all-gather along each sharded dim.  Backward: this rank's slice (model-axis peers see the same
    upstream gradient because they run the same replica of the batch)."""

    @staticmethod
    def forward(ctx, local, info, slices):
        ctx.slices = slices
        out = local
        for dim, parts, index, group in info:
            pieces = [torch.empty_like(out) for _ in range(parts)]
            dist.all_gather(pieces, out.contiguous(), group=group)
            out = torch.cat(pieces, dim=dim)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad[ctx.slices].contiguous(), None, None


def gather_variable(variable, local=None):
    """Full logical value of a sharded variable (autograd-aware)."""
    layout = variable._layout
    info = _axis_info(layout, layout.device_mesh.backend_mesh)
    local = variable._value if local is None else local
    if not info:
        return local
    return _GatherShards.apply(local, info, variable._shard_slices)


@contextlib.contextmanager
def local_shards():
    """Inside this scope ``Variable.value`` of a sharded variable is its local shard (optimizer updates)."""
    prev = global_state.get_global_attribute("tp_local_shards", False)
    global_state.set_global_attribute("tp_local_shards", True)
    try:
        yield
    finally:
        global_state.set_global_attribute("tp_local_shards", prev)


def in_local_shards():
    return bool(global_state.get_global_attribute("tp_local_shards", False))


def plan_for_model(distribution, model):
    """{variable path: layout axes} of every sharded variable of ``model`` (diagnostics and checkpoints)."""
    plan = {}
    for v in model.variables:
        layout = getattr(v, "_layout", None)
        if layout is not None and any(a is not None for a in layout.axes):
            plan[v.path] = tuple(layout.axes)
    return plan
