"""Core ops: control flow, scatter/slice, casting (``keras.ops`` core set).

Semantics follow keras/src/ops/core.py and keras/src/backend/torch/core.py:395-842.  Control
flow runs as Python loops (eager execution); hot training loops are captured in CUDA graphs by
the trainer instead of by a tracing compiler.
"""

import ml_dtypes
import numpy as np
import torch

from keras_b200 import tree
from keras_b200.core import tensor as _tensor
from keras_b200.core.dtypes import result_type, standardize_dtype, to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.core.tensor import convert_to_numpy as _to_numpy
from keras_b200.core.tensor import convert_to_tensor as _convert
from keras_b200.core.variables import Variable
from keras_b200.ops._dispatch import op
from keras_b200.ops.numpy import _t


@op()
def cast(x, dtype):
    return _tensor.cast(x, dtype)


@op()
def saturate_cast(x, dtype):
    """Cast after clipping to the value range both dtypes share.  A limit that the input dtype cannot represent exactly
    (float32 -> int32: 2147483647) is moved one step towards zero, other limits are used as they are
    (keras/src/ops/core.py:950-990)."""
    x = _t(x)
    td = to_torch_dtype(dtype)
    out_name, in_name = standardize_dtype(dtype), standardize_dtype(x.dtype)

    def limits(name):
        if name == "bool":
            return 0, 1
        if "int" in name:
            info = ml_dtypes.iinfo(name)
            return int(info.min), int(info.max)
        info = ml_dtypes.finfo(name)
        return float(info.min), float(info.max)

    (in_lo, in_hi), (out_lo, out_hi) = limits(in_name), limits(out_name)
    np_in = np.dtype(in_name) if in_name != "bfloat16" else ml_dtypes.bfloat16
    lo = np.maximum(in_lo, out_lo).astype(np_in)
    if lo < out_lo:
        lo = np.nextafter(lo, 0, dtype=np_in)
    hi = np.minimum(in_hi, out_hi).astype(np_in)
    if hi > out_hi:
        hi = np.nextafter(hi, 0, dtype=np_in)
    if x.dtype == torch.bool:
        return x.to(td)
    lo_v = float(lo) if x.dtype.is_floating_point else int(lo)
    hi_v = float(hi) if x.dtype.is_floating_point else int(hi)
    return torch.clip(x, lo_v, hi_v).to(td)


@keras_export("keras.ops.convert_to_tensor")
def convert_to_tensor(x, dtype=None, sparse=None, ragged=None):
    if isinstance(x, KerasTensor):
        return x if dtype is None else KerasTensor(x.shape, dtype=dtype)
    return _convert(x, dtype=dtype)


@keras_export("keras.ops.convert_to_numpy")
def convert_to_numpy(x):
    return _to_numpy(x)


@keras_export("keras.ops.is_tensor")
def is_tensor(x):
    return isinstance(x, torch.Tensor)


@keras_export("keras.ops.shape")
def shape(x):
    if isinstance(x, (KerasTensor, torch.Tensor, Variable, np.ndarray)):
        return tuple(x.shape)
    return tuple(_convert(x).shape)


@keras_export("keras.ops.dtype")
def dtype(x):
    return standardize_dtype(x.dtype)


@op()
def stop_gradient(variable):
    if isinstance(variable, Variable):
        variable = variable.value
    return _t(variable).detach()


@op()
def scatter(indices, values, shape):
    indices = _t(indices).long()
    values = _t(values)
    out = torch.zeros(tuple(shape), dtype=values.dtype, device=values.device)
    k = indices.shape[-1]
    idx = indices.reshape(-1, k)
    vals = values.reshape((-1,) + tuple(shape[k:]))
    return out.index_put_(tuple(idx[:, i] for i in range(k)), vals, accumulate=True)


@op()
def scatter_update(inputs, indices, updates, reduction=None):
    inputs = _t(inputs)
    indices = _t(indices).long()
    updates = _t(updates).to(inputs.dtype)
    k = indices.shape[-1]
    idx = tuple(indices.reshape(-1, k)[:, i] for i in range(k))
    upd = updates.reshape((-1,) + tuple(inputs.shape[k:]))
    out = inputs.clone()
    if reduction is None:
        out[idx] = upd
    elif reduction == "add":
        out.index_put_(idx, upd, accumulate=True)
    elif reduction in ("max", "min", "mul"):
        flat_stride = [int(np.prod(inputs.shape[i + 1:k])) for i in range(k)]
        lin = sum(idx[i] * flat_stride[i] for i in range(k))
        lead = int(np.prod(inputs.shape[:k]))
        o2 = out.reshape((lead, -1))
        u2 = upd.reshape((upd.shape[0], -1))
        red = {"max": "amax", "min": "amin", "mul": "prod"}[reduction]
        o2 = o2.scatter_reduce(0, lin[:, None].expand_as(u2), u2, reduce=red, include_self=True)
        out = o2.reshape(inputs.shape)
    else:
        raise ValueError(f"Invalid reduction: {reduction}")
    return out


@op()
def slice(inputs, start_indices, shape):
    inputs = _t(inputs)
    starts = [int(s) for s in (start_indices.tolist() if isinstance(start_indices, (torch.Tensor, np.ndarray)) else start_indices)]
    sizes = [inputs.shape[i] - starts[i] if s == -1 else int(s) for i, s in enumerate(shape)]
    index = tuple(builtins_slice(st, st + sz) for st, sz in zip(starts, sizes))
    return inputs[index]


builtins_slice = __builtins__["slice"] if isinstance(__builtins__, dict) else __builtins__.slice


@op()
def slice_update(inputs, start_indices, updates):
    inputs = _t(inputs)
    updates = _t(updates).to(inputs.dtype)
    starts = [int(s) for s in (start_indices.tolist() if isinstance(start_indices, (torch.Tensor, np.ndarray)) else start_indices)]
    index = tuple(builtins_slice(st, st + sz) for st, sz in zip(starts, updates.shape))
    out = inputs.clone()
    out[index] = updates
    return out


@op()
def unstack(x, num=None, axis=0):
    return list(torch.unbind(_t(x), dim=axis))


@keras_export("keras.ops.cond")
def cond(pred, true_fn, false_fn):
    if isinstance(pred, KerasTensor):
        from keras_b200.core.tensor import compute_output_spec

        return compute_output_spec(true_fn)
    if isinstance(pred, (torch.Tensor, Variable)):
        pred = bool(_t(pred))
    return true_fn() if pred else false_fn()


@keras_export("keras.ops.switch")
def switch(index, branches, *operands):
    index = int(_t(index)) if not isinstance(index, int) else index
    index = min(max(index, 0), len(branches) - 1)
    return branches[index](*operands)


@keras_export("keras.ops.while_loop")
def while_loop(cond, body, loop_vars, maximum_iterations=None):
    is_seq = isinstance(loop_vars, (list, tuple))
    state = tuple(loop_vars) if is_seq else (loop_vars,)
    state = tree.map_structure(lambda v: _convert(v) if not isinstance(v, (KerasTensor,)) and v is not None else v, state)
    it = 0
    while (maximum_iterations is None or it < maximum_iterations) and bool(cond(*state)):
        out = body(*state)
        state = tuple(out) if isinstance(out, (list, tuple)) else (out,)
        it += 1
    return (list(state) if isinstance(loop_vars, list) else state) if is_seq else state[0]


@keras_export("keras.ops.fori_loop")
def fori_loop(lower, upper, body_fun, init_val):
    val = init_val
    lo = int(_t(lower)) if not isinstance(lower, int) else lower
    hi = int(_t(upper)) if not isinstance(upper, int) else upper
    for i in range(lo, hi):
        val = body_fun(i, val)
    return val


@keras_export("keras.ops.scan")
def scan(f, init, xs=None, length=None, reverse=False, unroll=1):
    if xs is None and length is None:
        raise ValueError("Got no `xs` to scan over and `length` not provided.")
    xs_flat = tree.flatten(xs) if xs is not None else []
    xs_flat = [_convert(x) for x in xs_flat]
    n = int(length) if length is not None else xs_flat[0].shape[0]
    carry = tree.map_structure(lambda v: _convert(v), init)
    ys = []
    order = range(n - 1, -1, -1) if reverse else range(n)
    for i in order:
        x_i = tree.pack_sequence_as(xs, [x[i] for x in xs_flat]) if xs is not None else None
        carry, y = f(carry, x_i)
        ys.append(y)
    if reverse:
        ys.reverse()
    if ys and ys[0] is not None:
        flat_ys = [tree.flatten(y) for y in ys]
        stacked = [torch.stack([_convert(fy[j]) for fy in flat_ys]) for j in range(len(flat_ys[0]))]
        ys_out = tree.pack_sequence_as(ys[0], stacked)
    else:
        ys_out = None
    return carry, ys_out


@keras_export("keras.ops.associative_scan")
def associative_scan(f, elems, reverse=False, axis=0):
    flat = [_convert(e) for e in tree.flatten(elems)]
    n = flat[0].shape[axis]
    if any(e.shape[axis] != n for e in flat):
        raise ValueError("Array inputs to associative_scan must have the same first dimension. (saw: {})".format([tuple(e.shape) for e in flat]))
    if reverse:
        flat = [torch.flip(e, dims=(axis,)) for e in flat]
    slices = [[torch.select(e, axis, i) for e in flat] for i in range(n)]
    outs = []
    acc = None
    for s in slices:
        cur = tree.pack_sequence_as(elems, s)
        # add a leading axis of size one so that `f` sees batched elements as in a tree scan
        cur_b = tree.map_structure(lambda t: t.unsqueeze(axis), cur)
        acc = cur_b if acc is None else f(acc, cur_b)
        outs.append(tree.flatten(acc))
    result = [torch.cat([o[j] for o in outs], dim=axis) for j in range(len(flat))]
    if reverse:
        result = [torch.flip(r, dims=(axis,)) for r in result]
    return tree.pack_sequence_as(elems, result)


@keras_export("keras.ops.map")
def map(f, xs):
    flat = [_convert(x) for x in tree.flatten(xs)]
    n = flat[0].shape[0]
    outs = [f(tree.pack_sequence_as(xs, [x[i] for x in flat])) for i in range(n)]
    flat_outs = [tree.flatten(o) for o in outs]
    stacked = [torch.stack([_convert(fo[j]) for fo in flat_outs]) for j in range(len(flat_outs[0]))]
    return tree.pack_sequence_as(outs[0], stacked)


@keras_export("keras.ops.vectorized_map")
def vectorized_map(function, elements):
    flat = [_convert(x) for x in tree.flatten(elements)]
    packed = tree.pack_sequence_as(elements, flat)
    try:
        return torch.vmap(function)(packed)
    except Exception:
        return map(function, elements)


@keras_export("keras.ops.custom_gradient")
def custom_gradient(f):
    """Decorator: ``f(*args)`` returns ``(output, grad_fn)``; ``grad_fn(*upstream)`` gives input grads."""

    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *args):
            with torch.enable_grad():
                pass
            output, grad_fn = f(*args)
            ctx.grad_fn_user = grad_fn
            ctx.n_in = len(args)
            return output

        @staticmethod
        def backward(ctx, *grad_outputs):
            grads = ctx.grad_fn_user(*grad_outputs)
            if not isinstance(grads, (tuple, list)):
                grads = (grads,)
            grads = tuple(grads) + (None,) * (ctx.n_in - len(grads))
            return grads

    def wrapper(*args, **kwargs):
        if kwargs:
            raise ValueError("custom_gradient functions only accept positional arguments.")
        if any(isinstance(a, KerasTensor) for a in args):
            from keras_b200.core.tensor import compute_output_spec

            return compute_output_spec(lambda *a: f(*a)[0], *args)
        args = [a.value if isinstance(a, Variable) else a for a in args]
        return _Fn.apply(*args)

    return wrapper


def remat(f):
    """Recompute ``f``'s activations in backward instead of storing them."""

    def wrapped(*args, **kwargs):
        import torch.utils.checkpoint as ckpt

        return ckpt.checkpoint(f, *args, use_reentrant=False, **kwargs)

    return wrapped
