"""Static shape arithmetic shared by ops and layers (keras/src/ops/operation_utils.py)."""

import math

import numpy as np

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export


def broadcast_shapes(shape1, shape2):
    shape1, shape2 = list(shape1), list(shape2)
    origin1, origin2 = tuple(shape1), tuple(shape2)
    if len(shape1) > len(shape2):
        shape2 = [1] * (len(shape1) - len(shape2)) + shape2
    if len(shape1) < len(shape2):
        shape1 = [1] * (len(shape2) - len(shape1)) + shape1
    out = list(shape1)
    for i in range(len(shape1)):
        a, b = shape1[i], shape2[i]
        if a == 1:
            out[i] = b
        elif a is None:
            out[i] = None if b == 1 else b
        elif b == 1 or b is None or b == a:
            out[i] = a
        else:
            raise ValueError(f"Cannot broadcast shape, the failure dim has value {a}, which cannot be broadcasted to {b}. Input shapes are: {origin1} and {origin2}.")
    return out


def compute_expand_dims_output_shape(input_shape, axis):
    input_shape = list(input_shape)
    if axis is None:
        axis = len(input_shape)
    axes = (axis,) if isinstance(axis, int) else tuple(axis)
    out_ndim = len(axes) + len(input_shape)
    axes = [a if a >= 0 else a + out_ndim for a in axes]
    it = iter(input_shape)
    return tuple(1 if i in axes else next(it) for i in range(out_ndim))


def compute_pooling_output_shape(input_shape, pool_size, strides, padding="valid", data_format="channels_last"):
    strides = pool_size if strides is None else strides
    shape = np.array(input_shape)
    spatial = shape[1:-1] if data_format == "channels_last" else shape[2:]
    none_dims = [i for i, d in enumerate(spatial) if d is None]
    spatial = np.array([-1 if d is None else d for d in spatial])
    pool_size, strides = np.array(pool_size), np.array(strides)
    if padding == "valid":
        out = np.floor((spatial - pool_size) / strides) + 1
        for i in range(len(out)):
            if i not in none_dims and out[i] < 0:
                raise ValueError(f"Computed output size would be negative. Received: `inputs.shape={input_shape}` and `pool_size={pool_size}`.")
    elif padding == "same":
        out = np.floor((spatial - 1) / strides) + 1
    else:
        raise ValueError(f"Argument `padding` must be either 'valid' or 'same'. Received: padding={padding}")
    out = [None if i in none_dims else int(o) for i, o in enumerate(out)]
    if data_format == "channels_last":
        return (input_shape[0],) + tuple(out) + (input_shape[-1],)
    return (input_shape[0], input_shape[1]) + tuple(out)


def compute_conv_output_shape(input_shape, filters, kernel_size, strides=1, padding="valid", data_format="channels_last", dilation_rate=1):
    if data_format == "channels_last":
        spatial = input_shape[1:-1]
        kernel_shape = tuple(kernel_size) + (input_shape[-1], filters)
    else:
        spatial = input_shape[2:]
        kernel_shape = tuple(kernel_size) + (input_shape[1], filters)
    n = len(spatial)
    if len(kernel_shape) != len(input_shape):
        raise ValueError(f"Kernel shape must have the same length as input, but received kernel of shape {kernel_shape} and input of shape {input_shape}.")
    if isinstance(dilation_rate, int):
        dilation_rate = (dilation_rate,) * n
    if isinstance(strides, int):
        strides = (strides,) * n
    if len(dilation_rate) != n:
        raise ValueError(f"Dilation must be None, scalar or tuple/list of length of inputs' spatial shape, but received `dilation_rate={dilation_rate}` and input of shape {input_shape}.")
    out = []
    for i, d in enumerate(spatial):
        if d is None:
            out.append(None)
            continue
        eff = (kernel_size[i] - 1) * dilation_rate[i] + 1
        if padding == "valid":
            o = (d - eff) // strides[i] + 1
            if o < 0:
                raise ValueError(f"Computed output size would be negative. Received `inputs shape={input_shape}`, `kernel shape={kernel_shape}`, `dilation_rate={dilation_rate}`.")
        elif padding in ("same", "causal"):
            o = (d - 1) // strides[i] + 1
        else:
            raise ValueError(f"`padding` must be either `'valid'` or `'same'`. Received {padding}.")
        out.append(o)
    if data_format == "channels_last":
        return (input_shape[0],) + tuple(out) + (filters,)
    return (input_shape[0], filters) + tuple(out)


def compute_matmul_output_shape(shape1, shape2):
    shape1, shape2 = list(shape1), list(shape2)
    if len(shape1) == 1:
        shape1 = [1] + shape1
    squeeze2 = False
    if len(shape2) == 1:
        shape2 = shape2 + [1]
        squeeze2 = True
    if shape1[-1] is not None and shape2[-2] is not None and shape1[-1] != shape2[-2]:
        raise ValueError(f"Inner dimensions (`x1.shape[-1]` and `x2.shape[-2]`) must be equal, but received `x1.shape={tuple(shape1)}` and `x2.shape={tuple(shape2)}`.")
    lead = broadcast_shapes(shape1[:-2], shape2[:-2])
    out = list(lead) + [shape1[-2], shape2[-1]]
    if len(shape1) == 2 and shape1[0] == 1 and False:
        out = out[1:]
    if squeeze2:
        out = out[:-1]
    return tuple(out)


def compute_reshape_output_shape(input_shape, newshape, newshape_arg_name):
    unknown = newshape.count(-1)
    if unknown > 1:
        raise ValueError(f"There must be at most one unknown dimension (-1) in {newshape_arg_name}. Received: {newshape_arg_name}={newshape}.")
    if None in input_shape:
        return tuple(d if d != -1 else None for d in newshape)
    size = math.prod(input_shape)
    if unknown == 0:
        if size != math.prod(newshape):
            raise ValueError(f"The total size of the tensor must be unchanged. Received: input_shape={input_shape}, {newshape_arg_name}={newshape}")
        return tuple(newshape)
    known = 1
    idx = None
    for i, d in enumerate(newshape):
        if d == -1:
            idx = i
        else:
            known *= d
    if known == 0 or size % known != 0:
        raise ValueError(f"The total size of the tensor must be unchanged, however, the input size {size} cannot by divided by the specified dimensions in {newshape_arg_name}. Received: input_shape={input_shape}, {newshape_arg_name}={newshape}")
    out = list(newshape)
    out[idx] = size // known
    return tuple(out)


def compute_transpose_output_shape(input_shape, axes):
    input_shape = list(input_shape)
    if axes is None:
        return tuple(input_shape[::-1])
    if len(axes) != len(input_shape):
        raise ValueError(f"axis must be a list of the same length as the input shape, expected {len(input_shape)}, but received {len(axes)}.")
    return tuple(input_shape[a] for a in axes)


def compute_take_along_axis_output_shape(input_shape, indices_shape, axis):
    input_shape, indices_shape = list(input_shape), list(indices_shape)
    if axis is None:
        input_shape = [None] if None in input_shape else [int(np.prod(input_shape))]
    if len(input_shape) != len(indices_shape):
        raise ValueError(f"`x` and `indices` must have the same number of dimensions, but receive shape {input_shape} and {indices_shape}.")
    input_shape[axis if axis is not None else 0] = indices_shape[axis if axis is not None else 0]
    return tuple(broadcast_shapes(input_shape, indices_shape))


def reduce_shape(shape, axis=None, keepdims=False):
    shape = list(shape)
    if axis is None:
        return tuple(1 for _ in shape) if keepdims else ()
    if isinstance(axis, int):
        axis = (axis,)
    axis = tuple(a if a >= 0 else a + len(shape) for a in axis)
    if keepdims:
        for a in axis:
            shape[a] = 1
        return tuple(shape)
    return tuple(d for i, d in enumerate(shape) if i not in axis)


@keras_export("keras.utils.get_source_inputs")
def get_source_inputs(tensor):
    """Input tensors (produced by ``Input``) that ``tensor`` depends on."""
    if not hasattr(tensor, "_keras_history"):
        return tensor
    operation, node_index, _ = tensor._keras_history
    if not operation or not operation._inbound_nodes:
        return [tensor]
    node = operation._inbound_nodes[node_index]
    if node.is_input:
        return tree.flatten(node.output_tensors)
    out = []
    for t in node.input_tensors:
        for x in get_source_inputs(t):
            if all(x is not y for y in out):
                out.append(x)
    return out
