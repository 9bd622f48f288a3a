"""Merging layers (keras/src/layers/merging/*.py): Add, Subtract, Multiply, Average, Maximum,
Minimum, Concatenate, Dot and their functional forms."""

import torch

from keras_b200 import ops
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.layer import Layer


class Merge(Layer):
    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.supports_masking = True

    def _merge_function(self, inputs):
        raise NotImplementedError

    def _apply_merge_op_and_or_mask(self, op_fn, inputs):
        out = None
        for x in inputs:
            out = x if out is None else op_fn(out, x)
        return out

    def _compute_elemwise_op_output_shape(self, shape1, shape2):
        if None in (shape1, shape2):
            return None
        if len(shape1) < len(shape2):
            return self._compute_elemwise_op_output_shape(shape2, shape1)
        if not shape2:
            return shape1
        out = list(shape1[: -len(shape2)])
        for i, j in zip(shape1[-len(shape2):], shape2):
            if i is None or j is None:
                out.append(None)
            elif i == 1:
                out.append(j)
            elif j == 1:
                out.append(i)
            else:
                if i != j:
                    raise ValueError(f"Inputs have incompatible shapes. Received shapes {shape1} and {shape2}")
                out.append(i)
        return tuple(out)

    def build(self, input_shape):
        if not isinstance(input_shape[0], (tuple, list)):
            raise ValueError(f"A merge layer should be called on a list of inputs. Received: input_shape={input_shape} (not a list of shapes)")
        if len(input_shape) < 1:
            raise ValueError(f"A merge layer should be called on a list of at least 1 input. Received {len(input_shape)} inputs. Full input_shape received: {input_shape}")
        batch_sizes = {s[0] for s in input_shape if s} - {None}
        if len(batch_sizes) > 1:
            raise ValueError(f"Cannot merge tensors with different batch sizes. Received tensors with shapes {input_shape}")
        out = None if input_shape[0] is None else input_shape[0][1:]
        for s in input_shape[1:]:
            out = self._compute_elemwise_op_output_shape(out, None if s is None else s[1:])
        self._reshape_required = None in {None if s is None else len(s) for s in input_shape} or len({len(s) for s in input_shape if s is not None}) != 1
        self.built = True

    def call(self, inputs):
        if not isinstance(inputs, (list, tuple)):
            raise ValueError(f"A merge layer should be called on a list of inputs. Received: inputs={inputs} (not a list of tensors)")
        if self._reshape_required:
            max_ndim = max(len(x.shape) for x in inputs)
            inputs = [ops.reshape(x, (x.shape[0],) + (1,) * (max_ndim - len(x.shape)) + tuple(x.shape[1:])) if len(x.shape) < max_ndim else x for x in inputs]
        return self._merge_function(inputs)

    def compute_output_shape(self, input_shape):
        out = input_shape[0][1:] if input_shape[0] is not None else None
        for s in input_shape[1:]:
            out = self._compute_elemwise_op_output_shape(out, None if s is None else s[1:])
        batch = {s[0] for s in input_shape if s is not None} - {None}
        return ((list(batch)[0] if len(batch) == 1 else None),) + tuple(out)

    def compute_output_spec(self, inputs):
        shape = self.compute_output_shape([x.shape for x in inputs])
        sparse = all(x.sparse for x in inputs)
        from keras_b200.core.dtypes import result_type

        return KerasTensor(shape, dtype=result_type(*[x.dtype for x in inputs]) if len({x.dtype for x in inputs}) > 1 else inputs[0].dtype, sparse=sparse)

    def compute_mask(self, inputs, mask=None):
        if mask is None:
            return None
        if not isinstance(mask, (tuple, list)):
            raise ValueError(f"`mask` should be a list. Received: mask={mask}")
        if not isinstance(inputs, (tuple, list)):
            raise ValueError(f"`inputs` should be a list. Received: inputs={inputs}")
        if len(mask) != len(inputs):
            raise ValueError(f"The lists `inputs` and `mask` should have the same length. Received: inputs={inputs} of length {len(inputs)}, and mask={mask} of length {len(mask)}")
        if any(m is None for m in mask):
            return None
        out = mask[0]
        for m in mask[1:]:
            out = ops.logical_or(out, m)
        return out


def _make_merge(name, fn, post=None):
    def _merge_function(self, inputs):
        out = inputs[0]
        for x in inputs[1:]:
            out = fn(out, x)
        return post(out, len(inputs)) if post else out

    cls = type(name, (Merge,), {"_merge_function": _merge_function})
    cls.__module__ = __name__
    keras_export(f"keras.layers.{name}")(cls)

    def functional(inputs, **kwargs):
        return cls(**kwargs)(inputs)

    functional.__name__ = name.lower()
    keras_export(f"keras.layers.{name.lower()}")(functional)
    return cls, functional


Add, add = _make_merge("Add", ops.add)
Multiply, multiply = _make_merge("Multiply", ops.multiply)
Maximum, maximum = _make_merge("Maximum", ops.maximum)
Minimum, minimum = _make_merge("Minimum", ops.minimum)
Average, average = _make_merge("Average", ops.add, post=lambda out, n: out / n)


@keras_export("keras.layers.Subtract")
class Subtract(Merge):
    def build(self, input_shape):
        super().build(input_shape)
        if len(input_shape) != 2:
            raise ValueError(f"A `Subtract` layer should be called on exactly 2 inputs. Received: input_shape={input_shape}")

    def _merge_function(self, inputs):
        if len(inputs) != 2:
            raise ValueError(f"A `Subtract` layer should be called on exactly 2 inputs. Received: inputs={inputs}")
        return ops.subtract(inputs[0], inputs[1])


@keras_export("keras.layers.subtract")
def subtract(inputs, **kwargs):
    return Subtract(**kwargs)(inputs)


@keras_export("keras.layers.Concatenate")
class Concatenate(Merge):
    def __init__(self, axis=-1, **kwargs):
        super().__init__(**kwargs)
        self.axis = axis
        self.supports_masking = True
        self._reshape_required = False

    def build(self, input_shape):
        if len(input_shape) < 1 or not isinstance(input_shape[0], (tuple, list)):
            raise ValueError(f"A `Concatenate` layer should be called on a list of at least 1 input. Received: input_shape={input_shape}")
        if all(s is None for s in input_shape):
            return
        reduced = [list(s) for s in input_shape]
        ranks = {len(s) for s in reduced}
        if len(ranks) != 1:
            raise ValueError(f"A `Concatenate` layer requires inputs with matching shapes except for the concatenation axis. Received: input_shape={input_shape}")
        for s in reduced:
            del s[self.axis]
        for axis in range(len(reduced[0])):
            dims = {s[axis] for s in reduced} - {None, 1} if False else {s[axis] for s in reduced} - {None}
            if len(dims) > 1:
                raise ValueError(f"A `Concatenate` layer requires inputs with matching shapes except for the concatenation axis. Received: input_shape={input_shape}")
        self.built = True

    def _merge_function(self, inputs):
        return ops.concatenate(inputs, axis=self.axis)

    def compute_output_shape(self, input_shape):
        if not isinstance(input_shape, (tuple, list)) or not isinstance(input_shape[0], (tuple, list)):
            raise ValueError(f"A `Concatenate` layer should be called on a list of inputs. Received: input_shape={input_shape}")
        out = list(input_shape[0])
        for s in input_shape[1:]:
            if out[self.axis] is None or s[self.axis] is None:
                out[self.axis] = None
                break
            out[self.axis] += s[self.axis]
        return tuple(out)

    def compute_mask(self, inputs, mask=None):
        if mask is None:
            return None
        if not isinstance(mask, (tuple, list)):
            raise ValueError(f"`mask` should be a list. Received mask={mask}")
        if not isinstance(inputs, (tuple, list)):
            raise ValueError(f"`inputs` should be a list. Received: inputs={inputs}")
        if len(mask) != len(inputs):
            raise ValueError(f"The lists `inputs` and `mask` should have the same length. Received: inputs={inputs} of length {len(inputs)}, and mask={mask} of length {len(mask)}")
        if all(m is None for m in mask):
            return None
        masks = []
        for x, m in zip(inputs, mask):
            if m is None:
                masks.append(ops.ones(tuple(x.shape[:-1]) + (1,) if self.axis in (-1, len(x.shape) - 1) else tuple(x.shape), dtype="bool") if False else ops.ones_like(x, dtype="bool"))
            elif len(m.shape) < len(x.shape):
                masks.append(ops.broadcast_to(ops.expand_dims(m, -1), tuple(x.shape)))
            else:
                masks.append(m)
        cat = ops.concatenate(masks, axis=self.axis)
        return ops.any(cat, axis=-1, keepdims=False)

    def get_config(self):
        return {**super().get_config(), "axis": self.axis}


@keras_export("keras.layers.concatenate")
def concatenate(inputs, axis=-1, **kwargs):
    return Concatenate(axis=axis, **kwargs)(inputs)


def batch_dot(x, y, axes=None):
    x_shape, y_shape = tuple(x.shape), tuple(y.shape)
    x_ndim, y_ndim = len(x_shape), len(y_shape)
    if x_ndim < 2 or y_ndim < 2:
        raise ValueError(f"Cannot do batch_dot on inputs with rank < 2. Received inputs with shapes {x_shape} and {y_shape}.")
    if x_shape[0] is not None and y_shape[0] is not None and x_shape[0] != y_shape[0]:
        raise ValueError(f"Cannot do batch_dot on inputs with different batch sizes. Received inputs with shapes {x_shape} and {y_shape}.")
    if isinstance(axes, int):
        axes = [axes, axes]
    if axes is None:
        axes = [x_ndim - 1, y_ndim - 1] if y_ndim == 2 else [x_ndim - 1, y_ndim - 2]
    axes = list(axes)
    a0 = axes[0] if axes[0] >= 0 else axes[0] + x_ndim
    a1 = axes[1] if axes[1] >= 0 else axes[1] + y_ndim
    if 0 in (a0, a1):
        raise ValueError(f"Cannot perform batch_dot over axis 0. If your inputs are not batched, add a dummy batch dimension to your inputs using keras.ops.expand_dims(x, 0)")
    d1, d2 = x_shape[a0], y_shape[a1]
    if d1 is not None and d2 is not None and d1 != d2:
        raise ValueError(f"Cannot do batch_dot on inputs with shapes {x_shape} and {y_shape} with axes={axes}. x.shape[{axes[0]}] != y.shape[{axes[1]}] ({d1} != {d2}).")
    letters = "abcdefghijklmnopqrstuvwxyz"
    xs = ["z"] + [letters[i] for i in range(x_ndim - 1)]
    ys = ["z"] + [letters[x_ndim - 1 + i] for i in range(y_ndim - 1)]
    ys[a1] = xs[a0]
    out = [c for i, c in enumerate(xs) if i != a0] + [c for i, c in enumerate(ys) if i != a1 and i != 0]
    result = ops.einsum(f"{''.join(xs)},{''.join(ys)}->{''.join(out)}", x, y)
    if len(out) == 1:
        result = ops.expand_dims(result, 1)
    return result


@keras_export("keras.layers.Dot")
class Dot(Merge):
    def __init__(self, axes, normalize=False, **kwargs):
        super().__init__(**kwargs)
        if not isinstance(axes, int):
            if not isinstance(axes, (list, tuple)):
                raise TypeError(f"Invalid type for argument `axes`: it should be a list or an int. Received: axes={axes}")
            if len(axes) != 2:
                raise ValueError(f"Invalid format for argument `axes`: it should contain two elements. Received: axes={axes}")
            if not isinstance(axes[0], int) or not isinstance(axes[1], int):
                raise ValueError(f"Invalid format for argument `axes`: list elements should be integers. Received: axes={axes}")
        self.axes = axes
        self.normalize = normalize
        self.supports_masking = True
        self._reshape_required = False

    def build(self, input_shape):
        if len(input_shape) != 2 or not isinstance(input_shape[0], (tuple, list)):
            raise ValueError(f"A `Dot` layer should be called on a list of 2 inputs. Received: input_shape={input_shape}")
        s1, s2 = input_shape
        if s1 is None or s2 is None:
            return
        axes = [self.axes % len(s1), self.axes % len(s2)] if isinstance(self.axes, int) and self.axes < 0 else ([self.axes] * 2 if isinstance(self.axes, int) else self.axes)
        if s1[axes[0]] != s2[axes[1]] and s1[axes[0]] is not None and s2[axes[1]] is not None:
            raise ValueError(f"Incompatible input shapes: axis values {s1[axes[0]]} (at axis {axes[0]}) != {s2[axes[1]]} (at axis {axes[1]}). Full input shapes: {s1}, {s2}")
        self.built = True

    def _merge_function(self, inputs):
        if len(inputs) != 2:
            raise ValueError(f"A `Dot` layer should be called on exactly 2 inputs. Received: inputs={inputs}")
        x1, x2 = inputs
        if isinstance(self.axes, int):
            axes = [self.axes % len(x1.shape), self.axes % len(x2.shape)] if self.axes < 0 else [self.axes] * 2
        else:
            axes = [self.axes[i] % len(inputs[i].shape) for i in range(2)]
        if self.normalize:
            x1 = ops.normalize(x1, axis=axes[0])
            x2 = ops.normalize(x2, axis=axes[1])
        return batch_dot(x1, x2, axes)

    def compute_output_shape(self, input_shape):
        if not isinstance(input_shape, (tuple, list)) or len(input_shape) != 2:
            raise ValueError(f"A `Dot` layer should be called on a list of 2 inputs. Received: input_shape={input_shape}")
        s1, s2 = list(input_shape[0]), list(input_shape[1])
        if isinstance(self.axes, int):
            axes = [self.axes % len(s1), self.axes % len(s2)] if self.axes < 0 else [self.axes] * 2
        else:
            axes = [self.axes[0] % len(s1), self.axes[1] % len(s2)]
        s1.pop(axes[0])
        s2.pop(axes[1])
        s2.pop(0)
        out = s1 + s2
        if len(out) == 1:
            out += [1]
        return tuple(out)

    def compute_mask(self, inputs, mask=None):
        return None

    def get_config(self):
        return {**super().get_config(), "axes": self.axes, "normalize": self.normalize}


@keras_export("keras.layers.dot")
def dot(inputs, axes=-1, **kwargs):
    return Dot(axes=axes, **kwargs)(inputs)
