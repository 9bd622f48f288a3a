"""Reshaping layers (keras/src/layers/reshaping/*.py)."""

import math

import torch

from keras_b200 import ops
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer


@keras_export("keras.layers.Flatten")
class Flatten(Layer):
    def __init__(self, data_format=None, **kwargs):
        super().__init__(**kwargs)
        self.data_format = config.standardize_data_format(data_format)
        self.input_spec = InputSpec(min_ndim=1)
        self._channels_first = self.data_format == "channels_first"
        self.built = True

    def call(self, inputs):
        rank = len(inputs.shape)
        if self._channels_first and rank > 1:
            inputs = ops.transpose(inputs, axes=(0, *range(2, rank), 1))
        if isinstance(inputs, KerasTensor):
            return KerasTensor(self.compute_output_shape(inputs.shape), inputs.dtype)
        return inputs.reshape(inputs.shape[0], -1) if rank > 1 else inputs.reshape(-1, 1)

    def compute_output_shape(self, input_shape):
        non_batch = input_shape[1:]
        if len(non_batch) == 0:
            flat = 1
        elif any(d is None for d in non_batch):
            flat = None
        else:
            flat = math.prod(non_batch)
        return (input_shape[0], flat)

    def compute_output_spec(self, inputs):
        return KerasTensor(self.compute_output_shape(inputs.shape), dtype=inputs.dtype, sparse=inputs.sparse)

    def get_config(self):
        return {**super().get_config(), "data_format": self.data_format}


@keras_export("keras.layers.Reshape")
class Reshape(Layer):
    def __init__(self, target_shape, **kwargs):
        super().__init__(**kwargs)
        target_shape = tuple(target_shape)
        if sum(1 for d in target_shape if d is None or d == -1) > 1:
            raise ValueError(f"There must be at most one unknown dimension (-1 or None) in `target_shape`. Received: target_shape={target_shape}.")
        self.target_shape = tuple(-1 if d is None else d for d in target_shape)
        self.built = True

    def _resolve(self, input_shape):
        known_in = input_shape[1:]
        tgt = list(self.target_shape)
        if -1 in tgt:
            if any(d is None for d in known_in):
                return tuple(None if d == -1 else d for d in tgt)
            total = math.prod(known_in)
            rest = math.prod(d for d in tgt if d != -1)
            if rest == 0 or total % rest != 0:
                raise ValueError(f"The total size of the tensor must be unchanged. Received: input_shape={input_shape}, target_shape={self.target_shape}")
            tgt[tgt.index(-1)] = total // rest
        elif not any(d is None for d in known_in) and math.prod(known_in) != math.prod(tgt):
            raise ValueError(f"The total size of the tensor must be unchanged. Received: input_shape={input_shape}, target_shape={self.target_shape}")
        return tuple(tgt)

    def compute_output_shape(self, input_shape):
        return (input_shape[0],) + self._resolve(input_shape)

    def compute_output_spec(self, inputs):
        return KerasTensor(self.compute_output_shape(inputs.shape), dtype=inputs.dtype, sparse=inputs.sparse)

    def call(self, inputs):
        tgt = self._resolve(tuple(inputs.shape))
        return ops.reshape(inputs, (inputs.shape[0],) + tuple(-1 if d is None else d for d in tgt))

    def get_config(self):
        return {**super().get_config(), "target_shape": self.target_shape}


@keras_export("keras.layers.Permute")
class Permute(Layer):
    def __init__(self, dims, **kwargs):
        super().__init__(**kwargs)
        self.dims = tuple(dims)
        if sorted(dims) != list(range(1, len(dims) + 1)):
            raise ValueError(f"Invalid permutation argument `dims` for Permute Layer. The set of indices in `dims` must be consecutive and start from 1. Received dims={dims}")
        self.input_spec = InputSpec(ndim=len(self.dims) + 1)
        self.built = True

    def compute_output_shape(self, input_shape):
        return (input_shape[0],) + tuple(input_shape[d] for d in self.dims)

    def compute_output_spec(self, inputs):
        return KerasTensor(self.compute_output_shape(inputs.shape), dtype=inputs.dtype, sparse=inputs.sparse)

    def call(self, inputs):
        return ops.transpose(inputs, axes=(0,) + self.dims)

    def get_config(self):
        return {**super().get_config(), "dims": self.dims}


@keras_export("keras.layers.RepeatVector")
class RepeatVector(Layer):
    def __init__(self, n, **kwargs):
        super().__init__(**kwargs)
        if not isinstance(n, int):
            raise TypeError(f"Expected an integer value for `n`, got {type(n)}.")
        self.n = n
        self.input_spec = InputSpec(ndim=2)
        self.built = True

    def compute_output_shape(self, input_shape):
        return (input_shape[0], self.n, input_shape[1])

    def call(self, inputs):
        return ops.repeat(ops.expand_dims(inputs, 1), self.n, axis=1)

    def get_config(self):
        return {**super().get_config(), "n": self.n}


def _norm_pairs(value, n, name):
    if isinstance(value, int):
        return tuple((value, value) for _ in range(n))
    if hasattr(value, "__len__"):
        if len(value) != n:
            raise ValueError(f"`{name}` should have {n} elements. Received: {name}={value}.")
        out = []
        for v in value:
            if isinstance(v, int):
                out.append((v, v))
            else:
                v = tuple(v)
                if len(v) != 2:
                    raise ValueError(f"`{name}` should be either an int, a tuple of {n} ints, or a tuple of {n} tuples of 2 ints. Received: {name}={value}.")
                out.append((int(v[0]), int(v[1])))
        return tuple(out)
    raise ValueError(f"`{name}` should be either an int, a tuple of {n} ints, or a tuple of {n} tuples of 2 ints. Received: {name}={value}.")


def _make_zero_padding(name, n):
    def __init__(self, padding=1 if n == 1 else (1,) * n, data_format=None, **kwargs):
        Layer.__init__(self, **kwargs)
        self.data_format = config.standardize_data_format(data_format)
        if n == 1:
            if isinstance(padding, int):
                padding = (padding, padding)
            p = tuple(padding)
            if len(p) != 2:
                raise ValueError(f"`padding` should be an int or a tuple of 2 ints. Received: padding={padding}")
            self.padding = (int(p[0]), int(p[1]))
            self._pairs = (self.padding,)
        else:
            self.padding = _norm_pairs(padding, n, "padding")
            self._pairs = self.padding
        self.input_spec = InputSpec(ndim=n + 2)
        self.built = True

    def _spatial_axes(self, ndim):
        return list(range(2, ndim)) if self.data_format == "channels_first" else list(range(1, ndim - 1))

    def compute_output_shape(self, input_shape):
        out = list(input_shape)
        for ax, (lo, hi) in zip(self._spatial_axes(len(input_shape)), self._pairs):
            if out[ax] is not None:
                out[ax] += lo + hi
        return tuple(out)

    def call(self, inputs):
        pads = [(0, 0)] * len(inputs.shape)
        for ax, pr in zip(self._spatial_axes(len(inputs.shape)), self._pairs):
            pads[ax] = pr
        return ops.pad(inputs, pads)

    def get_config(self):
        return {**Layer.get_config(self), "padding": self.padding, "data_format": self.data_format}

    cls = type(name, (Layer,), {"__init__": __init__, "_spatial_axes": _spatial_axes, "compute_output_shape": compute_output_shape, "call": call, "get_config": get_config})
    cls.__module__ = __name__
    return keras_export(f"keras.layers.{name}")(cls)


ZeroPadding1D = _make_zero_padding("ZeroPadding1D", 1)
ZeroPadding2D = _make_zero_padding("ZeroPadding2D", 2)
ZeroPadding3D = _make_zero_padding("ZeroPadding3D", 3)


def _make_cropping(name, n):
    def __init__(self, cropping=(1, 1) if n == 1 else ((0, 0),) * n if False else ((1, 1),) * n, data_format=None, **kwargs):
        Layer.__init__(self, **kwargs)
        self.data_format = config.standardize_data_format(data_format)
        if n == 1:
            if isinstance(cropping, int):
                cropping = (cropping, cropping)
            c = tuple(cropping)
            if len(c) != 2:
                raise ValueError(f"`cropping` should be an int or a tuple of 2 ints. Received: cropping={cropping}")
            self.cropping = (int(c[0]), int(c[1]))
            self._pairs = (self.cropping,)
        else:
            self.cropping = _norm_pairs(cropping, n, "cropping")
            self._pairs = self.cropping
        self.input_spec = InputSpec(ndim=n + 2)
        self.built = True

    def _spatial_axes(self, ndim):
        if n == 1:
            return [1]
        return list(range(2, ndim)) if self.data_format == "channels_first" else list(range(1, ndim - 1))

    def compute_output_shape(self, input_shape):
        out = list(input_shape)
        for ax, (lo, hi) in zip(self._spatial_axes(len(input_shape)), self._pairs):
            if out[ax] is not None:
                if lo + hi >= out[ax]:
                    raise ValueError(f"Values in `cropping` argument should be smaller than the corresponding spatial dimension of the input. Received: input_shape={input_shape}, cropping={self.cropping}")
                out[ax] -= lo + hi
        return tuple(out)

    def call(self, inputs):
        idx = [slice(None)] * len(inputs.shape)
        for ax, (lo, hi) in zip(self._spatial_axes(len(inputs.shape)), self._pairs):
            if inputs.shape[ax] is not None and lo + hi >= inputs.shape[ax]:
                raise ValueError(f"Values in `cropping` argument should be smaller than the corresponding spatial dimension of the input. Received: inputs.shape={tuple(inputs.shape)}, cropping={self.cropping}")
            idx[ax] = slice(lo, None if hi == 0 else -hi)
        return inputs[tuple(idx)]

    def get_config(self):
        return {**Layer.get_config(self), "cropping": self.cropping, "data_format": self.data_format}

    ns = {"__init__": __init__, "_spatial_axes": _spatial_axes, "compute_output_shape": compute_output_shape, "call": call, "get_config": get_config}
    cls = type(name, (Layer,), ns)
    cls.__module__ = __name__
    return keras_export(f"keras.layers.{name}")(cls)


Cropping1D = _make_cropping("Cropping1D", 1)
Cropping2D = _make_cropping("Cropping2D", 2)
Cropping3D = _make_cropping("Cropping3D", 3)


@keras_export("keras.layers.UpSampling1D")
class UpSampling1D(Layer):
    def __init__(self, size=2, **kwargs):
        super().__init__(**kwargs)
        self.size = int(size)
        self.input_spec = InputSpec(ndim=3)
        self.built = True

    def compute_output_shape(self, input_shape):
        return (input_shape[0], None if input_shape[1] is None else self.size * input_shape[1], input_shape[2])

    def call(self, inputs):
        return ops.repeat(inputs, self.size, axis=1)

    def get_config(self):
        return {**super().get_config(), "size": self.size}


@keras_export("keras.layers.UpSampling2D")
class UpSampling2D(Layer):
    def __init__(self, size=(2, 2), data_format=None, interpolation="nearest", **kwargs):
        super().__init__(**kwargs)
        self.data_format = config.standardize_data_format(data_format)
        self.size = (size, size) if isinstance(size, int) else tuple(size)
        self.interpolation = interpolation.lower()
        self.input_spec = InputSpec(ndim=4)
        self.built = True

    def compute_output_shape(self, input_shape):
        if self.data_format == "channels_first":
            h = None if input_shape[2] is None else self.size[0] * input_shape[2]
            w = None if input_shape[3] is None else self.size[1] * input_shape[3]
            return (input_shape[0], input_shape[1], h, w)
        h = None if input_shape[1] is None else self.size[0] * input_shape[1]
        w = None if input_shape[2] is None else self.size[1] * input_shape[2]
        return (input_shape[0], h, w, input_shape[3])

    def call(self, inputs):
        if self.interpolation == "nearest":
            ha, wa = (2, 3) if self.data_format == "channels_first" else (1, 2)
            return ops.repeat(ops.repeat(inputs, self.size[0], axis=ha), self.size[1], axis=wa)
        shape = inputs.shape
        if self.data_format == "channels_first":
            new = (shape[2] * self.size[0], shape[3] * self.size[1])
        else:
            new = (shape[1] * self.size[0], shape[2] * self.size[1])
        return ops.image.resize(inputs, new, interpolation=self.interpolation, data_format=self.data_format)

    def get_config(self):
        return {**super().get_config(), "size": self.size, "data_format": self.data_format, "interpolation": self.interpolation}


@keras_export("keras.layers.UpSampling3D")
class UpSampling3D(Layer):
    def __init__(self, size=(2, 2, 2), data_format=None, **kwargs):
        super().__init__(**kwargs)
        self.data_format = config.standardize_data_format(data_format)
        self.size = (size,) * 3 if isinstance(size, int) else tuple(size)
        self.input_spec = InputSpec(ndim=5)
        self.built = True

    def compute_output_shape(self, input_shape):
        axes = (2, 3, 4) if self.data_format == "channels_first" else (1, 2, 3)
        out = list(input_shape)
        for a, s in zip(axes, self.size):
            out[a] = None if out[a] is None else out[a] * s
        return tuple(out)

    def call(self, inputs):
        axes = (2, 3, 4) if self.data_format == "channels_first" else (1, 2, 3)
        x = inputs
        for a, s in zip(axes, self.size):
            x = ops.repeat(x, s, axis=a)
        return x

    def get_config(self):
        return {**super().get_config(), "size": self.size, "data_format": self.data_format}
