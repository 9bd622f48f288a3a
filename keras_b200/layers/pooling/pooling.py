"""Pooling layers (keras/src/layers/pooling/*.py): max/average 1-3D, global, adaptive."""

import torch

from keras_b200 import ops
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.convolutional.base_conv import standardize_tuple
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer


class BasePooling(Layer):
    def __init__(self, pool_size, strides, pool_dimensions, pool_mode="max", padding="valid", data_format=None, name=None, **kwargs):
        super().__init__(name=name, **kwargs)
        self.pool_size = standardize_tuple(pool_size, pool_dimensions, "pool_size")
        strides = pool_size if strides is None else strides
        self.strides = standardize_tuple(strides, pool_dimensions, "strides", allow_zero=True)
        self.pool_mode = pool_mode
        self.padding = padding
        self.data_format = config.standardize_data_format(data_format)
        self.input_spec = InputSpec(ndim=pool_dimensions + 2)
        self._dims = pool_dimensions
        self.built = True

    def call(self, inputs):
        if self.pool_mode == "max":
            return ops.max_pool(inputs, pool_size=self.pool_size, strides=self.strides, padding=self.padding, data_format=self.data_format)
        if self.pool_mode == "average":
            return ops.average_pool(inputs, pool_size=self.pool_size, strides=self.strides, padding=self.padding, data_format=self.data_format)
        raise ValueError(f"`pool_mode` must be either 'max' or 'average'. Received: {self.pool_mode}.")

    def compute_output_shape(self, input_shape):
        spatial = input_shape[1:-1] if self.data_format == "channels_last" else input_shape[2:]
        out = []
        for i, d in enumerate(spatial):
            if d is None:
                out.append(None)
            elif self.padding == "valid":
                out.append((d - self.pool_size[i]) // self.strides[i] + 1)
            else:
                out.append((d - 1) // self.strides[i] + 1)
        if self.data_format == "channels_last":
            return (input_shape[0],) + tuple(out) + (input_shape[-1],)
        return (input_shape[0], input_shape[1]) + tuple(out)

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"pool_size": self.pool_size, "padding": self.padding, "strides": self.strides, "data_format": self.data_format})
        return cfg


def _make_pool(name, dims, mode, exports, default_size):
    def __init__(self, pool_size=default_size, strides=None, padding="valid", data_format=None, name=None, **kwargs):
        BasePooling.__init__(self, pool_size, strides, pool_dimensions=dims, pool_mode=mode, padding=padding, data_format=data_format, name=name, **kwargs)

    cls = type(name, (BasePooling,), {"__init__": __init__})
    cls.__module__ = __name__
    return keras_export(exports)(cls)


MaxPooling1D = _make_pool("MaxPooling1D", 1, "max", ["keras.layers.MaxPooling1D", "keras.layers.MaxPool1D"], 2)
MaxPooling2D = _make_pool("MaxPooling2D", 2, "max", ["keras.layers.MaxPooling2D", "keras.layers.MaxPool2D"], (2, 2))
MaxPooling3D = _make_pool("MaxPooling3D", 3, "max", ["keras.layers.MaxPooling3D", "keras.layers.MaxPool3D"], (2, 2, 2))
AveragePooling1D = _make_pool("AveragePooling1D", 1, "average", ["keras.layers.AveragePooling1D", "keras.layers.AvgPool1D"], 2)
AveragePooling2D = _make_pool("AveragePooling2D", 2, "average", ["keras.layers.AveragePooling2D", "keras.layers.AvgPool2D"], (2, 2))
AveragePooling3D = _make_pool("AveragePooling3D", 3, "average", ["keras.layers.AveragePooling3D", "keras.layers.AvgPool3D"], (2, 2, 2))


class BaseGlobalPooling(Layer):
    def __init__(self, pool_dimensions, data_format=None, keepdims=False, **kwargs):
        super().__init__(**kwargs)
        self.data_format = config.standardize_data_format(data_format)
        self.keepdims = keepdims
        self.input_spec = InputSpec(ndim=pool_dimensions + 2)
        self._dims = pool_dimensions
        self.built = True

    def _axes(self):
        n = self._dims
        return list(range(1, n + 1)) if self.data_format == "channels_last" else list(range(2, n + 2))

    def compute_output_shape(self, input_shape):
        n = self._dims
        if self.data_format == "channels_last":
            if self.keepdims:
                return (input_shape[0],) + (1,) * n + (input_shape[-1],)
            return (input_shape[0], input_shape[-1])
        if self.keepdims:
            return (input_shape[0], input_shape[1]) + (1,) * n
        return (input_shape[0], input_shape[1])

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"data_format": self.data_format, "keepdims": self.keepdims})
        return cfg


def _make_global(name, dims, mode, exports):
    def __init__(self, data_format=None, keepdims=False, **kwargs):
        BaseGlobalPooling.__init__(self, pool_dimensions=dims, data_format=data_format, keepdims=keepdims, **kwargs)
        if mode == "avg" and dims == 1:
            self.supports_masking = True

    if mode == "max":
        def call(self, inputs):
            return ops.max(inputs, axis=self._axes(), keepdims=self.keepdims)
        ns = {"__init__": __init__, "call": call}
    elif dims == 1:
        def call(self, inputs, mask=None):
            steps_axis = 1 if self.data_format == "channels_last" else 2
            if mask is not None:
                mask = ops.cast(mask, inputs.dtype)
                mask = ops.expand_dims(mask, 2 if self.data_format == "channels_last" else 1)
                inputs = inputs * mask
                return ops.sum(inputs, axis=steps_axis, keepdims=self.keepdims) / ops.sum(mask, axis=steps_axis, keepdims=self.keepdims)
            return ops.mean(inputs, axis=steps_axis, keepdims=self.keepdims)

        def compute_mask(self, inputs, mask=None):
            return None
        ns = {"__init__": __init__, "call": call, "compute_mask": compute_mask}
    else:
        def call(self, inputs):
            if self.data_format == "channels_last" and isinstance(inputs, torch.Tensor) and inputs.is_cuda:
                from keras_b200.kernels import dispatch

                out = dispatch.global_avg_pool(inputs)
                if out is not None:
                    return out.reshape((inputs.shape[0],) + (1,) * dims + (inputs.shape[-1],)) if self.keepdims else out
            return ops.mean(inputs, axis=self._axes(), keepdims=self.keepdims)
        ns = {"__init__": __init__, "call": call}
    cls = type(name, (BaseGlobalPooling,), ns)
    cls.__module__ = __name__
    return keras_export(exports)(cls)


GlobalMaxPooling1D = _make_global("GlobalMaxPooling1D", 1, "max", ["keras.layers.GlobalMaxPooling1D", "keras.layers.GlobalMaxPool1D"])
GlobalMaxPooling2D = _make_global("GlobalMaxPooling2D", 2, "max", ["keras.layers.GlobalMaxPooling2D", "keras.layers.GlobalMaxPool2D"])
GlobalMaxPooling3D = _make_global("GlobalMaxPooling3D", 3, "max", ["keras.layers.GlobalMaxPooling3D", "keras.layers.GlobalMaxPool3D"])
GlobalAveragePooling1D = _make_global("GlobalAveragePooling1D", 1, "avg", ["keras.layers.GlobalAveragePooling1D", "keras.layers.GlobalAvgPool1D"])
GlobalAveragePooling2D = _make_global("GlobalAveragePooling2D", 2, "avg", ["keras.layers.GlobalAveragePooling2D", "keras.layers.GlobalAvgPool2D"])
GlobalAveragePooling3D = _make_global("GlobalAveragePooling3D", 3, "avg", ["keras.layers.GlobalAveragePooling3D", "keras.layers.GlobalAvgPool3D"])


class BaseAdaptivePooling(Layer):
    def __init__(self, output_size, dims, mode, data_format=None, **kwargs):
        super().__init__(**kwargs)
        if isinstance(output_size, int):
            output_size = (output_size,) * dims
        self.output_size = tuple(output_size)
        if len(self.output_size) != dims:
            raise ValueError(f"`output_size` must be an int or a tuple of {dims} ints. Received: {output_size}")
        self.data_format = config.standardize_data_format(data_format)
        self._dims, self._mode = dims, mode
        self.built = True

    def call(self, inputs):
        fn = ops.adaptive_max_pool if self._mode == "max" else ops.adaptive_average_pool
        return fn(inputs, self.output_size, data_format=self.data_format)

    def compute_output_shape(self, input_shape):
        if self.data_format == "channels_last":
            return (input_shape[0],) + self.output_size + (input_shape[-1],)
        return (input_shape[0], input_shape[1]) + self.output_size

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"output_size": self.output_size, "data_format": self.data_format})
        return cfg


def _make_adaptive(name, dims, mode):
    def __init__(self, output_size, data_format=None, **kwargs):
        BaseAdaptivePooling.__init__(self, output_size, dims, mode, data_format=data_format, **kwargs)

    cls = type(name, (BaseAdaptivePooling,), {"__init__": __init__})
    cls.__module__ = __name__
    return keras_export(f"keras.layers.{name}")(cls)


AdaptiveMaxPooling1D = _make_adaptive("AdaptiveMaxPooling1D", 1, "max")
AdaptiveMaxPooling2D = _make_adaptive("AdaptiveMaxPooling2D", 2, "max")
AdaptiveMaxPooling3D = _make_adaptive("AdaptiveMaxPooling3D", 3, "max")
AdaptiveAveragePooling1D = _make_adaptive("AdaptiveAveragePooling1D", 1, "avg")
AdaptiveAveragePooling2D = _make_adaptive("AdaptiveAveragePooling2D", 2, "avg")
AdaptiveAveragePooling3D = _make_adaptive("AdaptiveAveragePooling3D", 3, "avg")
