"""Convolution layers.

Behaviour of keras/src/layers/convolutional/base_conv.py:16-420: kernel layout ``(*kernel_size,
in/groups, filters)``, channels-last by default, ``ops.conv`` + bias + activation, LoRA on the
kernel.  On a B200, channels-last 2-D convolutions route to the implicit-GEMM tcgen05 kernels.
"""

import math

import torch

from keras_b200 import activations, constraints, initializers, ops, regularizers
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer


def standardize_tuple(value, n, name, allow_zero=False):
    if isinstance(value, int):
        value = (value,) * n
    try:
        value = tuple(int(v) for v in value)
    except (TypeError, ValueError):
        raise ValueError(f"The `{name}` argument must be a tuple of {n} integers. Received {name}={value}")
    if len(value) != n:
        raise ValueError(f"The `{name}` argument must be a tuple of {n} integers. Received {name}={value}")
    bad = [v for v in value if (v < 0 if allow_zero else v <= 0)]
    if bad:
        raise ValueError(f"The `{name}` argument must be a tuple of {n} integers. Received {name}={value}, including values {bad} that do not satisfy `value {'>=' if allow_zero else '>'} 0`")
    return value


def standardize_padding(value, allow_causal=False):
    if isinstance(value, (list, tuple)):
        return value
    p = value.lower()
    allowed = {"valid", "same"} | ({"causal"} if allow_causal else set())
    if p not in allowed:
        raise ValueError(f"The `padding` argument must be a list/tuple or one of {allowed}. Received: {p}")
    return p


def conv_output_shape(input_shape, filters, kernel_size, strides, padding, data_format, dilation_rate):
    if data_format == "channels_last":
        spatial = input_shape[1:-1]
    else:
        spatial = input_shape[2:]
    out = []
    for i, d in enumerate(spatial):
        if d is None:
            out.append(None)
            continue
        eff = (kernel_size[i] - 1) * dilation_rate[i] + 1
        if padding == "valid":
            o = (d - eff) // strides[i] + 1
        else:
            o = (d - 1) // strides[i] + 1
        if o <= 0:
            raise ValueError(
                "Computed output size would be negative. Received `inputs shape="
                f"{input_shape}`, `kernel shape={kernel_size}`, `dilation_rate={dilation_rate}`."
            )
        out.append(o)
    if data_format == "channels_last":
        return (input_shape[0],) + tuple(out) + (filters,)
    return (input_shape[0], filters) + tuple(out)


class BaseConv(Layer):
    def __init__(self, rank, filters, kernel_size, strides=1, padding="valid", data_format=None, dilation_rate=1, groups=1,
                 activation=None, use_bias=True, kernel_initializer="glorot_uniform", bias_initializer="zeros",
                 kernel_regularizer=None, bias_regularizer=None, activity_regularizer=None, kernel_constraint=None,
                 bias_constraint=None, lora_rank=None, lora_alpha=None, **kwargs):
        super().__init__(activity_regularizer=activity_regularizer, **kwargs)
        self.rank = rank
        self.filters = filters
        self.groups = groups
        self.kernel_size = standardize_tuple(kernel_size, rank, "kernel_size")
        self.strides = standardize_tuple(strides, rank, "strides")
        self.dilation_rate = standardize_tuple(dilation_rate, rank, "dilation_rate")
        self.padding = standardize_padding(padding, allow_causal=rank == 1)
        self.data_format = config.standardize_data_format(data_format)
        self.activation = activations.get(activation)
        self.use_bias = use_bias
        self.kernel_initializer = initializers.get(kernel_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.kernel_regularizer = regularizers.get(kernel_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.kernel_constraint = constraints.get(kernel_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.lora_rank = lora_rank
        self.lora_alpha = lora_alpha if lora_alpha is not None else lora_rank
        self.lora_enabled = False
        self.input_spec = InputSpec(min_ndim=self.rank + 2)
        if self.filters is not None and self.filters <= 0:
            raise ValueError(f"Invalid value for argument `filters`. Expected a strictly positive value. Received filters={self.filters}.")
        if self.groups <= 0:
            raise ValueError(f"The number of groups must be a positive integer. Received: groups={self.groups}.")
        if self.filters is not None and self.filters % self.groups != 0:
            raise ValueError(f"The number of filters must be evenly divisible by the number of groups. Received: groups={self.groups}, filters={self.filters}.")
        if max(self.strides) > 1 and max(self.dilation_rate) > 1:
            raise ValueError(f"`strides > 1` not supported in conjunction with `dilation_rate > 1`. Received: strides={self.strides} and dilation_rate={self.dilation_rate}")

    def build(self, input_shape):
        channel_axis = -1 if self.data_format == "channels_last" else 1
        input_channel = input_shape[channel_axis]
        self.input_spec = InputSpec(min_ndim=self.rank + 2, axes={channel_axis: input_channel})
        if input_channel % self.groups != 0:
            raise ValueError(f"The number of input channels must be evenly divisible by the number of groups. Received groups={self.groups}, but the input has {input_channel} channels (full input shape is {input_shape}).")
        kernel_shape = self.kernel_size + (input_channel // self.groups, self.filters)
        self.compute_output_shape(input_shape)
        self._kernel = self.add_weight(name="kernel", shape=kernel_shape, initializer=self.kernel_initializer,
                                       regularizer=self.kernel_regularizer, constraint=self.kernel_constraint, trainable=True, dtype=self.dtype)
        if self.use_bias:
            self.bias = self.add_weight(name="bias", shape=(self.filters,), initializer=self.bias_initializer,
                                        regularizer=self.bias_regularizer, constraint=self.bias_constraint, trainable=True, dtype=self.dtype)
        else:
            self.bias = None
        self.built = True
        if self.lora_rank:
            self.enable_lora(self.lora_rank, lora_alpha=self.lora_alpha)

    @property
    def kernel(self):
        if not self.built:
            raise AttributeError("You must build the layer before accessing `kernel`.")
        if self.lora_enabled:
            return ops.add(self._kernel.value, (self.lora_alpha / self.lora_rank) * ops.matmul(self.lora_kernel_a.value, self.lora_kernel_b.value))
        return self._kernel

    def convolution_op(self, inputs, kernel):
        return ops.conv(inputs, kernel, strides=list(self.strides), padding=self.padding, dilation_rate=self.dilation_rate, data_format=self.data_format)

    def call(self, inputs):
        outputs = self.convolution_op(inputs, self.kernel)
        if self.use_bias:
            if self.data_format == "channels_last":
                outputs = ops.add(outputs, self.bias)
            else:
                outputs = ops.add(outputs, ops.reshape(self.bias, (1, self.filters) + (1,) * self.rank))
        if self.activation is not None:
            return self.activation(outputs)
        return outputs

    def compute_output_shape(self, input_shape):
        return conv_output_shape(input_shape, self.filters, self.kernel_size, self.strides, self.padding, self.data_format, self.dilation_rate)

    def enable_lora(self, rank, lora_alpha=None, a_initializer="he_uniform", b_initializer="zeros"):
        if self.kernel_constraint:
            raise ValueError("Lora is incompatible with kernel constraints. In order to enable lora on this layer, remove the `kernel_constraint` argument.")
        if not self.built:
            raise ValueError("Cannot enable lora on a layer that isn't yet built.")
        if self.lora_enabled:
            raise ValueError("lora is already enabled. This can only be done once per layer.")
        self._tracker_unlock()
        self.lora_kernel_a = self.add_weight(name="lora_kernel_a", shape=self._kernel.shape[:-1] + (rank,), initializer=initializers.get(a_initializer), regularizer=self.kernel_regularizer)
        self.lora_kernel_b = self.add_weight(name="lora_kernel_b", shape=(rank, self.filters), initializer=initializers.get(b_initializer), regularizer=self.kernel_regularizer)
        self._kernel.trainable = False
        self._lock_state()
        self._invalidate()
        self.lora_enabled = True
        self.lora_rank = rank
        self.lora_alpha = lora_alpha if lora_alpha is not None else rank

    def save_own_variables(self, store):
        if not self.built:
            return
        kernel = self._kernel
        if self.lora_enabled:
            kernel = self._kernel._value + (self.lora_alpha / self.lora_rank) * torch.matmul(self.lora_kernel_a._value, self.lora_kernel_b._value)
        targets = [kernel] + ([self.bias] if self.use_bias else [])
        for i, v in enumerate(targets):
            store[str(i)] = v

    def load_own_variables(self, store):
        if not self.built:
            return
        targets = [self._kernel] + ([self.bias] if self.use_bias else [])
        if len(store.keys()) != len(targets):
            raise ValueError(f"Layer '{self.name}' expected {len(targets)} variables, but received {len(store.keys())} variables during loading. Expected: {[v.name for v in targets]}")
        for i, v in enumerate(targets):
            v.assign(store[str(i)])
        if self.lora_enabled:
            self.lora_kernel_a.assign(torch.zeros_like(self.lora_kernel_a._value))
            self.lora_kernel_b.assign(torch.zeros_like(self.lora_kernel_b._value))

    def get_config(self):
        cfg = super().get_config()
        cfg.update({
            "filters": self.filters, "kernel_size": self.kernel_size, "strides": self.strides, "padding": self.padding,
            "data_format": self.data_format, "dilation_rate": self.dilation_rate, "groups": self.groups,
            "activation": activations.serialize(self.activation), "use_bias": self.use_bias,
            "kernel_initializer": initializers.serialize(self.kernel_initializer),
            "bias_initializer": initializers.serialize(self.bias_initializer),
            "kernel_regularizer": regularizers.serialize(self.kernel_regularizer),
            "bias_regularizer": regularizers.serialize(self.bias_regularizer),
            "activity_regularizer": regularizers.serialize(self.activity_regularizer),
            "kernel_constraint": constraints.serialize(self.kernel_constraint),
            "bias_constraint": constraints.serialize(self.bias_constraint),
        })
        if self.lora_rank:
            cfg["lora_rank"] = self.lora_rank
            cfg["lora_alpha"] = self.lora_alpha
        return cfg


def _make_conv(name, rank, exports):
    def __init__(self, filters, kernel_size, strides=1, padding="valid", data_format=None, dilation_rate=1, groups=1, activation=None,
                 use_bias=True, kernel_initializer="glorot_uniform", bias_initializer="zeros", kernel_regularizer=None,
                 bias_regularizer=None, activity_regularizer=None, kernel_constraint=None, bias_constraint=None, **kwargs):
        BaseConv.__init__(self, rank=rank, filters=filters, kernel_size=kernel_size, strides=strides, padding=padding,
                          data_format=data_format, dilation_rate=dilation_rate, groups=groups, activation=activation, use_bias=use_bias,
                          kernel_initializer=kernel_initializer, bias_initializer=bias_initializer, kernel_regularizer=kernel_regularizer,
                          bias_regularizer=bias_regularizer, activity_regularizer=activity_regularizer, kernel_constraint=kernel_constraint,
                          bias_constraint=bias_constraint, **kwargs)

    cls = type(name, (BaseConv,), {"__init__": __init__})
    cls.__module__ = __name__
    return keras_export(exports)(cls)


Conv1D = _make_conv("Conv1D", 1, ["keras.layers.Conv1D", "keras.layers.Convolution1D"])
Conv2D = _make_conv("Conv2D", 2, ["keras.layers.Conv2D", "keras.layers.Convolution2D"])
Conv3D = _make_conv("Conv3D", 3, ["keras.layers.Conv3D", "keras.layers.Convolution3D"])


def _conv1d_causal_call(self, inputs):
    return BaseConv.call(self, inputs)


def _conv1d_output_shape(self, input_shape):
    if self.padding == "causal":
        spatial = input_shape[1] if self.data_format == "channels_last" else input_shape[2]
        out = None if spatial is None else (spatial - 1) // self.strides[0] + 1
        if self.data_format == "channels_last":
            return (input_shape[0], out, self.filters)
        return (input_shape[0], self.filters, out)
    return BaseConv.compute_output_shape(self, input_shape)


Conv1D.compute_output_shape = _conv1d_output_shape


class BaseConvTranspose(Layer):
    def __init__(self, rank, filters, kernel_size, strides=1, padding="valid", output_padding=None, data_format=None, dilation_rate=1,
                 activation=None, use_bias=True, kernel_initializer="glorot_uniform", bias_initializer="zeros", kernel_regularizer=None,
                 bias_regularizer=None, activity_regularizer=None, kernel_constraint=None, bias_constraint=None, trainable=True, name=None, **kwargs):
        super().__init__(trainable=trainable, name=name, activity_regularizer=activity_regularizer, **kwargs)
        self.rank, self.filters = rank, filters
        self.kernel_size = standardize_tuple(kernel_size, rank, "kernel_size")
        self.strides = standardize_tuple(strides, rank, "strides")
        self.dilation_rate = standardize_tuple(dilation_rate, rank, "dilation_rate")
        self.padding = standardize_padding(padding)
        self.output_padding = None if output_padding is None else standardize_tuple(output_padding, rank, "output_padding", allow_zero=True)
        self.data_format = config.standardize_data_format(data_format)
        self.activation = activations.get(activation)
        self.use_bias = use_bias
        self.kernel_initializer = initializers.get(kernel_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.kernel_regularizer = regularizers.get(kernel_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.kernel_constraint = constraints.get(kernel_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.input_spec = InputSpec(min_ndim=rank + 2)
        if self.filters is not None and self.filters <= 0:
            raise ValueError(f"Invalid value for argument `filters`. Expected a strictly positive value. Received filters={self.filters}.")
        if max(self.strides) > 1 and max(self.dilation_rate) > 1:
            raise ValueError(f"`strides > 1` not supported in conjunction with `dilation_rate > 1`. Received: strides={self.strides} and dilation_rate={self.dilation_rate}")

    def build(self, input_shape):
        channel_axis = -1 if self.data_format == "channels_last" else 1
        input_channel = input_shape[channel_axis]
        self.input_spec = InputSpec(min_ndim=self.rank + 2, axes={channel_axis: input_channel})
        self.kernel = self.add_weight(name="kernel", shape=self.kernel_size + (self.filters, input_channel), initializer=self.kernel_initializer,
                                      regularizer=self.kernel_regularizer, constraint=self.kernel_constraint, trainable=True, dtype=self.dtype)
        if self.use_bias:
            self.bias = self.add_weight(name="bias", shape=(self.filters,), initializer=self.bias_initializer, regularizer=self.bias_regularizer,
                                        constraint=self.bias_constraint, trainable=True, dtype=self.dtype)
        else:
            self.bias = None
        self.built = True

    def call(self, inputs):
        outputs = ops.conv_transpose(inputs, self.kernel, strides=list(self.strides), padding=self.padding, output_padding=self.output_padding,
                                     dilation_rate=self.dilation_rate, data_format=self.data_format)
        if self.use_bias:
            if self.data_format == "channels_last":
                outputs = ops.add(outputs, self.bias)
            else:
                outputs = ops.add(outputs, ops.reshape(self.bias, (1, self.filters) + (1,) * self.rank))
        if self.activation is not None:
            return self.activation(outputs)
        return outputs

    def compute_output_shape(self, input_shape):
        spatial = input_shape[1:-1] if self.data_format == "channels_last" else input_shape[2:]
        out = []
        for i, d in enumerate(spatial):
            if d is None:
                out.append(None)
                continue
            out.append(deconv_output_length(d, self.kernel_size[i], self.padding, None if self.output_padding is None else self.output_padding[i], self.strides[i], self.dilation_rate[i]))
        if self.data_format == "channels_last":
            return (input_shape[0],) + tuple(out) + (self.filters,)
        return (input_shape[0], self.filters) + tuple(out)

    def get_config(self):
        cfg = super().get_config()
        cfg.update({
            "filters": self.filters, "kernel_size": self.kernel_size, "strides": self.strides, "padding": self.padding,
            "data_format": self.data_format, "dilation_rate": self.dilation_rate, "activation": activations.serialize(self.activation),
            "use_bias": self.use_bias, "kernel_initializer": initializers.serialize(self.kernel_initializer),
            "bias_initializer": initializers.serialize(self.bias_initializer), "kernel_regularizer": regularizers.serialize(self.kernel_regularizer),
            "bias_regularizer": regularizers.serialize(self.bias_regularizer), "activity_regularizer": regularizers.serialize(self.activity_regularizer),
            "kernel_constraint": constraints.serialize(self.kernel_constraint), "bias_constraint": constraints.serialize(self.bias_constraint),
        })
        if self.output_padding is not None:
            cfg["output_padding"] = self.output_padding
        return cfg


def deconv_output_length(input_length, kernel_size, padding, output_padding, stride, dilation=1):
    if input_length is None:
        return None
    eff = kernel_size + (kernel_size - 1) * (dilation - 1)
    if output_padding is None:
        if padding == "valid":
            return input_length * stride + max(eff - stride, 0)
        return input_length * stride
    pad = eff // 2 if padding == "same" else 0
    return (input_length - 1) * stride + eff - 2 * pad + output_padding


def _make_conv_t(name, rank, exports):
    def __init__(self, filters, kernel_size, strides=1, padding="valid", output_padding=None, data_format=None, dilation_rate=1, activation=None,
                 use_bias=True, kernel_initializer="glorot_uniform", bias_initializer="zeros", kernel_regularizer=None, bias_regularizer=None,
                 activity_regularizer=None, kernel_constraint=None, bias_constraint=None, **kwargs):
        BaseConvTranspose.__init__(self, rank=rank, filters=filters, kernel_size=kernel_size, strides=strides, padding=padding,
                                   output_padding=output_padding, data_format=data_format, dilation_rate=dilation_rate, activation=activation,
                                   use_bias=use_bias, kernel_initializer=kernel_initializer, bias_initializer=bias_initializer,
                                   kernel_regularizer=kernel_regularizer, bias_regularizer=bias_regularizer, activity_regularizer=activity_regularizer,
                                   kernel_constraint=kernel_constraint, bias_constraint=bias_constraint, **kwargs)

    cls = type(name, (BaseConvTranspose,), {"__init__": __init__})
    cls.__module__ = __name__
    return keras_export(exports)(cls)


Conv1DTranspose = _make_conv_t("Conv1DTranspose", 1, ["keras.layers.Conv1DTranspose", "keras.layers.Convolution1DTranspose"])
Conv2DTranspose = _make_conv_t("Conv2DTranspose", 2, ["keras.layers.Conv2DTranspose", "keras.layers.Convolution2DTranspose"])
Conv3DTranspose = _make_conv_t("Conv3DTranspose", 3, ["keras.layers.Conv3DTranspose", "keras.layers.Convolution3DTranspose"])


class BaseDepthwiseConv(Layer):
    def __init__(self, rank, depth_multiplier, kernel_size, strides=1, padding="valid", data_format=None, dilation_rate=1, activation=None,
                 use_bias=True, depthwise_initializer="glorot_uniform", bias_initializer="zeros", depthwise_regularizer=None,
                 bias_regularizer=None, activity_regularizer=None, depthwise_constraint=None, bias_constraint=None, trainable=True, name=None, **kwargs):
        super().__init__(trainable=trainable, name=name, activity_regularizer=regularizers.get(activity_regularizer), **kwargs)
        self.rank, self.depth_multiplier = rank, depth_multiplier
        self.kernel_size = standardize_tuple(kernel_size, rank, "kernel_size")
        self.strides = standardize_tuple(strides, rank, "strides")
        self.dilation_rate = standardize_tuple(dilation_rate, rank, "dilation_rate")
        self.padding = standardize_padding(padding)
        self.data_format = config.standardize_data_format(data_format)
        self.activation = activations.get(activation)
        self.use_bias = use_bias
        self.depthwise_initializer = initializers.get(depthwise_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.depthwise_regularizer = regularizers.get(depthwise_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.depthwise_constraint = constraints.get(depthwise_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.input_spec = InputSpec(min_ndim=rank + 2)
        if self.depth_multiplier is not None and self.depth_multiplier <= 0:
            raise ValueError(f"Invalid value for argument `depth_multiplier`. Expected a strictly positive value. Received depth_multiplier={self.depth_multiplier}.")
        if max(self.strides) > 1 and max(self.dilation_rate) > 1:
            raise ValueError(f"`strides > 1` not supported in conjunction with `dilation_rate > 1`. Received: strides={self.strides} and dilation_rate={self.dilation_rate}")

    def build(self, input_shape):
        channel_axis = -1 if self.data_format == "channels_last" else 1
        input_channel = input_shape[channel_axis]
        self.input_spec = InputSpec(min_ndim=self.rank + 2, axes={channel_axis: input_channel})
        self.kernel = self.add_weight(name="kernel", shape=self.kernel_size + (input_channel, self.depth_multiplier), initializer=self.depthwise_initializer,
                                      regularizer=self.depthwise_regularizer, constraint=self.depthwise_constraint, trainable=True, dtype=self.dtype)
        if self.use_bias:
            self.bias = self.add_weight(name="bias", shape=(self.depth_multiplier * input_channel,), initializer=self.bias_initializer,
                                        regularizer=self.bias_regularizer, constraint=self.bias_constraint, trainable=True, dtype=self.dtype)
        else:
            self.bias = None
        self.built = True

    def call(self, inputs):
        outputs = ops.depthwise_conv(inputs, self.kernel, strides=self.strides, padding=self.padding, dilation_rate=self.dilation_rate, data_format=self.data_format)
        if self.use_bias:
            if self.data_format == "channels_last":
                outputs = ops.add(outputs, self.bias)
            else:
                outputs = ops.add(outputs, ops.reshape(self.bias, (1, -1) + (1,) * self.rank))
        if self.activation is not None:
            return self.activation(outputs)
        return outputs

    def compute_output_shape(self, input_shape):
        channel_axis = -1 if self.data_format == "channels_last" else 1
        return conv_output_shape(input_shape, self.depth_multiplier * input_shape[channel_axis], self.kernel_size, self.strides, self.padding, self.data_format, self.dilation_rate)

    def get_config(self):
        cfg = super().get_config()
        cfg.update({
            "depth_multiplier": self.depth_multiplier, "kernel_size": self.kernel_size, "strides": self.strides, "padding": self.padding,
            "data_format": self.data_format, "dilation_rate": self.dilation_rate, "activation": activations.serialize(self.activation),
            "use_bias": self.use_bias, "depthwise_initializer": initializers.serialize(self.depthwise_initializer),
            "bias_initializer": initializers.serialize(self.bias_initializer), "depthwise_regularizer": regularizers.serialize(self.depthwise_regularizer),
            "bias_regularizer": regularizers.serialize(self.bias_regularizer), "activity_regularizer": regularizers.serialize(self.activity_regularizer),
            "depthwise_constraint": constraints.serialize(self.depthwise_constraint), "bias_constraint": constraints.serialize(self.bias_constraint),
        })
        return cfg


def _make_dw(name, rank, exports):
    def __init__(self, kernel_size, strides=1, padding="valid", depth_multiplier=1, data_format=None, dilation_rate=1, activation=None, use_bias=True,
                 depthwise_initializer="glorot_uniform", bias_initializer="zeros", depthwise_regularizer=None, bias_regularizer=None,
                 activity_regularizer=None, depthwise_constraint=None, bias_constraint=None, **kwargs):
        BaseDepthwiseConv.__init__(self, rank=rank, depth_multiplier=depth_multiplier, kernel_size=kernel_size, strides=strides, padding=padding,
                                   data_format=data_format, dilation_rate=dilation_rate, activation=activation, use_bias=use_bias,
                                   depthwise_initializer=depthwise_initializer, bias_initializer=bias_initializer,
                                   depthwise_regularizer=depthwise_regularizer, bias_regularizer=bias_regularizer,
                                   activity_regularizer=activity_regularizer, depthwise_constraint=depthwise_constraint,
                                   bias_constraint=bias_constraint, **kwargs)

    cls = type(name, (BaseDepthwiseConv,), {"__init__": __init__})
    cls.__module__ = __name__
    return keras_export(exports)(cls)


DepthwiseConv1D = _make_dw("DepthwiseConv1D", 1, ["keras.layers.DepthwiseConv1D"])
DepthwiseConv2D = _make_dw("DepthwiseConv2D", 2, ["keras.layers.DepthwiseConv2D"])


class BaseSeparableConv(Layer):
    def __init__(self, rank, depth_multiplier, filters, kernel_size, strides=1, padding="valid", data_format=None, dilation_rate=1, activation=None,
                 use_bias=True, depthwise_initializer="glorot_uniform", pointwise_initializer="glorot_uniform", bias_initializer="zeros",
                 depthwise_regularizer=None, pointwise_regularizer=None, bias_regularizer=None, activity_regularizer=None,
                 depthwise_constraint=None, pointwise_constraint=None, bias_constraint=None, trainable=True, name=None, **kwargs):
        super().__init__(trainable=trainable, name=name, activity_regularizer=regularizers.get(activity_regularizer), **kwargs)
        self.rank, self.depth_multiplier, self.filters = rank, depth_multiplier, filters
        self.kernel_size = standardize_tuple(kernel_size, rank, "kernel_size")
        self.strides = standardize_tuple(strides, rank, "strides")
        self.dilation_rate = standardize_tuple(dilation_rate, rank, "dilation_rate")
        self.padding = standardize_padding(padding)
        self.data_format = config.standardize_data_format(data_format)
        self.activation = activations.get(activation)
        self.use_bias = use_bias
        self.depthwise_initializer = initializers.get(depthwise_initializer)
        self.pointwise_initializer = initializers.get(pointwise_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.depthwise_regularizer = regularizers.get(depthwise_regularizer)
        self.pointwise_regularizer = regularizers.get(pointwise_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.depthwise_constraint = constraints.get(depthwise_constraint)
        self.pointwise_constraint = constraints.get(pointwise_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.input_spec = InputSpec(min_ndim=rank + 2)
        if self.depth_multiplier is not None and self.depth_multiplier <= 0:
            raise ValueError(f"Invalid value for argument `depth_multiplier`. Expected a strictly positive value. Received depth_multiplier={self.depth_multiplier}.")
        if self.filters is not None and self.filters <= 0:
            raise ValueError(f"Invalid value for argument `filters`. Expected a strictly positive value. Received filters={self.filters}.")
        if max(self.strides) > 1 and max(self.dilation_rate) > 1:
            raise ValueError(f"`strides > 1` not supported in conjunction with `dilation_rate > 1`. Received: strides={self.strides} and dilation_rate={self.dilation_rate}")

    def build(self, input_shape):
        channel_axis = -1 if self.data_format == "channels_last" else 1
        input_channel = input_shape[channel_axis]
        self.input_spec = InputSpec(min_ndim=self.rank + 2, axes={channel_axis: input_channel})
        self.depthwise_kernel = self.add_weight(name="depthwise_kernel", shape=self.kernel_size + (input_channel, self.depth_multiplier),
                                                initializer=self.depthwise_initializer, regularizer=self.depthwise_regularizer,
                                                constraint=self.depthwise_constraint, trainable=True, dtype=self.dtype)
        self.pointwise_kernel = self.add_weight(name="pointwise_kernel", shape=(1,) * self.rank + (self.depth_multiplier * input_channel, self.filters),
                                                initializer=self.pointwise_initializer, regularizer=self.pointwise_regularizer,
                                                constraint=self.pointwise_constraint, trainable=True, dtype=self.dtype)
        if self.use_bias:
            self.bias = self.add_weight(name="bias", shape=(self.filters,), initializer=self.bias_initializer, regularizer=self.bias_regularizer,
                                        constraint=self.bias_constraint, trainable=True, dtype=self.dtype)
        else:
            self.bias = None
        self.built = True

    def call(self, inputs):
        outputs = ops.separable_conv(inputs, self.depthwise_kernel, self.pointwise_kernel, strides=self.strides, padding=self.padding,
                                     dilation_rate=self.dilation_rate, data_format=self.data_format)
        if self.use_bias:
            if self.data_format == "channels_last":
                outputs = ops.add(outputs, self.bias)
            else:
                outputs = ops.add(outputs, ops.reshape(self.bias, (1, self.filters) + (1,) * self.rank))
        if self.activation is not None:
            return self.activation(outputs)
        return outputs

    def compute_output_shape(self, input_shape):
        return conv_output_shape(input_shape, self.filters, self.kernel_size, self.strides, self.padding, self.data_format, self.dilation_rate)

    def get_config(self):
        cfg = super().get_config()
        cfg.update({
            "depth_multiplier": self.depth_multiplier, "filters": self.filters, "kernel_size": self.kernel_size, "strides": self.strides,
            "padding": self.padding, "data_format": self.data_format, "dilation_rate": self.dilation_rate,
            "activation": activations.serialize(self.activation), "use_bias": self.use_bias,
            "depthwise_initializer": initializers.serialize(self.depthwise_initializer),
            "pointwise_initializer": initializers.serialize(self.pointwise_initializer),
            "bias_initializer": initializers.serialize(self.bias_initializer),
            "depthwise_regularizer": regularizers.serialize(self.depthwise_regularizer),
            "pointwise_regularizer": regularizers.serialize(self.pointwise_regularizer),
            "bias_regularizer": regularizers.serialize(self.bias_regularizer),
            "activity_regularizer": regularizers.serialize(self.activity_regularizer),
            "depthwise_constraint": constraints.serialize(self.depthwise_constraint),
            "pointwise_constraint": constraints.serialize(self.pointwise_constraint),
            "bias_constraint": constraints.serialize(self.bias_constraint),
        })
        return cfg


def _make_sep(name, rank, exports):
    def __init__(self, filters, kernel_size, strides=1, padding="valid", data_format=None, dilation_rate=1, depth_multiplier=1, activation=None,
                 use_bias=True, depthwise_initializer="glorot_uniform", pointwise_initializer="glorot_uniform", bias_initializer="zeros",
                 depthwise_regularizer=None, pointwise_regularizer=None, bias_regularizer=None, activity_regularizer=None,
                 depthwise_constraint=None, pointwise_constraint=None, bias_constraint=None, **kwargs):
        BaseSeparableConv.__init__(self, rank=rank, depth_multiplier=depth_multiplier, filters=filters, kernel_size=kernel_size, strides=strides,
                                   padding=padding, data_format=data_format, dilation_rate=dilation_rate, activation=activation, use_bias=use_bias,
                                   depthwise_initializer=depthwise_initializer, pointwise_initializer=pointwise_initializer,
                                   bias_initializer=bias_initializer, depthwise_regularizer=depthwise_regularizer,
                                   pointwise_regularizer=pointwise_regularizer, bias_regularizer=bias_regularizer,
                                   activity_regularizer=activity_regularizer, depthwise_constraint=depthwise_constraint,
                                   pointwise_constraint=pointwise_constraint, bias_constraint=bias_constraint, **kwargs)

    cls = type(name, (BaseSeparableConv,), {"__init__": __init__})
    cls.__module__ = __name__
    return keras_export(exports)(cls)


SeparableConv1D = _make_sep("SeparableConv1D", 1, ["keras.layers.SeparableConv1D", "keras.layers.SeparableConvolution1D"])
SeparableConv2D = _make_sep("SeparableConv2D", 2, ["keras.layers.SeparableConv2D", "keras.layers.SeparableConvolution2D"])
