"""Activation functions (``keras.activations``; keras/src/activations/activations.py)."""

import types

import torch

from keras_b200.core.export_registry import keras_export
from keras_b200.ops import nn as _nn
from keras_b200.ops import numpy as _np


def _export(name, fn, aliases=()):
    fn.__name__ = name
    keras_export([f"keras.activations.{name}"] + [f"keras.activations.{a}" for a in aliases])(fn)
    return fn


def relu(x, negative_slope=0.0, max_value=None, threshold=0.0):
    from keras_b200.core.keras_tensor import KerasTensor

    if negative_slope == 0.0 and max_value is None and threshold == 0.0:
        return _nn.relu(x)
    if isinstance(x, KerasTensor):
        return KerasTensor(x.shape, x.dtype)
    x = _np._floatize(x)
    if negative_slope != 0.0:
        if max_value is None and threshold == 0.0:
            return _nn.leaky_relu(x, negative_slope=negative_slope)
        neg = torch.relu(-x + threshold) if threshold != 0 else torch.relu(-x)
    else:
        neg = None
    if threshold != 0:
        x = x * (x > threshold).to(x.dtype)
    elif max_value == 6 and neg is None:
        return _nn.relu6(x)
    else:
        x = torch.relu(x)
    if max_value is not None:
        x = torch.clip(x, 0.0, max_value)
    if neg is not None:
        x = x - negative_slope * neg
    return x


relu = _export("relu", relu)
leaky_relu = _export("leaky_relu", lambda x, negative_slope=0.2: _nn.leaky_relu(x, negative_slope=negative_slope))
relu6 = _export("relu6", lambda x: _nn.relu6(x))
softmax = _export("softmax", lambda x, axis=-1: _nn.softmax(x, axis=axis))
elu = _export("elu", lambda x, alpha=1.0: _nn.elu(x, alpha=alpha))
selu = _export("selu", lambda x: _nn.selu(x))
softplus = _export("softplus", lambda x: _nn.softplus(x))
softsign = _export("softsign", lambda x: _nn.softsign(x))
soft_shrink = _export("soft_shrink", lambda x, threshold=0.5: _nn.soft_shrink(x, threshold=threshold))
sparse_plus = _export("sparse_plus", lambda x: _nn.sparse_plus(x))
silu = _export("silu", lambda x: _nn.silu(x), aliases=("swish",))
swish = silu
squareplus = _export("squareplus", lambda x, b=4: _nn.squareplus(x, b=b))
gelu = _export("gelu", lambda x, approximate=False: _nn.gelu(x, approximate=approximate))
celu = _export("celu", lambda x, alpha=1.0: _nn.celu(x, alpha=alpha))
glu = _export("glu", lambda x, axis=-1: _nn.glu(x, axis=axis))
tanh = _export("tanh", lambda x: _nn.tanh(x))
tanh_shrink = _export("tanh_shrink", lambda x: _nn.tanh_shrink(x))
threshold = _export("threshold", lambda x, threshold, default_value: _nn.threshold(x, threshold, default_value))
sigmoid = _export("sigmoid", lambda x: _nn.sigmoid(x))
sparse_sigmoid = _export("sparse_sigmoid", lambda x: _nn.sparse_sigmoid(x))
exponential = _export("exponential", lambda x: _np.exp(x))
hard_sigmoid = _export("hard_sigmoid", lambda x: _nn.hard_sigmoid(x))
log_sigmoid = _export("log_sigmoid", lambda x: _nn.log_sigmoid(x))
hard_silu = _export("hard_silu", lambda x: _nn.hard_silu(x), aliases=("hard_swish",))
hard_swish = hard_silu
hard_tanh = _export("hard_tanh", lambda x: _nn.hard_tanh(x))
hard_shrink = _export("hard_shrink", lambda x, threshold=0.5: _nn.hard_shrink(x, threshold=threshold))
linear = _export("linear", lambda x: x)
mish = _export("mish", lambda x: _np.multiply(x, _nn.tanh(_nn.softplus(x))))
log_softmax = _export("log_softmax", lambda x, axis=-1: _nn.log_softmax(x, axis=axis))
sparsemax = _export("sparsemax", lambda x, axis=-1: _nn.sparsemax(x, axis=axis))

ALL_OBJECTS = {
    relu, leaky_relu, relu6, softmax, celu, elu, selu, softplus, softsign, squareplus, soft_shrink,
    sparse_plus, silu, gelu, glu, tanh, tanh_shrink, threshold, sigmoid, sparse_sigmoid, exponential,
    hard_sigmoid, hard_silu, hard_tanh, hard_shrink, linear, mish, log_softmax, log_sigmoid, sparsemax,
}
ALL_OBJECTS_DICT = {fn.__name__: fn for fn in ALL_OBJECTS}
ALL_OBJECTS_DICT["swish"] = silu
ALL_OBJECTS_DICT["hard_swish"] = hard_silu


@keras_export("keras.activations.serialize")
def serialize(activation):
    if activation is None or activation is linear:
        return "linear"
    name = getattr(activation, "__name__", None)
    if name in ALL_OBJECTS_DICT and ALL_OBJECTS_DICT[name] is activation:
        return name
    from keras_b200.saving import serialization_lib

    fn_config = serialization_lib.serialize_keras_object(activation)
    if isinstance(fn_config, dict) and "config" in fn_config and not isinstance(fn_config["config"], dict):
        return fn_config
    return fn_config


@keras_export("keras.activations.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(config, module_objects=ALL_OBJECTS_DICT, custom_objects=custom_objects)


@keras_export("keras.activations.get")
def get(identifier):
    if identifier is None:
        return linear
    if isinstance(identifier, dict):
        obj = deserialize(identifier)
    elif isinstance(identifier, str):
        obj = ALL_OBJECTS_DICT.get(identifier)
        if obj is None:
            from keras_b200.saving import object_registration

            obj = object_registration.get_registered_object(identifier)
    else:
        obj = identifier
    if callable(obj):
        return obj
    raise ValueError(f"Could not interpret activation function identifier: {identifier}")
