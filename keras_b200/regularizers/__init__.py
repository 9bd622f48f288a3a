"""Weight regularizers (``keras.regularizers``; keras/src/regularizers/regularizers.py)."""

import math

import torch

from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.utils.registry import build_lookup


def _check(x, name):
    if not isinstance(x, (float, int)) or math.isinf(x) or math.isnan(x) or x < 0:
        raise ValueError(f"Invalid value for argument {name}: expected a non-negative float. Received: {name}={x}")
    return float(x)


@keras_export(["keras.Regularizer", "keras.regularizers.Regularizer"])
class Regularizer:
    def __call__(self, x):
        return 0.0

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def get_config(self):
        raise NotImplementedError(f"{self} does not implement get_config()")


@keras_export(["keras.regularizers.L1L2", "keras.regularizers.l1_l2"])
class L1L2(Regularizer):
    def __init__(self, l1=0.0, l2=0.0):
        self.l1 = _check(0.0 if l1 is None else l1, "l1")
        self.l2 = _check(0.0 if l2 is None else l2, "l2")

    def __call__(self, x):
        x = convert_to_tensor(x)
        out = torch.zeros((), dtype=x.dtype, device=x.device)
        if self.l1:
            out = out + self.l1 * torch.sum(torch.abs(x))
        if self.l2:
            out = out + self.l2 * torch.sum(torch.square(x))
        return out

    def get_config(self):
        return {"l1": self.l1, "l2": self.l2}


@keras_export(["keras.regularizers.L1", "keras.regularizers.l1"])
class L1(Regularizer):
    def __init__(self, l1=0.01):
        self.l1 = _check(0.01 if l1 is None else l1, "l1")

    def __call__(self, x):
        return self.l1 * torch.sum(torch.abs(convert_to_tensor(x)))

    def get_config(self):
        return {"l1": self.l1}


@keras_export(["keras.regularizers.L2", "keras.regularizers.l2"])
class L2(Regularizer):
    def __init__(self, l2=0.01):
        self.l2 = _check(0.01 if l2 is None else l2, "l2")

    def __call__(self, x):
        return self.l2 * torch.sum(torch.square(convert_to_tensor(x)))

    def get_config(self):
        return {"l2": self.l2}


@keras_export(["keras.regularizers.OrthogonalRegularizer", "keras.regularizers.orthogonal_regularizer"])
class OrthogonalRegularizer(Regularizer):
    def __init__(self, factor=0.01, mode="rows"):
        self.factor = _check(factor, "factor")
        if mode not in {"rows", "columns"}:
            raise ValueError(f"Invalid value for argument `mode`. Expected one of {{'rows', 'columns'}}. Received: mode={mode}")
        self.mode = mode

    def __call__(self, inputs):
        x = convert_to_tensor(inputs)
        if x.ndim != 2:
            raise ValueError(f"Inputs to OrthogonalRegularizer must have rank 2. Received: inputs.shape={tuple(x.shape)}")
        if self.mode == "rows":
            x = torch.nn.functional.normalize(x, dim=1)
            prod = x @ x.t()
            size = x.shape[0]
        else:
            x = torch.nn.functional.normalize(x, dim=0)
            prod = x.t() @ x
            size = x.shape[1]
        off = prod * (1.0 - torch.eye(size, dtype=x.dtype, device=x.device))
        pairs = size * (size - 1.0) / 2.0
        return self.factor * 0.5 * torch.sum(torch.abs(off)) / pairs

    def get_config(self):
        return {"factor": self.factor, "mode": self.mode}


ALL_OBJECTS = [Regularizer, L1, L2, L1L2, OrthogonalRegularizer]
_LOOKUP = build_lookup(ALL_OBJECTS, {"l1": L1, "l2": L2, "l1_l2": L1L2, "l1l2": L1L2})
l1, l2, l1_l2, orthogonal_regularizer = L1, L2, L1L2, OrthogonalRegularizer


@keras_export("keras.regularizers.serialize")
def serialize(regularizer):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(regularizer)


@keras_export("keras.regularizers.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(config, module_objects=_LOOKUP, custom_objects=custom_objects)


@keras_export("keras.regularizers.get")
def get(identifier):
    if identifier is None:
        return None
    if isinstance(identifier, dict):
        obj = deserialize(identifier)
    elif isinstance(identifier, str):
        obj = _LOOKUP.get(identifier)
        if obj is None:
            raise ValueError(f"Could not interpret regularizer identifier: {identifier}")
    else:
        obj = identifier
    if callable(obj):
        return obj() if isinstance(obj, type) else obj
    raise ValueError(f"Could not interpret regularizer identifier: {identifier}")
