"""Weight constraints (``keras.constraints``; keras/src/constraints/constraints.py)."""

import torch

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.utils.registry import build_lookup


@keras_export("keras.constraints.Constraint")
class Constraint:
    def __call__(self, w):
        return w

    def get_config(self):
        return {}

    @classmethod
    def from_config(cls, config):
        return cls(**config)


def _norms(w, axis):
    return torch.sqrt(torch.sum(torch.square(w), dim=axis, keepdim=True))


@keras_export(["keras.constraints.MaxNorm", "keras.constraints.max_norm"])
class MaxNorm(Constraint):
    def __init__(self, max_value=2, axis=0):
        self.max_value, self.axis = max_value, axis

    def __call__(self, w):
        w = convert_to_tensor(w)
        norms = _norms(w, self.axis)
        desired = torch.clip(norms, 0, self.max_value)
        return w * (desired / (config.epsilon() + norms))

    def get_config(self):
        return {"max_value": self.max_value, "axis": self.axis}


@keras_export(["keras.constraints.NonNeg", "keras.constraints.non_neg"])
class NonNeg(Constraint):
    def __call__(self, w):
        w = convert_to_tensor(w)
        return w * (w >= 0).to(w.dtype)


@keras_export(["keras.constraints.UnitNorm", "keras.constraints.unit_norm"])
class UnitNorm(Constraint):
    def __init__(self, axis=0):
        self.axis = axis

    def __call__(self, w):
        w = convert_to_tensor(w)
        return w / (config.epsilon() + _norms(w, self.axis))

    def get_config(self):
        return {"axis": self.axis}


@keras_export(["keras.constraints.MinMaxNorm", "keras.constraints.min_max_norm"])
class MinMaxNorm(Constraint):
    def __init__(self, min_value=0.0, max_value=1.0, rate=1.0, axis=0):
        self.min_value, self.max_value, self.rate, self.axis = min_value, max_value, rate, axis

    def __call__(self, w):
        w = convert_to_tensor(w)
        norms = _norms(w, self.axis)
        desired = self.rate * torch.clip(norms, self.min_value, self.max_value) + (1 - self.rate) * norms
        return w * (desired / (config.epsilon() + norms))

    def get_config(self):
        return {"min_value": self.min_value, "max_value": self.max_value, "rate": self.rate, "axis": self.axis}


ALL_OBJECTS = [Constraint, MaxNorm, MinMaxNorm, NonNeg, UnitNorm]
_LOOKUP = build_lookup(ALL_OBJECTS)
max_norm, min_max_norm, non_neg, unit_norm = MaxNorm, MinMaxNorm, NonNeg, UnitNorm


@keras_export("keras.constraints.serialize")
def serialize(constraint):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(constraint)


@keras_export("keras.constraints.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(config, module_objects=_LOOKUP, custom_objects=custom_objects)


@keras_export("keras.constraints.get")
def get(identifier):
    if identifier is None:
        return None
    if isinstance(identifier, dict):
        obj = deserialize(identifier)
    elif isinstance(identifier, str):
        obj = _LOOKUP.get(identifier)
        if obj is None:
            raise ValueError(f"Could not interpret constraint identifier: {identifier}")
    else:
        obj = identifier
    if callable(obj):
        return obj() if isinstance(obj, type) else obj
    raise ValueError(f"Could not interpret constraint identifier: {identifier}")
