"""Dtype policies (``keras.dtype_policies`` / ``keras.mixed_precision``).

Behaviour of keras/src/dtype_policies/dtype_policy.py:7-638 and dtype_policy_map.py:10-294:
``"mixed_bfloat16"`` → compute bf16 / variables fp32; quantized policies are spelled
``"<mode>_from_<source>"``.
"""

import re

from keras_b200.core import config as _config
from keras_b200.core import global_state
from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.export_registry import keras_export

QUANTIZATION_MODES = ("int8", "float8", "int4", "gptq", "awq", "ternary")


@keras_export(["keras.DTypePolicy", "keras.dtype_policies.DTypePolicy", "keras.mixed_precision.DTypePolicy",
               "keras.mixed_precision.Policy", "keras.FloatDTypePolicy", "keras.dtype_policies.FloatDTypePolicy"])
class DTypePolicy:
    def __init__(self, name=None):
        if name is None:
            name = dtype_policy().name
        if not isinstance(name, str):
            raise TypeError(f"'name' must be a string, such as 'mixed_float16'. Received: name={name} (of type {type(name)})")
        self._name = name
        self._compute_dtype, self._variable_dtype = self._parse_name(name)
        self._quantization_mode = None
        self._is_quantized = False

    def _parse_name(self, name):
        if name == "mixed_float16":
            return "float16", "float32"
        if name == "mixed_bfloat16":
            return "bfloat16", "float32"
        try:
            d = standardize_dtype(name)
            return d, d
        except ValueError:
            raise ValueError(
                f"Cannot convert '{name}' to a mixed precision DTypePolicy. Valid policies include "
                "'mixed_float16', 'mixed_bfloat16', and the name of any float dtype such as 'float32'."
            )

    variable_dtype = property(lambda self: self._variable_dtype)
    compute_dtype = property(lambda self: self._compute_dtype)
    name = property(lambda self: self._name)
    quantization_mode = property(lambda self: self._quantization_mode)
    is_quantized = property(lambda self: self._is_quantized)

    def convert_input(self, x, autocast, dtype):
        import numpy as np
        import torch

        from keras_b200.core.keras_tensor import KerasTensor

        dtype = standardize_dtype(dtype)
        if isinstance(x, torch.Tensor):
            if autocast and x.dtype.is_floating_point:
                from keras_b200.core.dtypes import to_torch_dtype

                td = to_torch_dtype(dtype)
                if x.dtype != td and td.is_floating_point:
                    x = x.to(td)
            from keras_b200.core.tensor import get_device

            dev = get_device()
            if x.device != dev and dev.type != "meta" and x.device.type != "meta" and not (x.device.type == dev.type and dev.index is None):
                x = x.to(dev)
            return x
        if isinstance(x, KerasTensor):
            if autocast and ("float" in x.dtype) and x.dtype != dtype:
                x = KerasTensor(x.shape, dtype=dtype, sparse=x.sparse, name=x.name) if False else _cast_keras_tensor(x, dtype)
            return x
        if hasattr(x, "__array__"):
            from keras_b200.core.tensor import convert_to_tensor

            t = convert_to_tensor(x)
            if autocast and t.dtype.is_floating_point:
                from keras_b200.core.dtypes import to_torch_dtype

                t = t.to(to_torch_dtype(dtype))
            return t
        return x

    def get_config(self):
        return {"name": self.name}

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def __repr__(self):
        return f'<{self.__class__.__name__} "{self._name}">'

    def __eq__(self, other):
        if self.__class__ in (DTypePolicy,):
            if type(other) is not DTypePolicy:
                return False
        elif type(other) is not self.__class__:
            return False
        return self._name == other._name

    def __hash__(self):
        return hash((self.__class__.__name__, self._name))

    def _get_quantized_dtype_policy_by_str(self, policy):
        raise NotImplementedError


def _cast_keras_tensor(x, dtype):
    from keras_b200 import ops

    return ops.cast(x, dtype)


FloatDTypePolicy = DTypePolicy


@keras_export("keras.dtype_policies.QuantizedDTypePolicy")
class QuantizedDTypePolicy(DTypePolicy):
    def __init__(self, mode, source_name=None):
        name = self._name_for(mode, source_name)
        self._source_name = name.split("_from_")[1]
        self._name = name
        self._compute_dtype, self._variable_dtype = self._parse_name(self._source_name)
        self._quantization_mode = mode
        self._is_quantized = True
        _validate_mode_dtype(mode, self._compute_dtype)

    def _name_for(self, mode, source_name):
        if source_name is None:
            source_name = dtype_policy().name
        return f"{mode}_from_{source_name}"

    def get_config(self):
        return {"mode": self._quantization_mode, "source_name": self._source_name}

    def __eq__(self, other):
        return type(other) is type(self) and self._name == other._name and self._quantization_mode == other._quantization_mode

    __hash__ = DTypePolicy.__hash__


def _validate_mode_dtype(mode, compute_dtype):
    valid = {"int8": ("bfloat16", "float16", "float32", "float64"), "float8": ("bfloat16", "float16", "float32", "float64"),
             "int4": ("bfloat16", "float16", "float32", "float64"), "gptq": ("bfloat16", "float16", "float32", "float64"),
             "awq": ("bfloat16", "float16", "float32", "float64"), "ternary": ("bfloat16", "float16", "float32", "float64")}
    if mode not in valid:
        raise ValueError(f"Invalid quantization mode. Expected one of {QUANTIZATION_MODES}. Received: mode={mode}")
    if compute_dtype not in valid[mode]:
        raise ValueError(f"Quantization mode='{mode}' doesn't work well with compute_dtype='{compute_dtype}'.")


@keras_export("keras.dtype_policies.QuantizedFloat8DTypePolicy")
class QuantizedFloat8DTypePolicy(QuantizedDTypePolicy):
    default_amax_history_length = 1024

    def __init__(self, mode, source_name=None, amax_history_length=1024):
        super().__init__(mode=mode, source_name=source_name)
        if not isinstance(amax_history_length, int):
            raise TypeError(f"`amax_history_length` must be an integer. Received: amax_history_length={amax_history_length}")
        self._amax_history_length = amax_history_length

    amax_history_length = property(lambda self: self._amax_history_length)

    def get_config(self):
        cfg = super().get_config()
        cfg["amax_history_length"] = self._amax_history_length
        return cfg

    def __eq__(self, other):
        return super().__eq__(other) and self._amax_history_length == other._amax_history_length

    __hash__ = DTypePolicy.__hash__


@keras_export("keras.dtype_policies.Int4DTypePolicy")
class Int4DTypePolicy(QuantizedDTypePolicy):
    """``"int4/<block>_from_<source>"``; ``block_size`` −1 means per-channel."""

    def __init__(self, mode="int4", source_name=None, block_size=None):
        if "/" in mode:
            mode, bs = mode.split("/")
            block_size = int(bs)
        self.block_size = 128 if block_size is None else block_size
        super().__init__(mode="int4", source_name=source_name)
        self._name = f"int4/{self.block_size}_from_{self._source_name}"

    def get_config(self):
        return {"mode": "int4", "source_name": self._source_name, "block_size": self.block_size}


@keras_export("keras.dtype_policies.TernaryDTypePolicy")
class TernaryDTypePolicy(QuantizedDTypePolicy):
    def __init__(self, mode="ternary", source_name=None):
        super().__init__(mode="ternary", source_name=source_name)


@keras_export("keras.dtype_policies.GPTQDTypePolicy")
class GPTQDTypePolicy(QuantizedDTypePolicy):
    """``"gptq/<weight_bits>/<group_size>_from_<source>"``."""

    def __init__(self, mode, source_name=None):
        parts = mode.split("/")
        if len(parts) != 3 or parts[0] != "gptq":
            raise ValueError(f"Invalid mode for GPTQDTypePolicy. Expected format `gptq/<weight_bits>/<group_size>`, but got '{mode}'.")
        self.weight_bits, self.group_size = int(parts[1]), int(parts[2])
        if self.weight_bits not in (2, 3, 4, 8):
            raise ValueError(f"Invalid weight_bits in mode. Supported values are 2, 3, 4, and 8, but got {self.weight_bits} from '{mode}'")
        if self.group_size < -1 or self.group_size == 0:
            raise ValueError(f"Invalid group_size in mode. Supported values are -1 (whole-tensor) or a positive integer, but got {self.group_size} from '{mode}'.")
        self._full_mode = mode
        super().__init__(mode="gptq", source_name=source_name)
        self._name = f"{mode}_from_{self._source_name}"

    def get_config(self):
        return {"mode": self._full_mode, "source_name": self._source_name}


@keras_export("keras.dtype_policies.AWQDTypePolicy")
class AWQDTypePolicy(QuantizedDTypePolicy):
    """``"awq/<weight_bits>/<group_size>_from_<source>"``."""

    def __init__(self, mode, source_name=None):
        parts = mode.split("/")
        if len(parts) != 3 or parts[0] != "awq":
            raise ValueError(f"Invalid mode for AWQDTypePolicy. Expected format `awq/<weight_bits>/<group_size>`, but got '{mode}'.")
        self.weight_bits, self.group_size = int(parts[1]), int(parts[2])
        if self.weight_bits != 4:
            raise ValueError(f"AWQ only supports 4-bit weights, but got {self.weight_bits} from '{mode}'")
        self._full_mode = mode
        super().__init__(mode="awq", source_name=source_name)
        self._name = f"{mode}_from_{self._source_name}"

    def get_config(self):
        return {"mode": self._full_mode, "source_name": self._source_name}


@keras_export(["keras.config.set_dtype_policy", "keras.mixed_precision.set_dtype_policy", "keras.mixed_precision.set_global_policy"])
def set_dtype_policy(policy):
    if not isinstance(policy, DTypePolicy):
        if isinstance(policy, str):
            policy = _policy_from_str(policy)
        else:
            raise ValueError(
                "Invalid `policy` argument. Expected the string name of a policy (such as "
                f"'mixed_float16') or a `DTypePolicy` instance. Received: policy={policy} (of type {type(policy)})"
            )
    global_state.set_global_attribute("dtype_policy", policy)


@keras_export(["keras.config.dtype_policy", "keras.mixed_precision.dtype_policy", "keras.mixed_precision.global_policy"])
def dtype_policy():
    policy = global_state.get_global_attribute("dtype_policy", None)
    if policy is None:
        policy = DTypePolicy(_config.floatx())
        global_state.set_global_attribute("dtype_policy", policy)
    return policy


def _policy_from_str(name):
    if "_from_" in name:
        mode, source = name.split("_from_", 1)
        if mode.startswith("int4"):
            return Int4DTypePolicy(mode, source)
        if mode.startswith("gptq"):
            return GPTQDTypePolicy(mode, source)
        if mode.startswith("awq"):
            return AWQDTypePolicy(mode, source)
        if mode == "float8":
            return QuantizedFloat8DTypePolicy(mode, source)
        if mode == "ternary":
            return TernaryDTypePolicy(mode, source)
        if mode == "int8":
            return QuantizedDTypePolicy(mode, source)
        raise ValueError(f"Cannot convert `policy` into a valid pre-defined `DTypePolicy`. Received: policy={name}")
    return DTypePolicy(name)


ALL_OBJECTS = [DTypePolicy, QuantizedDTypePolicy, QuantizedFloat8DTypePolicy, Int4DTypePolicy, TernaryDTypePolicy, GPTQDTypePolicy, AWQDTypePolicy]
_LOOKUP = {c.__name__: c for c in ALL_OBJECTS}
_LOOKUP["FloatDTypePolicy"] = DTypePolicy


@keras_export("keras.dtype_policies.serialize")
def serialize(policy):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(policy)


@keras_export("keras.dtype_policies.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(config, module_objects=_LOOKUP, custom_objects=custom_objects)


@keras_export("keras.dtype_policies.get")
def get(identifier):
    from keras_b200.dtype_policies.dtype_policy_map import DTypePolicyMap

    if identifier is None:
        return dtype_policy()
    if isinstance(identifier, (DTypePolicy, DTypePolicyMap)):
        return identifier
    if isinstance(identifier, dict):
        return deserialize(identifier)
    if isinstance(identifier, str):
        return _policy_from_str(identifier)
    try:
        return DTypePolicy(standardize_dtype(identifier))
    except Exception:
        raise ValueError(f"Cannot interpret `dtype` argument. Expected a string or an instance of DTypePolicy. Received: dtype={identifier}")


def __getattr__(name):
    if name == "DTypePolicyMap":
        from keras_b200.dtype_policies.dtype_policy_map import DTypePolicyMap

        return DTypePolicyMap
    raise AttributeError(f"module 'keras_b200.dtype_policies' has no attribute {name!r}")
