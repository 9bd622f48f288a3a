"""``DTypePolicyMap``: dict-like ``layer path → DTypePolicy`` (keras/src/dtype_policies/dtype_policy_map.py:10-294)."""

import re
from collections.abc import MutableMapping

from keras_b200.core.export_registry import keras_export


@keras_export("keras.dtype_policies.DTypePolicyMap")
class DTypePolicyMap(MutableMapping):
    def __init__(self, default_policy=None, policy_map=None):
        from keras_b200 import dtype_policies

        if isinstance(default_policy, DTypePolicyMap):
            raise ValueError("`default_policy` cannot be a `DTypePolicyMap`.")
        if policy_map is not None and not isinstance(policy_map, dict):
            raise TypeError(f"If specified, `policy_map` must be a dict. Received: policy_map={policy_map} of type {type(policy_map)}")
        self._default_policy_arg = default_policy
        self._default_policy = dtype_policies.get(default_policy)
        self._policy_map = policy_map or {}

    name = property(lambda self: f"map_{self.default_policy._name}")
    default_policy = property(lambda self: __import__("keras_b200").dtype_policies.get(self._default_policy))
    variable_dtype = property(lambda self: self.default_policy.variable_dtype)
    compute_dtype = property(lambda self: self.default_policy.compute_dtype)
    quantization_mode = property(lambda self: self.default_policy.quantization_mode)
    is_quantized = property(lambda self: self.default_policy.is_quantized)

    def __getitem__(self, key):
        from keras_b200 import dtype_policies

        if key in self._policy_map:
            return self._policy_map[key]
        matches = [k for k in self._policy_map if re.fullmatch(k, key) or key.startswith(k + "/") or re.search(f"^{k}(/|$)", key)]
        matches = [k for k in matches]
        if len(matches) > 1:
            exact = [k for k in matches if re.fullmatch(k, key)]
            if len(exact) == 1:
                return self._policy_map[exact[0]]
            raise ValueError(f"Path '{key}' matches multiple dtype policy specification keys: {matches}. Please make sure each path only matches at most one dtype policy specification key in the DTypePolicyMap.")
        if len(matches) == 1:
            return self._policy_map[matches[0]]
        return self.default_policy

    def __setitem__(self, key, policy):
        from keras_b200 import dtype_policies

        if key in self._policy_map:
            raise ValueError(f"{key} already exist in the DTypePolicyMap with value {self._policy_map[key]}. Please make sure to not use duplicated keys.")
        try:
            policy = dtype_policies.get(policy)
        except Exception:
            raise ValueError(f"Cannot interpret the assigned value by `keras.dtype_policies.get`. Received: {policy} of type {type(policy)}")
        self._policy_map[key] = policy

    def __delitem__(self, key):
        return self._policy_map.pop(key)

    def __contains__(self, key):
        return key in self._policy_map

    def __len__(self):
        return len(self._policy_map)

    def __iter__(self):
        return iter(self._policy_map)

    def __repr__(self):
        default = self._default_policy.name if self._default_policy is not None else None
        mapping = [(k, v._name) for k, v in self._policy_map.items()]
        return f"<DTypePolicyMap at {hex(id(self))} default_policy={default}, mapping={mapping}>"

    def convert_input(self, x, autocast, dtype):
        return self.default_policy.convert_input(x, autocast, dtype)

    def get_config(self):
        from keras_b200 import dtype_policies

        policy_map = {k: dtype_policies.serialize(v) for k, v in self._policy_map.items()}
        return {"default_policy": self._default_policy_arg if isinstance(self._default_policy_arg, (str, type(None))) else self._default_policy.name, "policy_map": policy_map}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        from keras_b200 import dtype_policies

        policy_map = {k: dtype_policies.deserialize(v, custom_objects=custom_objects) for k, v in config["policy_map"].items()}
        return cls(default_policy=config["default_policy"], policy_map=policy_map)
