"""``Operation``: the callable unit of both eager execution and symbolic graph building.

Behaviour of keras/src/ops/operation.py:21-448: calling with any ``KerasTensor`` argument
records a ``Node`` and returns symbolic outputs; otherwise ``call`` runs eagerly.  Constructor
arguments are captured so that ``get_config`` works without boilerplate.
"""

import inspect

from keras_b200 import tree
from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor, any_symbolic_tensors
from keras_b200.core.naming import auto_name
from keras_b200.ops.node import Node


class KerasSaveable:
    """Marker base for objects the archive writer walks (layers, optimizers, metrics…)."""

    def _obj_type(self):
        raise NotImplementedError

    def __reduce__(self):
        from keras_b200.saving import pickle_support

        return pickle_support.reduce_saveable(self)


@keras_export(["keras.Operation", "keras.ops.Operation"])
class Operation(KerasSaveable):
    def __init__(self, name=None):
        if name is None:
            name = auto_name(self.__class__.__name__)
        if not isinstance(name, str) or "/" in name:
            raise ValueError(
                "Argument `name` must be a string and cannot contain character `/`. "
                f"Received: name={name} (of type {type(name)})"
            )
        self.name = name
        self._inbound_nodes = []
        self._outbound_nodes = []

    def __new__(cls, *args, **kwargs):
        instance = super().__new__(cls)
        # Capture constructor arguments for the default `get_config`.
        try:
            sig = _init_signature(cls)
            names = [p for p in sig if p != "self"]
            captured = dict(kwargs)
            positional = [n for n, kind in sig.items() if kind in (0, 1) and n != "self"]
            for n, v in zip(positional, args):
                captured[n] = v
            if len(args) > len(positional):
                captured = None  # *args present: cannot map
            instance._auto_config = captured
        except Exception:
            instance._auto_config = None
        instance._lock = False
        return instance

    def __call__(self, *args, **kwargs):
        if any_symbolic_tensors(args, kwargs):
            return self.symbolic_call(*args, **kwargs)
        return self.call(*args, **kwargs)

    def symbolic_call(self, *args, **kwargs):
        outputs = self.compute_output_spec(*args, **kwargs)
        Node(operation=self, call_args=args, call_kwargs=kwargs, outputs=outputs)
        return outputs

    def call(self, *args, **kwargs):
        raise NotImplementedError

    def quantized_call(self, *args, **kwargs):
        raise NotImplementedError

    def compute_output_spec(self, *args, **kwargs):
        from keras_b200.core.tensor import compute_output_spec

        try:
            return compute_output_spec(self.call, *args, **kwargs)
        except Exception as e:
            raise e.__class__(
                "Could not automatically infer the output shape / dtype of "
                f"'{self.name}' (of type {self.__class__.__name__}). Either the "
                "`call()` method is incorrect, or you need to implement "
                "`compute_output_spec()` / `compute_output_shape()`. Error encountered:\n\n"
                f"{e}"
            )

    def get_config(self):
        config = {"name": self.name}
        auto = getattr(self, "_auto_config", None)
        if auto is None:
            if type(self).__init__ is not Operation.__init__ and _has_extra_init_args(type(self)):
                raise NotImplementedError(
                    f"Operation {self.__class__.__name__} has constructor arguments that could not "
                    "be captured automatically. Implement `get_config()` (and `from_config()`) "
                    "to make it serializable."
                )
            return config
        from keras_b200.saving import serialization_lib

        for k, v in auto.items():
            if k in config:
                continue
            try:
                config[k] = serialization_lib.serialize_keras_object(v)
            except Exception:
                raise NotImplementedError(
                    f"Argument `{k}` of {self.__class__.__name__} is not serializable; implement "
                    "`get_config()` explicitly."
                )
        return config

    @classmethod
    def from_config(cls, config):
        config = dict(config)
        if "dtype" in config and isinstance(config["dtype"], dict):
            from keras_b200 import dtype_policies

            config["dtype"] = dtype_policies.deserialize(config["dtype"])
        try:
            return cls(**config)
        except Exception as e:
            raise TypeError(
                f"Error when deserializing class '{cls.__name__}' using config={config}.\n\n"
                f"Exception encountered: {e}"
            )

    def __repr__(self):
        return f"<Operation name={self.name}>"

    # -- graph accessors -----------------------------------------------------------------
    def _node_attr(self, node_index, attr, label):
        if not self._inbound_nodes:
            raise AttributeError(f"The layer {self.name} has never been called and thus has no defined {label}.")
        if node_index >= len(self._inbound_nodes):
            raise ValueError(
                f"Asked to get {label} at node {node_index}, but the operation has only "
                f"{len(self._inbound_nodes)} inbound nodes."
            )
        values = getattr(self._inbound_nodes[node_index], attr)
        if isinstance(values, list) and len(values) == 1:
            return values[0]
        return values

    @property
    def input(self):
        return self._node_attr(0, "input_tensors", "input")

    @property
    def output(self):
        return self._node_attr(0, "output_tensors", "output")

    def _obj_type(self):
        return "Operation"


_SIG_CACHE = {}


def _init_signature(cls):
    sig = _SIG_CACHE.get(cls)
    if sig is None:
        params = inspect.signature(cls.__init__).parameters
        kinds = {
            inspect.Parameter.POSITIONAL_ONLY: 0, inspect.Parameter.POSITIONAL_OR_KEYWORD: 1,
            inspect.Parameter.VAR_POSITIONAL: 2, inspect.Parameter.KEYWORD_ONLY: 3,
            inspect.Parameter.VAR_KEYWORD: 4,
        }
        sig = {n: kinds[p.kind] for n, p in params.items()}
        _SIG_CACHE[cls] = sig
    return sig


def _has_extra_init_args(cls):
    sig = _init_signature(cls)
    return any(n not in ("self", "name") and k in (0, 1, 3) for n, k in sig.items())
