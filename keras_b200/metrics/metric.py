"""``Metric`` base class: state in ``Variable``s, ``update_state`` / ``result`` / ``reset_state``.

Behaviour of keras/src/metrics/metric.py:12-253 including the stateless API.
"""

import torch

from keras_b200 import initializers
from keras_b200.core import config
from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.naming import auto_name
from keras_b200.core.scopes import StatelessScope, name_scope
from keras_b200.core.variables import Variable
from keras_b200.ops.operation import KerasSaveable


@keras_export(["keras.Metric", "keras.metrics.Metric"])
class Metric(KerasSaveable):
    def __init__(self, dtype=None, name=None):
        self.name = name or auto_name(self.__class__.__name__)
        from keras_b200 import dtype_policies

        self._dtype_policy = dtype_policies.get(dtype or config.floatx())
        self._dtype = self._dtype_policy.compute_dtype
        self._metrics = []
        self._variables = []

    def reset_state(self):
        for v in self.variables:
            v.assign(torch.zeros(tuple(v.shape), dtype=v._torch_dtype, device=v._value.device))

    def update_state(self, *args, **kwargs):
        raise NotImplementedError

    def stateless_update_state(self, metric_variables, *args, **kwargs):
        if len(metric_variables) != len(self.variables):
            raise ValueError(
                "Argument `metric_variables` must be a list of tensors corresponding 1:1 to "
                f"{self.__class__.__name__}().variables. Received list with length {len(metric_variables)}, "
                f"but expected {len(self.variables)} variables."
            )
        mapping = list(zip(self.variables, metric_variables))
        with StatelessScope(state_mapping=mapping) as scope:
            self.update_state(*args, **kwargs)
        out = []
        for v in self.variables:
            nv = scope.get_current_value(v)
            out.append(nv if nv is not None else v.value)
        return out

    def result(self):
        raise NotImplementedError

    def stateless_result(self, metric_variables):
        if len(metric_variables) != len(self.variables):
            raise ValueError(
                "Argument `metric_variables` must be a list of tensors corresponding 1:1 to "
                f"{self.__class__.__name__}().variables. Received list with length {len(metric_variables)}, "
                f"but expected {len(self.variables)} variables."
            )
        with StatelessScope(state_mapping=list(zip(self.variables, metric_variables))):
            return self.result()

    def stateless_reset_state(self):
        with StatelessScope() as scope:
            self.reset_state()
        out = []
        for v in self.variables:
            nv = scope.get_current_value(v)
            out.append(nv if nv is not None else v.value)
        return out

    @property
    def dtype(self):
        return self._dtype

    def add_variable(self, shape, initializer, dtype=None, aggregation="sum", name=None):
        self._check_super_called()
        with name_scope(self.name.replace("/", ">"), caller=self):
            initializer = initializers.get(initializer)
            v = Variable(initializer=initializer, shape=shape, dtype=dtype or self.dtype, trainable=False, aggregation=aggregation, synchronization="on_read", name=name)
        self._variables.append(v)
        return v

    def add_weight(self, shape=(), initializer=None, dtype=None, name=None):
        return self.add_variable(shape=shape, initializer=initializer, dtype=dtype, name=name)

    @property
    def variables(self):
        out = list(self._variables)
        for m in self._metrics:
            out.extend(m.variables)
        return out

    def __call__(self, *args, **kwargs):
        self._check_super_called()
        self.update_state(*args, **kwargs)
        return self.result()

    def get_config(self):
        return {"name": self.name, "dtype": self.dtype}

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def __setattr__(self, name, value):
        if hasattr(self, "_metrics"):
            if isinstance(value, Metric):
                if not any(value is m for m in self._metrics):
                    self._metrics.append(value)
            elif isinstance(value, Variable) and "_variables" in self.__dict__:
                if not any(value is v for v in self._variables):
                    self._variables.append(value)
            elif isinstance(value, (list, tuple)) and name != "_metrics" and name != "_variables":
                for v in value:
                    if isinstance(v, Metric) and not any(v is m for m in self._metrics):
                        self._metrics.append(v)
        object.__setattr__(self, name, value)

    def _check_super_called(self):
        if not hasattr(self, "_variables"):
            raise RuntimeError("You forgot to call `super().__init__()` in the `__init__()` method. Go add it!")

    def __repr__(self):
        return f"<{self.__class__.__name__} name={self.name}>"

    def __str__(self):
        return self.__repr__()

    def _obj_type(self):
        return "Metric"
