"""Different optimizers for different variables (``keras.optimizers.OptimizerMap`` / ``MultiOptimizer``;
behaviour of keras/src/optimizers/multi_optimizer.py:10-413).

``OptimizerMap`` resolves a variable path to an optimizer: an exact key wins, otherwise the single key that matches the
whole path as a regular expression, otherwise the default.  ``MultiOptimizer`` turns any such selector (a map or a
callable) into a routing table built once: ``route[i]`` is the slot of the inner optimizer that owns variable ``i`` of
the list the optimizer was built on, so ``apply`` is one pass that fills per-optimizer buckets by index.
"""

import re
from collections.abc import MutableMapping

from keras_b200.core.export_registry import keras_export
from keras_b200.optimizers.loss_scale_optimizer import LossScaleOptimizer
from keras_b200.optimizers.optimizers import Optimizer
from keras_b200.saving import serialization_lib


def _check_inner(optimizer, where):
    """An inner optimizer is a plain optimizer: wrappers that rescale or re-route gradients cannot nest."""
    if not isinstance(optimizer, Optimizer):
        raise ValueError(f"optimizer must be a Keras Optimizer instance. Received: {optimizer}")
    if isinstance(optimizer, LossScaleOptimizer):
        raise ValueError("optimizer cannot be LossScaleOptimizer." if where == "map" else "LossScaleOptimizer cannot be used inside an MultiOptimizer.")
    if isinstance(optimizer, MultiOptimizer):
        raise ValueError("optimizer cannot be MultiOptimizer." if where == "map" else "MultiOptimizer cannot be used inside an MultiOptimizer.")


@keras_export("keras.optimizers.OptimizerMap")
class OptimizerMap(MutableMapping):
    def __init__(self, default_optimizer, optimizer_map=None):
        if not isinstance(default_optimizer, Optimizer):
            raise TypeError(f"default_optimizer must be a Keras Optimizer instance. Received: {default_optimizer}")
        if optimizer_map is not None and not isinstance(optimizer_map, dict):
            raise TypeError(f"optimizer_map must be a dictionary. Received: {optimizer_map}")
        self._default_optimizer = default_optimizer
        self._optimizer_map = {}
        self._patterns = {}  # key -> compiled pattern, filled lazily
        for key, optimizer in (optimizer_map or {}).items():
            self._optimizer_map[key] = optimizer

    @property
    def default_optimizer(self):
        return self._default_optimizer

    def _pattern(self, key):
        compiled = self._patterns.get(key)
        if compiled is None:
            compiled = self._patterns[key] = re.compile(key)
        return compiled

    def __getitem__(self, path):
        exact = self._optimizer_map.get(path)
        if exact is not None:
            return exact
        hits = [key for key in self._optimizer_map if self._pattern(key).fullmatch(path)]
        if len(hits) > 1:
            raise ValueError(f"Multiple optimizers assigned to variable {path}.")
        return self._optimizer_map[hits[0]] if hits else self._default_optimizer

    def __setitem__(self, key, optimizer):
        if key in self._optimizer_map:
            raise ValueError(f"'{key}' already exists in the OptimizerMap with value {self._optimizer_map[key]}. "
                             "Please make sure to not use duplicated keys.")
        if not isinstance(key, str):
            raise ValueError(f"key must be a string. Received: {key}")
        _check_inner(optimizer, "map")
        self._optimizer_map[key] = optimizer

    def __delitem__(self, key):
        del self._optimizer_map[key]
        self._patterns.pop(key, None)

    def __len__(self):
        return len(self._optimizer_map)

    def __iter__(self):
        return iter(self._optimizer_map)

    def __call__(self, variable):
        return self[variable.path]

    def get_config(self):
        return {"default_optimizer": serialization_lib.serialize_keras_object(self._default_optimizer),
                "optimizer_map": serialization_lib.serialize_keras_object(self._optimizer_map)}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        load = lambda part: serialization_lib.deserialize_keras_object(part, custom_objects=custom_objects)  # noqa: E731
        return cls(load(config["default_optimizer"]), load(config["optimizer_map"]))


@keras_export("keras.optimizers.MultiOptimizer")
class MultiOptimizer(Optimizer):
    """``optimizer_map``: an ``OptimizerMap`` or any ``variable -> Optimizer`` callable."""

    def __init__(self, optimizer_map, loss_scale_factor=None, name=None):
        self._inner_optimizers = []
        super().__init__(learning_rate=0.0, loss_scale_factor=loss_scale_factor, name=name)
        self._optimizer_map = optimizer_map
        self._route = {}  # variable key -> slot in _inner_optimizers
        # optimizers that are known before any variable is seen get their slots now, in map order, the default last
        known = list(optimizer_map.values()) if hasattr(optimizer_map, "values") else []
        default = getattr(optimizer_map, "default_optimizer", None)
        if default is not None:
            known.append(default)
        for optimizer in known:
            self._slot_of(optimizer)

    def _slot_of(self, optimizer):
        for slot, existing in enumerate(self._inner_optimizers):
            if existing is optimizer:
                return slot
        optimizer.loss_scale_factor = self.loss_scale_factor
        self._inner_optimizers.append(optimizer)
        return len(self._inner_optimizers) - 1

    def _buckets(self, variables, payload=None):
        """Per-slot lists of ``variables`` (or of ``(payload[i], variables[i])`` pairs) according to the routing table."""
        buckets = [[] for _ in self._inner_optimizers]
        for i, variable in enumerate(variables):
            slot = self._route[self._var_key(variable)]
            buckets[slot].append(variable if payload is None else (payload[i], variable))
        return buckets

    def build(self, var_list):
        if self.built:
            return
        self._route = {}
        self._trainable_variables_indices = {}
        for position, variable in enumerate(var_list):
            optimizer = self._optimizer_map(variable)
            if not isinstance(optimizer, Optimizer):
                raise ValueError(f"Optimizer for variable {variable} is not an Optimizer instance.")
            _check_inner(optimizer, "build")
            key = self._var_key(variable)
            self._route[key] = self._slot_of(optimizer)
            self._trainable_variables_indices[key] = position
        for optimizer, owned in zip(self._inner_optimizers, self._buckets(var_list)):
            if owned:
                optimizer.build(owned)
        super().build(var_list)

    @property
    def optimizers(self):
        return self._inner_optimizers

    @property
    def variables(self):
        collected = list(self._variables)
        for optimizer in self._inner_optimizers:
            collected.extend(optimizer.variables)
        return collected

    @property
    def learning_rate(self):
        raise AttributeError("Learning rate cannot be accessed on a MultiOptimizer. Access the learning rate on the individual sub-optimizers instead.")

    @learning_rate.setter
    def learning_rate(self, value):
        raise AttributeError("Learning rate cannot be set on a MultiOptimizer. Set the learning rate on the individual sub-optimizers instead.")

    @property
    def loss_scale_factor(self):
        return getattr(self, "_loss_scale_factor", None)

    @loss_scale_factor.setter
    def loss_scale_factor(self, value):
        self._loss_scale_factor = value
        for optimizer in getattr(self, "_inner_optimizers", ()):
            optimizer.loss_scale_factor = value

    def apply(self, grads, trainable_variables=None):
        if len(grads) == 0:
            return
        if trainable_variables is None:
            if not self.built:
                raise ValueError("When passing `grads` without `variables`, the optimizer must already be built on a list of variables. "
                                 "Call `optimizer.build(trainable_variables)` first.")
            trainable_variables = self._trainable_variables
        if not self.built:
            self.build(trainable_variables)
            self.built = True
        if len(grads) != len(self._route):
            raise ValueError(f"Gradients must match trainable variables one-to-one. Received {len(grads)} gradients and {len(self._route)} variables.")
        for optimizer, pairs in zip(self._inner_optimizers, self._buckets(trainable_variables, payload=grads)):
            if pairs:
                optimizer.apply([g for g, _ in pairs], [v for _, v in pairs])
        self._iterations.assign_add(1)

    def finalize_variable_values(self, var_list):
        for optimizer, owned in zip(self._inner_optimizers, self._buckets(var_list)):
            if owned:
                optimizer.finalize_variable_values(owned)

    def set_weights(self, weights):
        if not self.built:
            raise ValueError("You are calling `set_weights()` on an optimizer that has not yet been built. Please call "
                             "`optimizer.build(trainable_variables)` to create the optimizer weights before calling `set_weights()`.")
        # layout of `weights`: this optimizer's own variables, then each inner optimizer's block in slot order
        cursor = 0
        for variable in self._variables:
            variable.assign(weights[cursor])
            cursor += 1
        for optimizer in self._inner_optimizers:
            count = len(optimizer.variables)
            if count:
                optimizer.set_weights(weights[cursor:cursor + count])
                cursor += count

    def get_config(self):
        return {"optimizer_map": serialization_lib.serialize_keras_object(self._optimizer_map), "loss_scale_factor": self.loss_scale_factor,
                "name": self.name}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        config = dict(config)
        config["optimizer_map"] = serialization_lib.deserialize_keras_object(config["optimizer_map"], custom_objects=custom_objects)
        return cls(**config)
