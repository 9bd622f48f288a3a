"""``OptimizerMap`` / ``MultiOptimizer``: different optimizers for different variables, chosen by regex on the
variable path (keras/src/optimizers/multi_optimizer.py:10-413)."""

import re
from collections.abc import MutableMapping

from keras_b200.core.export_registry import keras_export
from keras_b200.optimizers.loss_scale_optimizer import LossScaleOptimizer
from keras_b200.optimizers.optimizers import Optimizer
from keras_b200.saving import serialization_lib


@keras_export("keras.optimizers.OptimizerMap")
class OptimizerMap(MutableMapping):
    def __init__(self, default_optimizer, optimizer_map=None):
        if not isinstance(default_optimizer, Optimizer):
            raise TypeError(f"default_optimizer must be a Keras Optimizer instance. Received: {default_optimizer}")
        if optimizer_map is not None and not isinstance(optimizer_map, dict):
            raise TypeError(f"optimizer_map must be a dictionary. Received: {optimizer_map}")
        self._default_optimizer = default_optimizer
        self._optimizer_map = optimizer_map or dict()

    default_optimizer = property(lambda self: self._default_optimizer)

    def __getitem__(self, key):
        if key in self._optimizer_map:
            return self._optimizer_map[key]
        matching = [p for p in self._optimizer_map.keys() if re.fullmatch(p, key)]
        if len(matching) > 1:
            raise ValueError(f"Multiple optimizers assigned to variable {key}.")
        if len(matching) == 1:
            return self._optimizer_map[matching[0]]
        return self.default_optimizer

    def __setitem__(self, key, optimizer):
        if key in self._optimizer_map:
            raise ValueError(f"'{key}' already exists in the OptimizerMap with value {self._optimizer_map[key]}. Please make sure to not use duplicated keys.")
        if not isinstance(key, str):
            raise ValueError(f"key must be a string. Received: {key}")
        if not isinstance(optimizer, Optimizer):
            raise ValueError(f"optimizer must be a Keras Optimizer instance. Received: {optimizer}")
        if isinstance(optimizer, LossScaleOptimizer):
            raise ValueError("optimizer cannot be LossScaleOptimizer.")
        if isinstance(optimizer, MultiOptimizer):
            raise ValueError("optimizer cannot be MultiOptimizer.")
        self._optimizer_map[key] = optimizer

    def __delitem__(self, key):
        del self._optimizer_map[key]

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
        return cls(serialization_lib.deserialize_keras_object(config["default_optimizer"], custom_objects=custom_objects),
                   serialization_lib.deserialize_keras_object(config["optimizer_map"], custom_objects=custom_objects))


@keras_export("keras.optimizers.MultiOptimizer")
class MultiOptimizer(Optimizer):
    def __init__(self, optimizer_map, loss_scale_factor=None, name=None):
        self._inner_optimizers = []
        super().__init__(learning_rate=0.0, loss_scale_factor=loss_scale_factor, name=name)
        self._optimizer_map = optimizer_map
        if hasattr(optimizer_map, "values"):
            for opt in optimizer_map.values():
                if opt not in self._inner_optimizers:
                    opt.loss_scale_factor = loss_scale_factor
                    self._inner_optimizers.append(opt)
        default_opt = getattr(optimizer_map, "default_optimizer", None)
        if default_opt is not None and default_opt not in self._inner_optimizers:
            default_opt.loss_scale_factor = loss_scale_factor
            self._inner_optimizers.append(default_opt)

    def build(self, var_list):
        if self.built:
            return
        self._var_to_optimizer_idx = {}
        self._trainable_variables_indices = {}
        per_opt = [[] for _ in self._inner_optimizers]
        for i, var in enumerate(var_list):
            opt = self._optimizer_map(var)
            if not isinstance(opt, Optimizer):
                raise ValueError(f"Optimizer for variable {var} is not an Optimizer instance.")
            if isinstance(opt, LossScaleOptimizer):
                raise ValueError("LossScaleOptimizer cannot be used inside an MultiOptimizer.")
            if isinstance(opt, MultiOptimizer):
                raise ValueError("MultiOptimizer cannot be used inside an MultiOptimizer.")
            if opt not in self._inner_optimizers:
                opt.loss_scale_factor = self.loss_scale_factor
                self._inner_optimizers.append(opt)
                per_opt.append([])
            idx = self._inner_optimizers.index(opt)
            self._var_to_optimizer_idx[self._var_key(var)] = idx
            self._trainable_variables_indices[self._var_key(var)] = i
            per_opt[idx].append(var)
        for opt, variables in zip(self._inner_optimizers, per_opt):
            if variables:
                opt.build(variables)
        super().build(var_list)

    optimizers = property(lambda self: self._inner_optimizers)

    @property
    def variables(self):
        out = self._variables[:]
        for opt in self._inner_optimizers:
            out.extend(opt.variables)
        return out

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
        for opt in getattr(self, "_inner_optimizers", []):
            opt.loss_scale_factor = value

    def apply(self, grads, trainable_variables=None):
        if len(grads) == 0:
            return
        if trainable_variables is None:
            if not self.built:
                raise ValueError("When passing `grads` without `variables`, the optimizer must already be built on a list of variables. Call `optimizer.build(trainable_variables)` first.")
            trainable_variables = self._trainable_variables
        if not self.built:
            self.build(trainable_variables)
            self.built = True
        if len(grads) != len(self._trainable_variables_indices):
            raise ValueError(f"Gradients must match trainable variables one-to-one. Received {len(grads)} gradients and {len(self._trainable_variables_indices)} variables.")
        per_opt = [[] for _ in self._inner_optimizers]
        for g, v in zip(grads, trainable_variables):
            per_opt[self._var_to_optimizer_idx[self._var_key(v)]].append((g, v))
        for opt, gv in zip(self._inner_optimizers, per_opt):
            if gv:
                sub_grads, sub_vars = zip(*gv)
                opt.apply(list(sub_grads), list(sub_vars))
        self._iterations.assign_add(1)

    def finalize_variable_values(self, var_list):
        per_opt = [[] for _ in self._inner_optimizers]
        for var in var_list:
            per_opt[self._var_to_optimizer_idx[self._var_key(var)]].append(var)
        for opt, variables in zip(self._inner_optimizers, per_opt):
            if variables:
                opt.finalize_variable_values(variables)

    def set_weights(self, weights):
        if not self.built:
            raise ValueError("You are calling `set_weights()` on an optimizer that has not yet been built. Please call `optimizer.build(trainable_variables)` to create the optimizer weights before calling `set_weights()`.")
        own = len(self._variables)
        for i in range(own):
            self._variables[i].assign(weights[i])
        idx = own
        for opt in self._inner_optimizers:
            n = len(opt.variables)
            if n > 0:
                opt.set_weights(weights[idx: idx + n])
                idx += n

    def get_config(self):
        return {"optimizer_map": serialization_lib.serialize_keras_object(self._optimizer_map), "loss_scale_factor": self.loss_scale_factor, "name": self.name}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        config = config.copy()
        config["optimizer_map"] = serialization_lib.deserialize_keras_object(config["optimizer_map"], custom_objects=custom_objects)
        return cls(**config)
