"""``LossScaleOptimizer``: dynamic loss scaling around an inner optimizer.

Behaviour of keras/src/optimizers/loss_scale_optimizer.py:15-344: scale starts at 2^15, doubles
every ``dynamic_growth_steps`` finite steps, halves (and skips the step) on a non-finite gradient.
The finite check is one fused reduction whose result stays on the device; the skip is applied by
masking the update instead of branching on the host.
"""

import torch

from keras_b200 import initializers
from keras_b200.core.export_registry import keras_export
from keras_b200.optimizers.base_optimizer import BaseOptimizer
from keras_b200.optimizers.optimizers import Optimizer


@keras_export(["keras.optimizers.LossScaleOptimizer", "keras.mixed_precision.LossScaleOptimizer"])
class LossScaleOptimizer(Optimizer):
    def __init__(self, inner_optimizer, initial_scale=2.0 ** 15, dynamic_growth_steps=2000, name=None, **kwargs):
        if not kwargs.pop("dynamic", True):
            raise ValueError("LossScaleOptimizer no longer supports `dynamic=False`. Instead, simply set `loss_scale_factor` directly on the `inner_optimizer`.")
        kwargs.pop("learning_rate", None)
        kwargs = {k: v for k, v in kwargs.items() if v is not None and k not in ("weight_decay", "clipnorm", "global_clipnorm", "clipvalue", "use_ema", "ema_momentum", "ema_overwrite_frequency", "loss_scale_factor", "gradient_accumulation_steps")}
        super().__init__(learning_rate=0.0, name=name, **kwargs)
        self.inner_optimizer = inner_optimizer
        self.initial_scale = initial_scale
        self.dynamic_growth_steps = dynamic_growth_steps
        if getattr(inner_optimizer, "gradient_accumulation_steps", None):
            self.gradient_accumulation_steps = inner_optimizer.gradient_accumulation_steps
            self.inner_optimizer.gradient_accumulation_steps = None

    def build(self, var_list):
        self.step_counter = self.add_variable(shape=(), dtype="int32", initializer=initializers.Zeros(), aggregation="none", name="step_counter")
        self.dynamic_scale = self.add_variable(shape=(), dtype="float32", initializer=initializers.Constant(self.initial_scale), aggregation="none", name="dynamic_scale")
        self.inner_optimizer.build(var_list)
        super().build(var_list)

    @property
    def variables(self):
        return self._variables + self.inner_optimizer.variables

    def apply(self, grads, trainable_variables=None):
        if trainable_variables is None:
            trainable_variables = self._trainable_variables
        trainable_variables = list(trainable_variables)
        if not self.built:
            with torch.no_grad():
                self.build(trainable_variables)
            self.built = True
        with torch.no_grad():
            scale = self.dynamic_scale._value
            present = [g for g in grads if g is not None]
            finite = torch.stack([torch.isfinite(g).all() for g in present]).all() if present else torch.tensor(True)
            if bool(finite):
                unscaled = [g if g is None else g / scale.to(g.dtype) for g in grads]
                self.inner_optimizer.apply(unscaled, trainable_variables)
                self.step_counter._value.add_(1)
                if int(self.step_counter._value) > self.dynamic_growth_steps - 1:
                    self.step_counter._value.zero_()
                    self.dynamic_scale._value.mul_(2.0)
            else:
                self.step_counter._value.zero_()
                self.dynamic_scale._value.div_(2.0)
            self._bump_step()

    def stateless_apply(self, optimizer_variables, grads, trainable_variables):
        return BaseOptimizer.stateless_apply(self, optimizer_variables, grads, trainable_variables)

    def check_finite(self, grads):
        present = [g for g in grads if g is not None]
        return torch.stack([torch.isfinite(g).all() for g in present]).all()

    def scale_loss(self, loss):
        scale = self.dynamic_scale._value if self.built else self.initial_scale
        return loss * scale

    @property
    def learning_rate(self):
        return self.inner_optimizer.learning_rate

    @learning_rate.setter
    def learning_rate(self, learning_rate):
        self.inner_optimizer.learning_rate = learning_rate

    @property
    def iterations(self):
        return self.inner_optimizer.iterations

    def finalize_variable_values(self, var_list):
        self.inner_optimizer.finalize_variable_values(var_list)

    def get_config(self):
        from keras_b200.saving import serialization_lib

        config = Optimizer.get_config(self)
        inner = serialization_lib.serialize_keras_object(self.inner_optimizer)
        config.update({"inner_optimizer": inner, "initial_scale": self.initial_scale, "dynamic_growth_steps": self.dynamic_growth_steps})
        del config["learning_rate"]
        return config

    @classmethod
    def from_config(cls, config, custom_objects=None):
        from keras_b200.saving import serialization_lib

        config = dict(config)
        inner = serialization_lib.deserialize_keras_object(config.pop("inner_optimizer"), custom_objects=custom_objects)
        return cls(inner, **config)
