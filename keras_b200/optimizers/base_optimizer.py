"""Optimizer base class.

Behaviour of keras/src/optimizers/base_optimizer.py:14-1197: ``apply`` = filter ``None`` grads →
overwrite-with-gradient variables → unscale by ``loss_scale_factor`` → clip → weight decay →
update step → constraints → ``iterations += 1``; gradient accumulation, EMA, stateless apply,
slot naming ``"{path with / → _}_{slot}"``, index-keyed persistence.

Design differences: the step counter is mirrored on the host (validated through the tensor
version counter) so Adam-style bias corrections never force a device→host sync; the update of
all variables is one call (``_update_all``) so that subclasses can hand the whole list to a fused
multi-tensor sm_100a kernel.
"""

import re
import warnings

import torch

from keras_b200 import initializers, tree
from keras_b200.core import global_state
from keras_b200.core.dtypes import standardize_dtype, to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.naming import auto_name
from keras_b200.core.scopes import StatelessScope, in_stateless_scope, name_scope
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.core.variables import Variable
from keras_b200.ops.operation import KerasSaveable
from keras_b200.optimizers.schedules import learning_rate_schedule


class BaseOptimizer(KerasSaveable):
    def __init__(self, learning_rate, weight_decay=None, clipnorm=None, clipvalue=None, global_clipnorm=None, use_ema=False,
                 ema_momentum=0.99, ema_overwrite_frequency=None, loss_scale_factor=None, gradient_accumulation_steps=None, name=None, **kwargs):
        self._lock = False
        if kwargs.pop("decay", None) is not None:
            warnings.warn("Argument `decay` is no longer supported and will be ignored.")
        if kwargs:
            raise ValueError(f"Argument(s) not recognized: {kwargs}")
        if name is None:
            name = auto_name(self.__class__.__name__)
        self.name = name
        self.weight_decay = weight_decay
        self.clipnorm = clipnorm
        self.global_clipnorm = global_clipnorm
        self.clipvalue = clipvalue
        self.use_ema = use_ema
        self.loss_scale_factor = loss_scale_factor
        self.gradient_accumulation_steps = gradient_accumulation_steps
        if gradient_accumulation_steps:
            if not gradient_accumulation_steps >= 2:
                raise ValueError(f"`gradient_accumulation_steps` must be an integer >= 2. Received: gradient_accumulation_steps={gradient_accumulation_steps}")
        if use_ema:
            if ema_momentum > 1 or ema_momentum < 0:
                raise ValueError(f"`ema_momentum` must be in the range [0, 1]. Received: ema_momentum={ema_momentum}")
            if ema_overwrite_frequency and (not isinstance(ema_overwrite_frequency, int) or ema_overwrite_frequency < 1):
                raise ValueError(f"`ema_overwrite_frequency` must be an integer >= 1 or None. Received: ema_overwrite_frequency={ema_overwrite_frequency}")
        self.ema_momentum = ema_momentum
        self.ema_overwrite_frequency = ema_overwrite_frequency
        clip_args = sum(a is not None for a in (clipnorm, clipvalue, global_clipnorm))
        if clip_args > 1:
            raise ValueError(f"Only one of `clipnorm`, `clipvalue` and `global_clipnorm` can be set. Received: clipnorm={clipnorm}, clipvalue={clipvalue}, global_clipnorm={global_clipnorm}")
        self.built = False
        self._variables = []
        self._trainable_variables = []
        self._trainable_variables_indices = {}
        self._exclude_from_weight_decay_names = []
        self._exclude_from_weight_decay = []
        self._exclude_ids = set()
        with name_scope(self.name, caller=self):
            iterations = Variable(0, name="iteration", dtype="int32", trainable=False, aggregation="only_first_replica")
        self._track_variable(iterations)
        self._iterations = iterations
        self._host_step = 0
        self._host_step_version = iterations._value._version
        if isinstance(learning_rate, learning_rate_schedule.LearningRateSchedule):
            self._learning_rate = learning_rate
        elif callable(learning_rate):
            self._learning_rate = learning_rate
        else:
            if not isinstance(learning_rate, float):
                raise ValueError(f"Argument `learning_rate` should be float, or an instance of LearningRateSchedule, or a callable (that takes in the current iteration value and returns the corresponding learning rate value). Received instead: learning_rate={learning_rate}")
            with name_scope(self.name, caller=self):
                lr = Variable(learning_rate, name="learning_rate", dtype="float32", trainable=False, aggregation="only_first_replica")
            self._track_variable(lr)
            self._learning_rate = lr
            self._host_lr = float(learning_rate)
            self._host_lr_version = lr._value._version

    # -- host mirrors of scalar state ------------------------------------------------------
    def _step(self):
        """Current value of ``iterations`` as a Python int, without a device sync on the hot path."""
        v = self._iterations._value._version
        if v != self._host_step_version:
            self._host_step = int(self._iterations._value)
            self._host_step_version = v
        return self._host_step

    def _local_step(self):
        """Number of completed *updates*: the value of the public ``iterations`` (the raw call counter divided by
        ``gradient_accumulation_steps``), which is what bias corrections and schedules count in
        (keras/src/optimizers/base_optimizer.py ``iterations``)."""
        step = self._step()
        if self.gradient_accumulation_steps:
            return step // self.gradient_accumulation_steps
        return step

    def _bump_step(self):
        with torch.no_grad():
            self._iterations._value.add_(1)
        if self._iterations._value._version == self._host_step_version + 1:
            self._host_step += 1
            self._host_step_version += 1

    def _note_replayed_step(self):
        """A captured replay of the update advanced ``iterations`` on the device (no Python-visible write): advance the
        host mirror with it."""
        self._step()
        self._host_step += 1

    def _lr_float(self):
        """Learning rate as a Python float when it is a plain variable (else ``None``)."""
        lr = self._learning_rate
        if isinstance(lr, Variable):
            v = lr._value._version
            if v != self._host_lr_version:
                self._host_lr = float(lr._value)
                self._host_lr_version = v
            return self._host_lr
        return None

    @property
    def iterations(self):
        if self.gradient_accumulation_steps:
            return self._iterations.value // self.gradient_accumulation_steps if not isinstance(self._iterations, int) else self._iterations
        return self._iterations

    def _track_variable(self, variable):
        self._variables.append(variable)

    def _overwrite_variable_with_gradient(self, variable):
        return getattr(variable, "overwrite_with_gradient", False)

    def build(self, variables):
        if self.use_ema:
            self._model_variables_moving_average = self.add_optimizer_variables(variables, "average")
        if self.gradient_accumulation_steps:
            self._accumulated_gradients = []
        for i, variable in enumerate(variables):
            self._trainable_variables_indices[id(variable)] = i
            if self.gradient_accumulation_steps:
                self._accumulated_gradients.append(self.add_variable_from_reference(variable, name="gradient_accumulator"))
        self._trainable_variables = list(variables)
        self._exclude_ids = {id(v) for v in self._exclude_from_weight_decay}
        self.built = True

    def _var_key(self, variable):
        return id(variable)

    @property
    def variables(self):
        return self._variables[:]

    def _get_variable_index(self, variable):
        return self._trainable_variables_indices[id(variable)]

    def add_variable(self, shape, initializer="zeros", dtype=None, aggregation="none", layout=None, name=None):
        self._check_super_called()
        initializer = initializers.get(initializer)
        with name_scope(self.name, caller=self):
            variable = Variable(initializer=initializer, shape=shape, dtype=dtype, trainable=False, aggregation=aggregation, layout=layout, name=name)
        self._track_variable(variable)
        return variable

    def add_variable_from_reference(self, reference_variable, name=None, initializer="zeros"):
        name = name or "var"
        if hasattr(reference_variable, "path"):
            name = f"{reference_variable.path.replace('/', '_')}_{name}"
        else:
            name = f"{str(reference_variable.name).replace('/', '_').replace(':', '_')}_{name}"
        var = self.add_variable(shape=reference_variable.shape, initializer=initializer, dtype=reference_variable.dtype, name=name,
                                layout=getattr(reference_variable, "_layout", None))
        var._global_shape = getattr(reference_variable, "_global_shape", None)
        var._shard_spec = getattr(reference_variable, "_shard_spec", None)
        return var

    def add_optimizer_variables(self, trainable_variables, name, initializer="zeros"):
        name_list = name
        initializer_list = initializer
        if isinstance(name, str):
            name_list = [name]
            initializer_list = [initializer]
        else:
            if isinstance(initializer, str) or not isinstance(initializer, (list, tuple)):
                initializer_list = [initializer] * len(name_list)
        optimizer_variables = tuple([] for _ in name_list)
        for variable in trainable_variables:
            if self._overwrite_variable_with_gradient(variable):
                for ov in optimizer_variables:
                    ov.append(None)
            else:
                for nm, init, ov in zip(name_list, initializer_list, optimizer_variables):
                    ov.append(self.add_variable_from_reference(variable, name=nm, initializer=init))
        if isinstance(name, str):
            return optimizer_variables[0]
        return optimizer_variables

    def _check_variables_are_known(self, variables):
        for v in variables:
            if id(v) not in self._trainable_variables_indices:
                raise ValueError(f"Unknown variable: {v}. This optimizer can only be called for the variables it was originally built with. When working with a new set of variables, you should recreate a new optimizer instance.")

    def assign(self, variable, value):
        variable.assign(value)

    def assign_add(self, variable, value):
        variable.assign_add(value)

    def assign_sub(self, variable, value):
        variable.assign_sub(value)

    def update_step(self, gradient, variable, learning_rate):
        raise NotImplementedError

    def apply_gradients(self, grads_and_vars):
        grads, trainable_variables = zip(*grads_and_vars)
        self.apply(grads, trainable_variables)
        return self._iterations

    def apply(self, grads, trainable_variables=None):
        if len(grads) == 0:
            return
        self._step_scalars_on_device = False  # set by a fused update that read its step scalars from device memory
        if trainable_variables is None:
            if not self.built:
                raise ValueError("When passing `grads` without `variables`, the optimizer must already be built on a list of variables. Call `optimizer.build(trainable_variables)` first. ")
            if len(grads) != len(self._trainable_variables_indices):
                raise ValueError(f"When passing `grads` as a list of gradient tensors, the gradients must match `optimizer.variables` one-to-on. Received a list of {len(grads)} gradients, but the optimizer is tracking {len(self._trainable_variables)} trainable variables.")
            trainable_variables = self._trainable_variables
        else:
            trainable_variables = list(trainable_variables)
            if not self.built:
                with torch.no_grad():
                    self.build(trainable_variables)
                self.built = True
            self._check_variables_are_known(trainable_variables)
        with torch.no_grad():
            grads_and_vars = list(zip(grads, trainable_variables))
            filtered = [(g, v) for g, v in grads_and_vars if g is not None]
            if not filtered:
                raise ValueError("No gradients provided for any variable.")
            if len(filtered) < len(grads_and_vars):
                missing = [v.path for g, v in grads_and_vars if g is None]
                if not getattr(self, "_warned_missing", False):
                    warnings.warn(f"Gradients do not exist for variables {missing} when minimizing the loss. If using `model.compile()`, did you forget to provide a `loss` argument?")
                    self._warned_missing = True
            grads, trainable_variables = [g for g, _ in filtered], [v for _, v in filtered]
            grads, trainable_variables = self._overwrite_variables_directly_with_gradients(grads, trainable_variables)
            if len(trainable_variables) > 0:
                self._backend_apply_gradients(grads, trainable_variables)
                for variable in trainable_variables:
                    if variable.constraint is not None:
                        variable.assign(variable.constraint(variable._value))
            self._bump_step()

    def _scaled_clipped(self, grads):
        """Unscale by ``loss_scale_factor`` and clip (returns new tensors unless nothing to do)."""
        scale = self.loss_scale_factor
        if scale is not None:
            grads = [g / scale for g in grads]
        return self._clip_gradients(grads)

    def _backend_apply_gradients(self, grads, trainable_variables):
        if self.gradient_accumulation_steps:
            steps = self.gradient_accumulation_steps
            is_update_step = (self._step() + 1) % steps == 0
            acc = [self._accumulated_gradients[self._get_variable_index(v)] for v in trainable_variables]
            if is_update_step:
                grads = [(g + a._value) / steps for g, a in zip(grads, acc)]
                grads = self._scaled_clipped(grads)
                self._apply_weight_decay(trainable_variables)
                self._backend_update_step(grads, trainable_variables, self.learning_rate)
                for a in acc:
                    a._value.zero_()
            else:
                for g, a in zip(grads, acc):
                    a._value.add_(g)
        else:
            fused = self._fused_apply(grads, trainable_variables)
            if not fused:
                grads = self._scaled_clipped(grads)
                self._apply_weight_decay(trainable_variables)
                self._backend_update_step(grads, trainable_variables, self.learning_rate)
        if self.use_ema:
            self._update_model_variables_moving_average(self._trainable_variables)
            if self.ema_overwrite_frequency:
                if (self._local_step() + 1) % self.ema_overwrite_frequency == 0:
                    self._overwrite_model_variables_with_average_value(self._trainable_variables)

    def _fused_apply(self, grads, trainable_variables):
        """Hook: run unscale + clip + decay + update in fused kernels. Return True when done."""
        return False

    def _backend_update_step(self, grads, trainable_variables, learning_rate):
        for grad, var in zip(grads, trainable_variables):
            self.update_step(grad, var, learning_rate)

    def _backend_reset_gradient_accumulators(self):
        for g_acc in self._accumulated_gradients:
            g_acc._value.zero_()

    def _backend_increment_gradient_accumulators(self, grads, acc_grads):
        for g, a in zip(grads, acc_grads):
            a._value.add_(g)

    def stateless_apply(self, optimizer_variables, grads, trainable_variables):
        self._check_super_called()
        if not self.built:
            raise ValueError(f"To call `stateless_apply`, {self.__class__.__name__} must be built (i.e. its variables must have been created). You can build it via `optimizer.build(trainable_variables)`.")
        if len(optimizer_variables) != len(self.variables):
            raise ValueError(f"Argument `optimizer_variables` must be a list of tensors corresponding 1:1 to {self.__class__.__name__}().variables. Received list with length {len(optimizer_variables)}, but expected {len(self.variables)} variables.")
        if len(trainable_variables) != len(self._trainable_variables):
            raise ValueError(f"Argument `optimizer_variables` must be a list of tensors corresponding 1:1 to the trainable variables list that the optimizer was built with. Received len(trainable_variables) == {len(trainable_variables)} whereas the optimizer was built with {len(self._trainable_variables)} variables.")
        # Functional form: run the update on clones so that the live state is untouched.
        saved_opt = [v._value.detach().clone() for v in self.variables]
        saved_tr = [v._value.detach().clone() for v in self._trainable_variables]
        saved_step = (self._host_step, self._host_step_version)
        try:
            with torch.no_grad():
                for v, val in zip(self.variables, optimizer_variables):
                    v._value.copy_(convert_to_tensor(val, dtype=v._torch_dtype))
                for v, val in zip(self._trainable_variables, trainable_variables):
                    v._value.copy_(convert_to_tensor(val, dtype=v._torch_dtype))
            self.apply(grads)
            new_tr = [v._value.detach().clone() for v in self._trainable_variables]
            new_opt = [v._value.detach().clone() for v in self.variables]
        finally:
            with torch.no_grad():
                for v, val in zip(self.variables, saved_opt):
                    v._value.copy_(val)
                for v, val in zip(self._trainable_variables, saved_tr):
                    v._value.copy_(val)
            self._host_step_version = -1
        return new_tr, new_opt

    def scale_loss(self, loss):
        if self.loss_scale_factor is not None:
            return loss * self.loss_scale_factor
        return loss

    @property
    def learning_rate(self):
        return self._get_current_learning_rate()

    @learning_rate.setter
    def learning_rate(self, learning_rate):
        if isinstance(self._learning_rate, learning_rate_schedule.LearningRateSchedule):
            prev = True
        else:
            prev = False
        if isinstance(learning_rate, learning_rate_schedule.LearningRateSchedule):
            self._learning_rate = learning_rate
        elif callable(learning_rate):
            self._learning_rate = learning_rate
        else:
            if prev or not isinstance(self._learning_rate, Variable):
                raise TypeError("This optimizer was created with a `LearningRateSchedule` object as its `learning_rate` constructor argument, hence its learning rate is not settable. If you need the learning rate to be settable, you should instantiate the optimizer with a float `learning_rate` argument.")
            self._learning_rate.assign(learning_rate)

    def set_weights(self, weights):
        if not self.built:
            raise ValueError("You are calling `set_weights()` on an optimizer that has not yet been built. Please call `optimizer.build(trainable_variables)` to create the optimizer weights before calling `set_weights()`.")
        for variable, weight in zip(self._variables, weights):
            if tuple(variable.shape) != tuple(weight.shape):
                raise ValueError(f"Optimizer variable {self._var_key(variable)} has shape {str(variable.shape)} not compatible with provided weight shape {str(weight.shape)}.")
            variable.assign(weight)

    def save_own_variables(self, store):
        for i, variable in enumerate(self.variables):
            store[str(i)] = variable.numpy()

    def load_own_variables(self, store):
        if len(store.keys()) != len(self.variables):
            msg = (f"Skipping variable loading for optimizer '{self.name}', because it has {len(self.variables)} variables whereas the saved optimizer has {len(store.keys())} variables. ")
            if len(self.variables) == 0:
                msg += "This is likely because the optimizer has not been called/built yet."
            warnings.warn(msg, stacklevel=2)
            return
        for i, variable in enumerate(self.variables):
            variable.assign(store[str(i)])

    def _get_current_learning_rate(self):
        if isinstance(self._learning_rate, learning_rate_schedule.LearningRateSchedule):
            return self._learning_rate(self._iterations.value)
        if isinstance(self._learning_rate, Variable):
            return self._learning_rate.value
        if callable(self._learning_rate):
            return self._learning_rate()
        return self._learning_rate

    def _overwrite_variables_directly_with_gradients(self, grads, vars):
        if not any(self._overwrite_variable_with_gradient(v) for v in vars):
            return grads, vars
        filtered_grads, filtered_vars = [], []
        for g, v in zip(grads, vars):
            if self._overwrite_variable_with_gradient(v):
                if self.gradient_accumulation_steps:
                    steps = self.gradient_accumulation_steps
                    is_update_step = (self._step() + 1) % steps == 0
                    acc = self._accumulated_gradients[self._get_variable_index(v)]
                    new_acc = torch.maximum(g, acc._value)
                    if is_update_step:
                        v._value.copy_(new_acc)
                        acc._value.zero_()
                    else:
                        acc._value.copy_(new_acc)
                else:
                    v._value.copy_(g.to(v._value.dtype))
            else:
                filtered_grads.append(g)
                filtered_vars.append(v)
        return filtered_grads, filtered_vars

    def _filter_empty_gradients(self, grads, vars):
        pairs = [(g, v) for g, v in zip(grads, vars) if g is not None]
        if not pairs:
            raise ValueError("No gradients provided for any variable.")
        return [g for g, _ in pairs], [v for _, v in pairs]

    def _clip_gradients(self, grads):
        if self.clipnorm and self.clipnorm > 0:
            return [self._clip_by_norm(g) for g in grads]
        if self.global_clipnorm and self.global_clipnorm > 0:
            return clip_by_global_norm(grads, self.global_clipnorm)
        if self.clipvalue and self.clipvalue > 0:
            v = self.clipvalue
            return [torch.clip(g, -v, v) for g in grads]
        return grads

    def exclude_from_weight_decay(self, var_list=None, var_names=None):
        if hasattr(self, "_built") and self._built or self.built:
            raise ValueError("`exclude_from_weight_decay()` can only be configured before the optimizer is built.")
        if var_list:
            self._exclude_from_weight_decay = list(var_list)
        else:
            self._exclude_from_weight_decay = []
        self._exclude_from_weight_decay_names = var_names or []

    def _use_weight_decay(self, variable):
        if id(variable) in self._exclude_ids or any(variable is v for v in self._exclude_from_weight_decay):
            return False
        for name in self._exclude_from_weight_decay_names:
            if re.search(name, variable.path) is not None:
                return False
        return True

    def _apply_weight_decay(self, variables):
        if self.weight_decay is None:
            return
        lr = self._lr_float()
        targets = [v._value for v in variables if self._use_weight_decay(v)]
        if not targets:
            return
        if lr is not None:
            torch._foreach_mul_(targets, 1.0 - self.weight_decay * lr)
        else:
            lr_t = convert_to_tensor(self.learning_rate)
            for t in targets:
                t.mul_((1.0 - self.weight_decay * lr_t).to(t.dtype))

    def _check_super_called(self):
        if not hasattr(self, "_lock"):
            raise RuntimeError(f"In optimizer '{self.__class__.__name__}', you forgot to call `super().__init__()` as the first statement in the `__init__()` method. Go add it!")

    def _update_model_variables_moving_average(self, trainable_variables):
        if self.use_ema:
            for var, average in zip(trainable_variables, self._model_variables_moving_average):
                if average is not None:
                    not_first = 0.0 if self._local_step() == 0 else 1.0
                    momentum = not_first * self.ema_momentum
                    average._value.mul_(momentum).add_(var._value, alpha=1 - momentum)

    def _overwrite_model_variables_with_average_value(self, trainable_variables):
        if len(trainable_variables) != len(self._model_variables_moving_average):
            raise ValueError(f"The length of model variables ({len(trainable_variables)}) to override does not match the length of model variables stored in the optimizer ({len(self._model_variables_moving_average)}). Please check if the optimizer was called on your model.")
        for var, average in zip(trainable_variables, self._model_variables_moving_average):
            if average is not None:
                var.assign(average._value)

    def finalize_variable_values(self, var_list):
        if self.use_ema:
            self._overwrite_model_variables_with_average_value(var_list)

    def _obj_type(self):
        return "Optimizer"

    def get_config(self):
        if isinstance(self._learning_rate, learning_rate_schedule.LearningRateSchedule):
            learning_rate = learning_rate_schedule.serialize(self._learning_rate)
        elif isinstance(self._learning_rate, Variable):
            learning_rate = float(self._learning_rate.numpy())
        elif isinstance(self._learning_rate, (float, int)):
            learning_rate = float(self._learning_rate)
        elif callable(self._learning_rate):
            from keras_b200.saving import serialization_lib

            learning_rate = serialization_lib.serialize_keras_object(self._learning_rate)
        else:
            learning_rate = 0.5
        return {
            "name": self.name, "learning_rate": learning_rate, "weight_decay": self.weight_decay, "clipnorm": self.clipnorm,
            "global_clipnorm": self.global_clipnorm, "clipvalue": self.clipvalue, "use_ema": self.use_ema,
            "ema_momentum": self.ema_momentum, "ema_overwrite_frequency": self.ema_overwrite_frequency,
            "loss_scale_factor": self.loss_scale_factor, "gradient_accumulation_steps": self.gradient_accumulation_steps,
        }

    @classmethod
    def from_config(cls, config, custom_objects=None):
        config = dict(config)
        if "learning_rate" in config:
            if isinstance(config["learning_rate"], dict):
                from keras_b200.saving import serialization_lib

                config["learning_rate"] = serialization_lib.deserialize_keras_object(config["learning_rate"], custom_objects=custom_objects)
        return cls(**config)

    def __setattr__(self, name, value):
        if name != "_lock":
            self._track_value(name, value)
        object.__setattr__(self, name, value)

    def _track_value(self, name, value):
        pass

    def _clip_by_norm(self, values, axes=None):
        l2sum = torch.sum(values * values) if axes is None else torch.sum(values * values, dim=axes, keepdim=True)
        pred = l2sum > 0
        l2sum_safe = torch.where(pred, l2sum, torch.ones_like(l2sum))
        l2norm = torch.where(pred, torch.sqrt(l2sum_safe), l2sum)
        intermediate = values * self.clipnorm
        return intermediate / torch.maximum(l2norm, torch.as_tensor(self.clipnorm, dtype=l2norm.dtype, device=l2norm.device))


def global_norm(value_list):
    squared = [torch.sum(torch.square(v.float())) for v in value_list if v is not None]
    return torch.sqrt(torch.sum(torch.stack(squared)))


def clip_by_global_norm(value_list, clip_norm):
    use_norm = global_norm(value_list)
    scale_for_finite = clip_norm * torch.minimum(1.0 / use_norm, torch.as_tensor(1.0 / clip_norm, device=use_norm.device))
    scale = scale_for_finite + (use_norm - use_norm)
    return [v * scale.to(v.dtype) if v is not None else v for v in value_list]
