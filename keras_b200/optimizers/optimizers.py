"""Concrete optimizers (``keras.optimizers``).

Update rules follow keras/src/optimizers/{sgd,adam,adamw,rmsprop,adagrad,adadelta,adamax,nadam,
lion,lamb,ftrl,adafactor,muon,schedule_free_adamw}.py.  SGD / Adam / AdamW update every variable
in one multi-tensor call: the fused sm_100a kernel on a B200, ``torch._foreach`` elsewhere.
"""

import math
import re

import torch

from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.kernels import dispatch
from keras_b200.optimizers.base_optimizer import BaseOptimizer


@keras_export(["keras.Optimizer", "keras.optimizers.Optimizer"])
class Optimizer(BaseOptimizer):
    pass


def _lr_for(opt, variable_dtype, learning_rate):
    """Learning rate as a float when possible (no sync), else a tensor."""
    lr = opt._lr_float()
    if lr is not None:
        return lr
    return convert_to_tensor(learning_rate).to(variable_dtype)


@keras_export("keras.optimizers.SGD")
class SGD(Optimizer):
    def __init__(self, learning_rate=0.01, momentum=0.0, nesterov=False, weight_decay=None, clipnorm=None, clipvalue=None,
                 global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None, loss_scale_factor=None,
                 gradient_accumulation_steps=None, name="SGD", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        if not isinstance(momentum, float) or momentum < 0 or momentum > 1:
            raise ValueError("`momentum` must be a float between [0, 1].")
        self.momentum = momentum
        self.nesterov = nesterov

    def build(self, variables):
        if self.built:
            return
        super().build(variables)
        self.momentums = []
        if self.momentum != 0:
            self.momentums = self.add_optimizer_variables(variables, "momentum")

    def _fused_apply(self, grads, variables):
        if self.clipnorm or self.global_clipnorm or self.clipvalue or self.use_ema:
            return False
        lr = self._lr_float()
        if lr is None:
            return False
        return dispatch.fused_sgd(self, grads, variables, lr)

    def _backend_update_step(self, grads, variables, learning_rate):
        lr = _lr_for(self, torch.float32, learning_rate)
        if isinstance(lr, float) and len(variables) > 1 and all(g.dtype == v._value.dtype for g, v in zip(grads, variables)):
            params = [v._value for v in variables]
            if self.momentum != 0:
                bufs = [self.momentums[self._get_variable_index(v)]._value for v in variables]
                torch._foreach_mul_(bufs, self.momentum)
                torch._foreach_add_(bufs, grads, alpha=-lr)
                if self.nesterov:
                    torch._foreach_add_(params, bufs, alpha=self.momentum)
                    torch._foreach_add_(params, grads, alpha=-lr)
                else:
                    torch._foreach_add_(params, bufs)
            else:
                torch._foreach_add_(params, grads, alpha=-lr)
            return
        for g, v in zip(grads, variables):
            self.update_step(g, v, learning_rate)

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        if self.momentum != 0:
            m = self.momentums[self._get_variable_index(variable)]._value
            m.mul_(self.momentum).sub_(g * lr)
            if self.nesterov:
                p.add_(m * self.momentum - g * lr)
            else:
                p.add_(m)
        else:
            p.sub_(g * lr)

    def get_config(self):
        return {**super().get_config(), "momentum": self.momentum, "nesterov": self.nesterov}


@keras_export("keras.optimizers.Adam")
class Adam(Optimizer):
    def __init__(self, learning_rate=0.001, beta_1=0.9, beta_2=0.999, epsilon=1e-7, amsgrad=False, weight_decay=None, clipnorm=None,
                 clipvalue=None, global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None,
                 loss_scale_factor=None, gradient_accumulation_steps=None, name="adam", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        self.beta_1, self.beta_2, self.epsilon, self.amsgrad = beta_1, beta_2, epsilon, amsgrad

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        self._momentums, self._velocities = self.add_optimizer_variables(var_list, ["momentum", "velocity"])
        if self.amsgrad:
            self._velocity_hats = self.add_optimizer_variables(var_list, "velocity_hat")

    def _alpha(self, lr):
        t = self._local_step() + 1
        return lr * math.sqrt(1 - self.beta_2 ** t) / (1 - self.beta_1 ** t)

    def _fused_apply(self, grads, variables):
        if self.amsgrad or self.clipnorm or self.global_clipnorm or self.clipvalue or self.use_ema:
            return False
        lr = self._lr_float()
        if lr is None:
            return False
        return dispatch.fused_adam(self, grads, variables, lr)

    def _backend_update_step(self, grads, variables, learning_rate):
        lr = self._lr_float()
        if lr is not None and not self.amsgrad and len(variables) > 1 and all(g.dtype == v._value.dtype for g, v in zip(grads, variables)):
            alpha = self._alpha(lr)
            params = [v._value for v in variables]
            ms = [self._momentums[self._get_variable_index(v)]._value for v in variables]
            vs = [self._velocities[self._get_variable_index(v)]._value for v in variables]
            torch._foreach_lerp_(ms, grads, 1 - self.beta_1)
            torch._foreach_mul_(vs, self.beta_2)
            torch._foreach_addcmul_(vs, grads, grads, value=1 - self.beta_2)
            denom = torch._foreach_sqrt(vs)
            torch._foreach_add_(denom, self.epsilon)
            torch._foreach_addcdiv_(params, ms, denom, value=-alpha)
            return
        for g, v in zip(grads, variables):
            self.update_step(g, v, learning_rate)

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        g = gradient.to(p.dtype)
        lr = self._lr_float()
        if lr is not None:
            alpha = self._alpha(lr)
        else:
            lr_t = convert_to_tensor(learning_rate).to(p.dtype)
            t = (self._iterations._value + 1).to(p.dtype)
            alpha = lr_t * torch.sqrt(1 - self.beta_2 ** t) / (1 - self.beta_1 ** t)
        i = self._get_variable_index(variable)
        m, v = self._momentums[i]._value, self._velocities[i]._value
        m.add_((g - m) * (1 - self.beta_1))
        v.add_((g * g - v) * (1 - self.beta_2))
        if self.amsgrad:
            v_hat = self._velocity_hats[i]._value
            torch.maximum(v_hat, v, out=v_hat)
            v = v_hat
        p.sub_(m * alpha / (torch.sqrt(v) + self.epsilon))

    def get_config(self):
        return {**super().get_config(), "beta_1": self.beta_1, "beta_2": self.beta_2, "epsilon": self.epsilon, "amsgrad": self.amsgrad}


@keras_export("keras.optimizers.AdamW")
class AdamW(Adam):
    def __init__(self, learning_rate=0.001, weight_decay=0.004, beta_1=0.9, beta_2=0.999, epsilon=1e-7, amsgrad=False, clipnorm=None,
                 clipvalue=None, global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None,
                 loss_scale_factor=None, gradient_accumulation_steps=None, name="adamw", **kwargs):
        super().__init__(learning_rate=learning_rate, beta_1=beta_1, beta_2=beta_2, epsilon=epsilon, amsgrad=amsgrad, name=name,
                         weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue, global_clipnorm=global_clipnorm,
                         use_ema=use_ema, ema_momentum=ema_momentum, ema_overwrite_frequency=ema_overwrite_frequency,
                         loss_scale_factor=loss_scale_factor, gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        if self.weight_decay is None:
            raise ValueError("Argument `weight_decay` must be a float. Received: weight_decay=None")


@keras_export("keras.optimizers.RMSprop")
class RMSprop(Optimizer):
    def __init__(self, learning_rate=0.001, rho=0.9, momentum=0.0, epsilon=1e-7, centered=False, weight_decay=None, clipnorm=None,
                 clipvalue=None, global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None,
                 loss_scale_factor=None, gradient_accumulation_steps=None, name="rmsprop", **kwargs):
        super().__init__(learning_rate=learning_rate, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, name=name, **kwargs)
        self.rho, self.momentum, self.epsilon, self.centered = rho, momentum, epsilon, centered

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        self._velocities = self.add_optimizer_variables(var_list, "velocity")
        self._momentums = []
        if self.momentum > 0:
            self._momentums = self.add_optimizer_variables(var_list, "momentum")
        self._average_gradients = []
        if self.centered:
            self._average_gradients = self.add_optimizer_variables(var_list, "average_gradient")

    def _fused_apply(self, grads, variables):
        if self.centered and self.momentum > 0:
            return False  # three slots per variable: the per-variable path
        if self.clipnorm or self.global_clipnorm or self.clipvalue or self.use_ema:
            return False
        lr = self._lr_float()
        if lr is None:
            return False
        second = self._momentums if self.momentum > 0 else (self._average_gradients if self.centered else None)
        return dispatch.fused_rule(self, grads, variables, lr, "rmsprop", [self._velocities, second], (self.rho, self.momentum, self.epsilon),
                                   flags=(1 if self.momentum > 0 else 0) | (2 if self.centered else 0))

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        i = self._get_variable_index(variable)
        v = self._velocities[i]._value
        v.mul_(self.rho).add_(g * g, alpha=1 - self.rho)
        if self.centered:
            ag = self._average_gradients[i]._value
            ag.mul_(self.rho).add_(g, alpha=1 - self.rho)
            denom = v - ag * ag + self.epsilon
        else:
            denom = v + self.epsilon
        inc = g * lr * torch.rsqrt(denom)
        if self.momentum > 0:
            m = self._momentums[i]._value
            m.mul_(self.momentum).add_(inc)
            p.sub_(m)
        else:
            p.sub_(inc)

    def get_config(self):
        return {**super().get_config(), "rho": self.rho, "momentum": self.momentum, "epsilon": self.epsilon, "centered": self.centered}


@keras_export("keras.optimizers.Adagrad")
class Adagrad(Optimizer):
    def __init__(self, learning_rate=0.001, initial_accumulator_value=0.1, epsilon=1e-7, weight_decay=None, clipnorm=None, clipvalue=None,
                 global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None, loss_scale_factor=None,
                 gradient_accumulation_steps=None, name="adagrad", **kwargs):
        super().__init__(learning_rate=learning_rate, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, name=name, **kwargs)
        self.initial_accumulator_value, self.epsilon = initial_accumulator_value, epsilon

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        from keras_b200 import initializers

        self._accumulators = self.add_optimizer_variables(var_list, "accumulator", initializer=initializers.Constant(self.initial_accumulator_value))

    def _fused_apply(self, grads, variables):
        if self.clipnorm or self.global_clipnorm or self.clipvalue or self.use_ema:
            return False
        lr = self._lr_float()
        if lr is None:
            return False
        return dispatch.fused_rule(self, grads, variables, lr, "adagrad", [self._accumulators], (self.epsilon,))

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        acc = self._accumulators[self._get_variable_index(variable)]._value
        acc.add_(g * g)
        p.sub_(lr * g / torch.sqrt(acc + self.epsilon))

    def get_config(self):
        return {**super().get_config(), "initial_accumulator_value": self.initial_accumulator_value, "epsilon": self.epsilon}


@keras_export("keras.optimizers.Adadelta")
class Adadelta(Optimizer):
    def __init__(self, learning_rate=0.001, rho=0.95, epsilon=1e-7, weight_decay=None, clipnorm=None, clipvalue=None, global_clipnorm=None,
                 use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None, loss_scale_factor=None,
                 gradient_accumulation_steps=None, name="adadelta", **kwargs):
        super().__init__(learning_rate=learning_rate, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, name=name, **kwargs)
        self.rho, self.epsilon = rho, epsilon

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        self._accumulated_grads, self._accumulated_delta_vars = self.add_optimizer_variables(var_list, ["accumulated_grad", "accumulated_delta_var"])

    def _fused_apply(self, grads, variables):
        if self.clipnorm or self.global_clipnorm or self.clipvalue or self.use_ema:
            return False
        lr = self._lr_float()
        if lr is None:
            return False
        return dispatch.fused_rule(self, grads, variables, lr, "adadelta", [self._accumulated_grads, self._accumulated_delta_vars], (self.rho, self.epsilon))

    def update_step(self, grad, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = grad.to(p.dtype)
        i = self._get_variable_index(variable)
        ag, ad = self._accumulated_grads[i]._value, self._accumulated_delta_vars[i]._value
        ag.mul_(self.rho).add_(g * g, alpha=1 - self.rho)
        delta = -torch.sqrt(ad + self.epsilon) * g / torch.sqrt(ag + self.epsilon)
        ad.mul_(self.rho).add_(delta * delta, alpha=1 - self.rho)
        p.add_(lr * delta)

    def get_config(self):
        return {**super().get_config(), "rho": self.rho, "epsilon": self.epsilon}


@keras_export("keras.optimizers.Adamax")
class Adamax(Optimizer):
    def __init__(self, learning_rate=0.001, beta_1=0.9, beta_2=0.999, epsilon=1e-7, weight_decay=None, clipnorm=None, clipvalue=None,
                 global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None, loss_scale_factor=None,
                 gradient_accumulation_steps=None, name="adamax", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        self.beta_1, self.beta_2, self.epsilon = beta_1, beta_2, epsilon

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        self._m, self._u = self.add_optimizer_variables(var_list, ["momentum", "norm"])

    def _fused_apply(self, grads, variables):
        if self.clipnorm or self.global_clipnorm or self.clipvalue or self.use_ema:
            return False
        lr = self._lr_float()
        if lr is None:
            return False
        t = self._local_step() + 1
        return dispatch.fused_rule(self, grads, variables, lr, "adamax", [self._m, self._u], (self.beta_1, self.beta_2, self.epsilon),
                                   step_scalars=(1 - self.beta_1 ** t,), beta1=self.beta_1, beta2=self.beta_2, needs_step=True)

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        t = self._local_step() + 1
        i = self._get_variable_index(variable)
        m, u = self._m[i]._value, self._u[i]._value
        m.add_((g - m) * (1 - self.beta_1))
        torch.maximum(self.beta_2 * u, torch.abs(g), out=u)
        p.sub_((lr * m) / ((1 - self.beta_1 ** t) * (u + self.epsilon)))

    def get_config(self):
        return {**super().get_config(), "beta_1": self.beta_1, "beta_2": self.beta_2, "epsilon": self.epsilon}


@keras_export("keras.optimizers.Nadam")
class Nadam(Optimizer):
    def __init__(self, learning_rate=0.001, beta_1=0.9, beta_2=0.999, epsilon=1e-7, weight_decay=None, clipnorm=None, clipvalue=None,
                 global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None, loss_scale_factor=None,
                 gradient_accumulation_steps=None, name="nadam", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        self.beta_1, self.beta_2, self.epsilon = beta_1, beta_2, epsilon

    def build(self, var_list):
        if self.built:
            return
        dtype = var_list[0].dtype if var_list else "float32"
        super().build(var_list)
        self._momentums, self._velocities = self.add_optimizer_variables(var_list, ["momentum", "velocity"])
        from keras_b200.core.variables import Variable
        from keras_b200.core.scopes import name_scope

        with name_scope(self.name, caller=self):
            self._u_product = Variable(1.0, dtype=dtype, trainable=False, name="u_product")
        self._track_variable(self._u_product)

    def _fused_apply(self, grads, variables):
        if self.clipnorm or self.global_clipnorm or self.clipvalue or self.use_ema:
            return False
        lr = self._lr_float()
        if lr is None:
            return False
        from keras_b200.kernels.dispatch import _device_scalars

        u = self._u_product._value
        if _device_scalars(self)[1] is None or not (u.is_cuda and u.dtype == torch.float32):
            return False
        # the kernel advances the running product and derives the step scalars from the device-resident iteration counter
        return dispatch.fused_rule(self, grads, variables, lr, "nadam", [self._momentums, self._velocities], (self.beta_1, self.beta_2, self.epsilon),
                                   beta1=self.beta_1, beta2=self.beta_2, u_product=u, needs_step=True)

    def _backend_update_step(self, grads, trainable_variables, learning_rate):
        dtype = self._u_product._value.dtype
        t = self._local_step() + 1
        u_t = self.beta_1 * (1.0 - 0.5 * (0.96 ** t))
        self._u_product._value.mul_(u_t)
        super()._backend_update_step(grads, trainable_variables, learning_rate)

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        t = self._local_step() + 1
        u_t = self.beta_1 * (1.0 - 0.5 * (0.96 ** t))
        u_t_1 = self.beta_1 * (1.0 - 0.5 * (0.96 ** (t + 1)))
        u_product_t = self._u_product._value.to(p.dtype)
        u_product_t_1 = u_product_t * u_t_1
        beta_2_power = self.beta_2 ** t
        i = self._get_variable_index(variable)
        m, v = self._momentums[i]._value, self._velocities[i]._value
        m.add_((g - m) * (1 - self.beta_1))
        v.add_((g * g - v) * (1 - self.beta_2))
        m_hat = (u_t_1 * m) / (1 - u_product_t_1) + ((1 - u_t) * g) / (1 - u_product_t)
        v_hat = v / (1 - beta_2_power)
        p.sub_((m_hat * lr) / (torch.sqrt(v_hat) + self.epsilon))

    def get_config(self):
        return {**super().get_config(), "beta_1": self.beta_1, "beta_2": self.beta_2, "epsilon": self.epsilon}


@keras_export("keras.optimizers.Lion")
class Lion(Optimizer):
    def __init__(self, learning_rate=0.001, beta_1=0.9, beta_2=0.99, weight_decay=None, clipnorm=None, clipvalue=None, global_clipnorm=None,
                 use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None, loss_scale_factor=None,
                 gradient_accumulation_steps=None, name="lion", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        self.beta_1, self.beta_2 = beta_1, beta_2
        if beta_1 <= 0 or beta_1 > 1:
            raise ValueError(f"Argument `beta_1` must be in the [0, 1] range. Otherwise, the optimizer degenerates to SignSGD. Received: beta_1={beta_1}.")

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        self._momentums = self.add_optimizer_variables(var_list, "momentum")

    def _fused_apply(self, grads, variables):
        if self.clipnorm or self.global_clipnorm or self.clipvalue or self.use_ema:
            return False
        lr = self._lr_float()
        if lr is None:
            return False
        return dispatch.fused_rule(self, grads, variables, lr, "lion", [self._momentums], (self.beta_1, self.beta_2))

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        m = self._momentums[self._get_variable_index(variable)]._value
        p.sub_(lr * torch.sign(m * self.beta_1 + g * (1.0 - self.beta_1)))
        m.mul_(self.beta_2).add_(g, alpha=1.0 - self.beta_2)

    def get_config(self):
        return {**super().get_config(), "beta_1": self.beta_1, "beta_2": self.beta_2}


@keras_export("keras.optimizers.Lamb")
class Lamb(Optimizer):
    def __init__(self, learning_rate=0.001, beta_1=0.9, beta_2=0.999, epsilon=1e-7, weight_decay=None, clipnorm=None, clipvalue=None,
                 global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None, loss_scale_factor=None,
                 gradient_accumulation_steps=None, name="lamb", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        self.beta_1, self.beta_2, self.epsilon = beta_1, beta_2, epsilon

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        self._momentums, self._velocities = self.add_optimizer_variables(var_list, ["momentum", "velocity"])

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        t = self._local_step() + 1
        i = self._get_variable_index(variable)
        m, v = self._momentums[i]._value, self._velocities[i]._value
        m.add_((g - m) * (1 - self.beta_1))
        v.add_((g * g - v) * (1 - self.beta_2))
        m_hat = m / (1.0 - self.beta_1 ** t)
        v_hat = v / (1.0 - self.beta_2 ** t)
        update = m_hat / (torch.sqrt(v_hat) + self.epsilon)
        w_norm = torch.sqrt(torch.sum(p * p))
        g_norm = torch.sqrt(torch.sum(update * update))
        ratio = torch.where(w_norm > 0, torch.where(g_norm > 0, w_norm / g_norm, torch.ones_like(w_norm)), torch.ones_like(w_norm))
        p.sub_(ratio * lr * update)

    def get_config(self):
        return {**super().get_config(), "beta_1": self.beta_1, "beta_2": self.beta_2, "epsilon": self.epsilon}


@keras_export("keras.optimizers.Ftrl")
class Ftrl(Optimizer):
    def __init__(self, learning_rate=0.001, learning_rate_power=-0.5, initial_accumulator_value=0.1, l1_regularization_strength=0.0,
                 l2_regularization_strength=0.0, l2_shrinkage_regularization_strength=0.0, beta=0.0, weight_decay=None, clipnorm=None,
                 clipvalue=None, global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None,
                 loss_scale_factor=None, gradient_accumulation_steps=None, name="ftrl", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        if initial_accumulator_value < 0.0:
            raise ValueError(f"`initial_accumulator_value` needs to be positive or zero. Received: initial_accumulator_value={initial_accumulator_value}.")
        if learning_rate_power > 0.0:
            raise ValueError(f"`learning_rate_power` needs to be negative or zero. Received: learning_rate_power={learning_rate_power}.")
        if l1_regularization_strength < 0.0:
            raise ValueError(f"`l1_regularization_strength` needs to be positive or zero. Received: l1_regularization_strength={l1_regularization_strength}.")
        if l2_regularization_strength < 0.0:
            raise ValueError(f"`l2_regularization_strength` needs to be positive or zero. Received: l2_regularization_strength={l2_regularization_strength}.")
        if l2_shrinkage_regularization_strength < 0.0:
            raise ValueError(f"`l2_shrinkage_regularization_strength` needs to be positive or zero. Received: l2_shrinkage_regularization_strength={l2_shrinkage_regularization_strength}.")
        self.learning_rate_power = learning_rate_power
        self.initial_accumulator_value = initial_accumulator_value
        self.l1_regularization_strength = l1_regularization_strength
        self.l2_regularization_strength = l2_regularization_strength
        self.l2_shrinkage_regularization_strength = l2_shrinkage_regularization_strength
        self.beta = beta

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        from keras_b200 import initializers

        self._accumulators, self._linears = self.add_optimizer_variables(
            var_list, ["accumulator", "linear"], initializer=[initializers.Constant(self.initial_accumulator_value), "zeros"])

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        i = self._get_variable_index(variable)
        accum, linear = self._accumulators[i]._value, self._linears[i]._value
        lr_power = self.learning_rate_power
        l2_reg = self.l2_regularization_strength + self.beta / (2.0 * lr)
        grad_to_use = g + 2 * self.l2_shrinkage_regularization_strength * p
        new_accum = accum + g * g
        linear.add_(grad_to_use - (torch.pow(new_accum, -lr_power) - torch.pow(accum, -lr_power)) / lr * p)
        quadratic = torch.pow(new_accum, -lr_power) / lr + 2 * l2_reg
        linear_clipped = torch.clip(linear, -self.l1_regularization_strength, self.l1_regularization_strength)
        p.copy_((linear_clipped - linear) / quadratic)
        accum.copy_(new_accum)

    def get_config(self):
        return {**super().get_config(), "learning_rate_power": self.learning_rate_power,
                "initial_accumulator_value": self.initial_accumulator_value,
                "l1_regularization_strength": self.l1_regularization_strength,
                "l2_regularization_strength": self.l2_regularization_strength,
                "l2_shrinkage_regularization_strength": self.l2_shrinkage_regularization_strength, "beta": self.beta}


@keras_export("keras.optimizers.Adafactor")
class Adafactor(Optimizer):
    def __init__(self, learning_rate=0.001, beta_2_decay=-0.8, epsilon_1=1e-30, epsilon_2=1e-3, clip_threshold=1.0, relative_step=True,
                 weight_decay=None, clipnorm=None, clipvalue=None, global_clipnorm=None, use_ema=False, ema_momentum=0.99,
                 ema_overwrite_frequency=None, loss_scale_factor=None, gradient_accumulation_steps=None, name="adafactor", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        self.beta_2_decay, self.epsilon_1, self.epsilon_2 = beta_2_decay, epsilon_1, epsilon_2
        self.clip_threshold, self.relative_step = clip_threshold, relative_step

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        from keras_b200.core.variables import Variable

        self._r, self._c, self._v = [], [], []
        for var in var_list:
            if len(var.shape) < 2:
                self._r.append(Variable(0, name=var.name, trainable=False))
                self._c.append(Variable(0, name=var.name, trainable=False))
            elif self._overwrite_variable_with_gradient(var):
                self._r.append(None)
                self._c.append(None)
            else:
                self._r.append(self.add_variable(shape=var.shape[:-1], dtype=var.dtype, name=var.name))
                self._c.append(self.add_variable(shape=var.shape[:-2] + (var.shape[-1],), dtype=var.dtype, name=var.name))
            if self._overwrite_variable_with_gradient(var):
                self._v.append(None)
            else:
                self._v.append(self.add_variable_from_reference(reference_variable=var, name="velocity"))

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        t = float(self._local_step() + 1)
        if not callable(self._learning_rate) and self.relative_step:
            lr = min(lr, 1 / math.sqrt(t)) if isinstance(lr, float) else torch.minimum(lr, torch.as_tensor(1 / math.sqrt(t), dtype=p.dtype, device=p.device))
        i = self._get_variable_index(variable)
        r, c, v = self._r[i], self._c[i], self._v[i]._value
        rho_t = min(lr, 1 / math.sqrt(t)) if isinstance(lr, float) else torch.minimum(lr, torch.as_tensor(1 / math.sqrt(t), dtype=p.dtype, device=p.device))
        rms = torch.sqrt(torch.mean(p * p))
        alpha_t = torch.clamp(rms, min=self.epsilon_2) * rho_t
        reg_sq = g * g + self.epsilon_1
        beta_2_t = 1 - t ** self.beta_2_decay
        if p.ndim >= 2:
            rv, cv = r._value, c._value
            rv.mul_(beta_2_t).add_(torch.mean(reg_sq, dim=-1), alpha=1 - beta_2_t)
            cv.mul_(beta_2_t).add_(torch.mean(reg_sq, dim=-2), alpha=1 - beta_2_t)
            v.copy_((rv / torch.mean(rv, dim=-1, keepdim=True)).unsqueeze(-1) * cv.unsqueeze(-2))
        else:
            v.mul_(beta_2_t).add_(reg_sq, alpha=1 - beta_2_t)
        u_t = g / torch.sqrt(v)
        u_t_hat = u_t / torch.clamp(torch.sqrt(torch.mean(u_t * u_t)) / self.clip_threshold, min=1.0)
        p.sub_(alpha_t * u_t_hat)

    def get_config(self):
        return {**super().get_config(), "beta_2_decay": self.beta_2_decay, "epsilon_1": self.epsilon_1, "epsilon_2": self.epsilon_2,
                "clip_threshold": self.clip_threshold, "relative_step": self.relative_step}


@keras_export("keras.optimizers.Muon")
class Muon(Optimizer):
    def __init__(self, learning_rate=0.001, adam_beta_1=0.9, adam_beta_2=0.999, adam_weight_decay=0.004, epsilon=1e-7, weight_decay=0.004,
                 clipnorm=None, clipvalue=None, global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None,
                 loss_scale_factor=None, gradient_accumulation_steps=None, name="muon", exclude_layers=None, exclude_embeddings=True,
                 muon_a=3.4445, muon_b=-4.7750, muon_c=2.0315, adam_lr_ratio=1, momentum=0.95, ns_steps=5, nesterov=True, rms_rate=0.2, **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        self.adam_beta_1, self.adam_beta_2, self.epsilon = adam_beta_1, adam_beta_2, epsilon
        self.muon_a, self.muon_b, self.muon_c = muon_a, muon_b, muon_c
        self.adam_lr_ratio, self.momentum, self.ns_steps, self.nesterov = adam_lr_ratio, momentum, ns_steps, nesterov
        self.exclude_embeddings = exclude_embeddings
        self.exclude_layers = exclude_layers or []
        self.adam_weight_decay = adam_weight_decay
        self.rms_rate = rms_rate

    def _should_use_adamw(self, variable):
        if len(variable.shape) != 2:
            return True
        if self.exclude_embeddings and "embedding" in variable.path.lower():
            return True
        return any(re.search(k, variable.path) for k in self.exclude_layers)

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        self.momentums = [None] * len(var_list)
        self.adam_velocities = [None] * len(var_list)
        for var in var_list:
            if not self._overwrite_variable_with_gradient(var):
                i = self._get_variable_index(var)
                self.momentums[i] = self.add_variable_from_reference(reference_variable=var, name="momentum")
                if self._should_use_adamw(var):
                    self.adam_velocities[i] = self.add_variable_from_reference(reference_variable=var, name="velocity")

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        i = self._get_variable_index(variable)
        m = self.momentums[i]._value
        v = self.adam_velocities[i]
        if v is not None:
            v = v._value
            t = self._local_step() + 1
            alpha = lr * self.adam_lr_ratio * math.sqrt(1 - self.adam_beta_2 ** t) / (1 - self.adam_beta_1 ** t)
            m.add_((g - m) * (1 - self.adam_beta_1))
            v.add_((g * g - v) * (1 - self.adam_beta_2))
            p.sub_(m * alpha / (torch.sqrt(v) + self.epsilon))
        else:
            m.add_(g + m * (self.momentum - 1))
            upd = g + self.momentum * m if self.nesterov else m
            upd = self.zeropower_via_newtonschulz5(upd, self.ns_steps)
            p.sub_(self.lr_adjust(lr * upd))

    def lr_adjust(self, x):
        if self.rms_rate is None:
            return x
        return x * math.sqrt(max(x.shape[0], x.shape[1])) * self.rms_rate

    def zeropower_via_newtonschulz5(self, x, steps):
        if x.ndim < 2:
            raise ValueError(f"Expected gradient or momentum to have at least 2 dimensions. Received: shape={tuple(x.shape)}")
        a, b, c = self.muon_a, self.muon_b, self.muon_c
        transposed = x.shape[-2] > x.shape[-1]
        if transposed:
            x = x.transpose(-1, -2)
        x = x / (torch.linalg.matrix_norm(x, dim=(-2, -1), keepdim=True) + 1e-7)
        for _ in range(steps):
            A = x @ x.transpose(-1, -2)
            B = b * A + c * A @ A
            x = a * x + B @ x
        return x.transpose(-1, -2) if transposed else x

    def _apply_weight_decay(self, variables):
        lr = self._lr_float()
        lr_v = lr if lr is not None else convert_to_tensor(self.learning_rate)
        for variable in variables:
            if not self._use_weight_decay(variable):
                continue
            wd = self.adam_weight_decay if self._should_use_adamw(variable) else self.weight_decay
            if wd is None:
                continue
            variable._value.mul_(1 - wd * lr_v)

    def get_config(self):
        return {**super().get_config(), "adam_beta_1": self.adam_beta_1, "adam_beta_2": self.adam_beta_2, "epsilon": self.epsilon,
                "exclude_layers": self.exclude_layers, "muon_a": self.muon_a, "muon_b": self.muon_b, "muon_c": self.muon_c,
                "adam_lr_ratio": self.adam_lr_ratio, "momentum": self.momentum, "ns_steps": self.ns_steps, "nesterov": self.nesterov,
                "exclude_embeddings": self.exclude_embeddings, "adam_weight_decay": self.adam_weight_decay, "rms_rate": self.rms_rate}


@keras_export("keras.optimizers.ScheduleFreeAdamW")
class ScheduleFreeAdamW(Optimizer):
    def __init__(self, learning_rate=0.0025, beta_1=0.9, beta_2=0.999, epsilon=1e-8, warmup_steps=0, weight_decay=0.0, clipnorm=None,
                 clipvalue=None, global_clipnorm=None, use_ema=False, ema_momentum=0.99, ema_overwrite_frequency=None,
                 loss_scale_factor=None, gradient_accumulation_steps=None, name="schedule_free_adamw", **kwargs):
        super().__init__(learning_rate=learning_rate, name=name, weight_decay=weight_decay, clipnorm=clipnorm, clipvalue=clipvalue,
                         global_clipnorm=global_clipnorm, use_ema=use_ema, ema_momentum=ema_momentum,
                         ema_overwrite_frequency=ema_overwrite_frequency, loss_scale_factor=loss_scale_factor,
                         gradient_accumulation_steps=gradient_accumulation_steps, **kwargs)
        self.beta_1, self.beta_2, self.epsilon, self.warmup_steps = beta_1, beta_2, epsilon, warmup_steps

    def build(self, var_list):
        if self.built:
            return
        super().build(var_list)
        self._momentums, self._velocities = self.add_optimizer_variables(var_list, ["momentum", "velocity"])
        for m, var in zip(self._momentums, var_list):
            if m is not None:
                m.assign(var._value.detach().clone())

    def update_step(self, gradient, variable, learning_rate):
        p = variable._value
        lr = _lr_for(self, p.dtype, learning_rate)
        g = gradient.to(p.dtype)
        t = float(self._local_step() + 1)
        if self.warmup_steps > 0:
            lr = lr * min(t / self.warmup_steps, 1.0)
        i = self._get_variable_index(variable)
        z, v = self._momentums[i]._value, self._velocities[i]._value
        # On the reference's torch backend "the momentum before the update" is read through `Variable.value`, which hands out
        # the parameter itself, so the value it then uses is the momentum *after* the in-place update
        # (keras/src/optimizers/schedule_free_adamw.py:137,156-167).  Checkpoints and trajectories of that backend are the
        # contract here, so the same value is used.
        z_old = z
        bc2 = 1 - self.beta_2 ** t
        v.add_((g * g - v) * (1 - self.beta_2))
        denom = torch.sqrt(v / bc2) + self.epsilon
        z.sub_(lr * g / denom)
        weight = 1.0 / t
        x_old = (p - (1 - self.beta_1) * z_old) / self.beta_1
        x_new = (1 - weight) * x_old + weight * z
        p.copy_((1 - self.beta_1) * z + self.beta_1 * x_new)

    def get_config(self):
        return {**super().get_config(), "beta_1": self.beta_1, "beta_2": self.beta_2, "epsilon": self.epsilon, "warmup_steps": self.warmup_steps}
