"""Learning-rate schedules (keras/src/optimizers/schedules/learning_rate_schedule.py)."""

import math

import torch

from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor


def _f(x):
    return convert_to_tensor(x).to(torch.float32) if not isinstance(x, (int, float)) else torch.as_tensor(float(x))


@keras_export("keras.optimizers.schedules.LearningRateSchedule")
class LearningRateSchedule:
    def __call__(self, step):
        raise NotImplementedError(f"Learning rate schedule '{self.__class__.__name__}' must override `__call__(self, step)`.")

    def get_config(self):
        raise NotImplementedError(f"Learning rate schedule '{self.__class__.__name__}' must override `get_config()` in order to be serializable.")

    @classmethod
    def from_config(cls, config):
        return cls(**config)


@keras_export("keras.optimizers.schedules.ExponentialDecay")
class ExponentialDecay(LearningRateSchedule):
    def __init__(self, initial_learning_rate, decay_steps, decay_rate, staircase=False, name="ExponentialDecay"):
        super().__init__()
        self.initial_learning_rate, self.decay_steps, self.decay_rate = initial_learning_rate, decay_steps, decay_rate
        self.staircase, self.name = staircase, name
        if self.decay_steps <= 0:
            raise ValueError(f"Argument `decay_steps` must be > 0. Received: decay_steps={self.decay_steps}")

    def __call__(self, step):
        p = _f(step) / float(self.decay_steps)
        if self.staircase:
            p = torch.floor(p)
        return self.initial_learning_rate * torch.pow(torch.as_tensor(float(self.decay_rate)), p)

    def get_config(self):
        return {"initial_learning_rate": self.initial_learning_rate, "decay_steps": self.decay_steps, "decay_rate": self.decay_rate,
                "staircase": self.staircase, "name": self.name}


@keras_export("keras.optimizers.schedules.PiecewiseConstantDecay")
class PiecewiseConstantDecay(LearningRateSchedule):
    def __init__(self, boundaries, values, name="PiecewiseConstant"):
        super().__init__()
        if len(boundaries) != len(values) - 1:
            raise ValueError(f"The length of boundaries should be 1 less than the length of values. Received: boundaries={boundaries} of length {len(boundaries)}, and values={values} of length {len(values)}.")
        self.boundaries, self.values, self.name = boundaries, values, name

    def __call__(self, step):
        s = _f(step)
        b = torch.as_tensor([float(x) for x in self.boundaries], device=s.device)
        v = torch.as_tensor([float(x) for x in self.values], device=s.device)
        idx = torch.sum((s > b).to(torch.int64))
        return v[idx]

    def get_config(self):
        return {"boundaries": self.boundaries, "values": self.values, "name": self.name}


@keras_export("keras.optimizers.schedules.PolynomialDecay")
class PolynomialDecay(LearningRateSchedule):
    def __init__(self, initial_learning_rate, decay_steps, end_learning_rate=0.0001, power=1.0, cycle=False, name="PolynomialDecay"):
        super().__init__()
        self.initial_learning_rate, self.decay_steps, self.end_learning_rate = initial_learning_rate, decay_steps, end_learning_rate
        self.power, self.cycle, self.name = power, cycle, name
        if self.decay_steps <= 0:
            raise ValueError(f"Argument `decay_steps` must be > 0. Received: decay_steps={self.decay_steps}")

    def __call__(self, step):
        s = _f(step)
        decay_steps = torch.as_tensor(float(self.decay_steps), device=s.device)
        if self.cycle:
            mult = torch.where(s == 0, torch.ones_like(s), torch.ceil(s / decay_steps))
            decay_steps = decay_steps * mult
        else:
            s = torch.minimum(s, decay_steps)
        p = s / decay_steps
        return (self.initial_learning_rate - self.end_learning_rate) * torch.pow(1 - p, self.power) + self.end_learning_rate

    def get_config(self):
        return {"initial_learning_rate": self.initial_learning_rate, "decay_steps": self.decay_steps,
                "end_learning_rate": self.end_learning_rate, "power": self.power, "cycle": self.cycle, "name": self.name}


@keras_export("keras.optimizers.schedules.InverseTimeDecay")
class InverseTimeDecay(LearningRateSchedule):
    def __init__(self, initial_learning_rate, decay_steps, decay_rate, staircase=False, name="InverseTimeDecay"):
        super().__init__()
        self.initial_learning_rate, self.decay_steps, self.decay_rate = initial_learning_rate, decay_steps, decay_rate
        self.staircase, self.name = staircase, name
        if self.decay_steps <= 0:
            raise ValueError(f"Argument `decay_steps` must be > 0. Received: decay_steps={self.decay_steps}")

    def __call__(self, step):
        p = _f(step) / float(self.decay_steps)
        if self.staircase:
            p = torch.floor(p)
        return self.initial_learning_rate / (1 + self.decay_rate * p)

    def get_config(self):
        return {"initial_learning_rate": self.initial_learning_rate, "decay_steps": self.decay_steps, "decay_rate": self.decay_rate,
                "staircase": self.staircase, "name": self.name}


@keras_export("keras.optimizers.schedules.CosineDecay")
class CosineDecay(LearningRateSchedule):
    def __init__(self, initial_learning_rate, decay_steps, alpha=0.0, name="CosineDecay", warmup_target=None, warmup_steps=0):
        super().__init__()
        self.initial_learning_rate, self.decay_steps, self.alpha, self.name = initial_learning_rate, decay_steps, alpha, name
        self.warmup_steps, self.warmup_target = warmup_steps, warmup_target
        if self.decay_steps <= 0:
            raise ValueError(f"Argument `decay_steps` must be > 0. Received: decay_steps={self.decay_steps}")

    def _decay(self, step, peak):
        completed = step / float(self.decay_steps)
        cosine = 0.5 * (1.0 + torch.cos(math.pi * completed))
        return peak * ((1 - self.alpha) * cosine + self.alpha)

    def __call__(self, step):
        s = _f(step)
        if self.warmup_target is None:
            return self._decay(torch.clamp(s, max=float(self.decay_steps)), self.initial_learning_rate)
        warm = (self.warmup_target - self.initial_learning_rate) * (s / float(self.warmup_steps)) + self.initial_learning_rate if self.warmup_steps > 0 else torch.as_tensor(float(self.warmup_target))
        dec = self._decay(torch.clamp(s - self.warmup_steps, min=0.0, max=float(self.decay_steps)), self.warmup_target)
        return torch.where(s < self.warmup_steps, warm, dec)

    def get_config(self):
        return {"initial_learning_rate": self.initial_learning_rate, "decay_steps": self.decay_steps, "alpha": self.alpha,
                "name": self.name, "warmup_target": self.warmup_target, "warmup_steps": self.warmup_steps}


@keras_export("keras.optimizers.schedules.CosineDecayRestarts")
class CosineDecayRestarts(LearningRateSchedule):
    def __init__(self, initial_learning_rate, first_decay_steps, t_mul=2.0, m_mul=1.0, alpha=0.0, name="SGDRDecay"):
        super().__init__()
        self.initial_learning_rate, self.first_decay_steps = initial_learning_rate, first_decay_steps
        self._t_mul, self._m_mul, self.alpha, self.name = t_mul, m_mul, alpha, name
        if self.first_decay_steps <= 0:
            raise ValueError(f"Argument `first_decay_steps` must be > 0. Received: first_decay_steps={self.first_decay_steps}")

    def __call__(self, step):
        s = _f(step)
        completed = s / float(self.first_decay_steps)
        t_mul, m_mul = float(self._t_mul), float(self._m_mul)
        if t_mul == 1.0:
            i_restart = torch.floor(completed)
            frac = completed - i_restart
        else:
            i_restart = torch.floor(torch.log(1.0 - completed * (1.0 - t_mul)) / math.log(t_mul))
            sum_r = (1.0 - t_mul ** i_restart) / (1.0 - t_mul)
            frac = (completed - sum_r) / t_mul ** i_restart
        m_fac = m_mul ** i_restart
        cosine = 0.5 * m_fac * (1.0 + torch.cos(math.pi * frac))
        return self.initial_learning_rate * ((1 - self.alpha) * cosine + self.alpha)

    def get_config(self):
        return {"initial_learning_rate": self.initial_learning_rate, "first_decay_steps": self.first_decay_steps,
                "t_mul": self._t_mul, "m_mul": self._m_mul, "alpha": self.alpha, "name": self.name}


@keras_export("keras.optimizers.schedules.serialize")
def serialize(learning_rate_schedule):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(learning_rate_schedule)


@keras_export("keras.optimizers.schedules.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(config, module_objects=globals(), custom_objects=custom_objects, printable_module_name="decay")
