"""``SeedGenerator``: stateful source of seeds for stateless random ops.

Behaviour of keras/src/random/seed_generator.py:15-170: the state is a 2-element variable
``[seed, counter]``; ``next()`` returns the current state and bumps the counter.
"""

import random as _py_random

import numpy as np
import torch

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export
from keras_b200.core.naming import auto_name
from keras_b200.core.scopes import name_scope


@keras_export("keras.random.SeedGenerator")
class SeedGenerator:
    def __init__(self, seed=None, name=None, **kwargs):
        from keras_b200.core.variables import Variable

        if name is None:
            name = auto_name(self.__class__.__name__)
        self.name = name
        custom_backend = kwargs.pop("backend", None)
        if kwargs:
            raise ValueError(f"Unrecognized keyword arguments: {kwargs}")
        self._initial_seed = seed  # what the caller gave (None: unseeded); random ops use it to pick their unseeded fast paths
        if seed is None:
            seed = make_default_seed()
        if not isinstance(seed, int):
            raise ValueError(f"Argument `seed` must be an integer. Received: seed={seed}")
        self._seed_value = seed

        def seed_init(*args, **kw):
            return torch.tensor([seed & 0x7FFFFFFF if seed > 0x7FFFFFFF else seed, 0], dtype=torch.int32)

        with name_scope(self.name, caller=self):
            self.state = Variable(seed_init, shape=(2,), dtype="int32", trainable=False, aggregation="none", name="seed_generator_state")
        # The counter is mirrored on the host so drawing a seed never forces a device sync.
        self._host_counter = 0

    def next(self, ordered=True):
        from keras_b200.core.scopes import in_stateless_scope

        if in_stateless_scope():
            state = self.state.value
            new = state + torch.tensor([0, 1], dtype=state.dtype, device=state.device)
            self.state.assign(new)
            return state
        counter = self._host_counter
        self._host_counter = counter + 1
        with torch.no_grad():
            self.state._value[1] = self._host_counter
        return (self._seed_value, counter)

    def get_config(self):
        return {"seed": self._initial_seed, "name": self.name}

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def _obj_type(self):
        return "SeedGenerator"


def global_seed_generator():
    gen = global_state.get_global_attribute("global_seed_generator")
    if gen is None:
        gen = SeedGenerator()
        global_state.set_global_attribute("global_seed_generator", gen)
    return gen


def make_default_seed():
    return _py_random.randint(1, int(1e9))


class CaptureUnsafe(RuntimeError):
    """Raised when a seed is drawn while a training step is being recorded for replay: the seed is host state, and a
    replay would repeat the recorded one."""


_capture_depth = 0


def begin_capture():
    global _capture_depth
    _capture_depth += 1


def end_capture():
    global _capture_depth
    _capture_depth = max(0, _capture_depth - 1)


def draw_seed(seed):
    """User-facing ``seed`` argument → integer seed for a ``torch.Generator``."""
    if _capture_depth:
        raise CaptureUnsafe("a random seed was drawn while the step was being recorded")
    if isinstance(seed, SeedGenerator):
        s = seed.next()
    elif isinstance(seed, int):
        return seed & 0xFFFFFFFF
    elif seed is None:
        s = global_seed_generator().next(ordered=False)
    elif isinstance(seed, (tuple, list)) and len(seed) == 2:
        s = seed
    elif isinstance(seed, torch.Tensor):
        s = seed.tolist()
    else:
        raise ValueError(
            "Argument `seed` must be either an integer or an instance of `SeedGenerator`. "
            f"Received: seed={seed} (of type {type(seed)})"
        )
    if isinstance(s, torch.Tensor):
        s = s.tolist()
    return (int(s[0]) + int(s[1])) & 0xFFFFFFFF
