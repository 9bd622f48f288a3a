"""Regularisation layers (keras/src/layers/regularization/*.py)."""

import math

import torch

from keras_b200 import ops, regularizers
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer
from keras_b200.random import random as _random
from keras_b200.random.seed_generator import SeedGenerator


@keras_export("keras.layers.Dropout")
class Dropout(Layer):
    def __init__(self, rate, noise_shape=None, seed=None, **kwargs):
        super().__init__(**kwargs)
        if not 0 <= rate <= 1:
            raise ValueError(f"Invalid value received for argument `rate`. Expected a float value between 0 and 1. Received: rate={rate}")
        self.rate = rate
        self.seed = seed
        self.noise_shape = self._validate_noise_shape(noise_shape)
        if rate > 0:
            self.seed_generator = SeedGenerator(seed)
        self.supports_masking = True
        self.built = True

    def _validate_noise_shape(self, noise_shape):
        if noise_shape is None:
            return None
        if isinstance(noise_shape, str):
            raise ValueError(f"The `noise_shape` argument should not be a string. Received: noise_shape={noise_shape}")
        if not isinstance(noise_shape, (tuple, list)):
            raise ValueError(f"`noise_shape` must be a tuple or a list of integers. Received: noise_shape={noise_shape}")
        for i, d in enumerate(noise_shape):
            if d is not None and not isinstance(d, int):
                raise ValueError(f"`noise_shape` must be a tuple or a list of integers or None. Received: noise_shape[{i}] = {d}")
        return tuple(noise_shape)

    def call(self, inputs, training=False):
        if training and self.rate > 0:
            return _random.dropout(inputs, self.rate, noise_shape=self.noise_shape, seed=self.seed_generator)
        return inputs

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "rate": self.rate, "seed": self.seed, "noise_shape": self.noise_shape}


class _BaseSpatialDropout(Dropout):
    def __init__(self, rate, seed=None, name=None, dtype=None):
        super().__init__(rate, seed=seed, name=name, dtype=dtype)

    def call(self, inputs, training=False):
        if training and self.rate > 0:
            return _random.dropout(inputs, self.rate, noise_shape=self._get_noise_shape(inputs), seed=self.seed_generator)
        return inputs

    def get_config(self):
        return {"rate": self.rate, "seed": self.seed, "name": self.name, "dtype": self.dtype}


@keras_export("keras.layers.SpatialDropout1D")
class SpatialDropout1D(_BaseSpatialDropout):
    def __init__(self, rate, seed=None, name=None, dtype=None):
        super().__init__(rate, seed=seed, name=name, dtype=dtype)
        self.input_spec = InputSpec(ndim=3)

    def _get_noise_shape(self, inputs):
        s = inputs.shape
        return (s[0], 1, s[2])


@keras_export("keras.layers.SpatialDropout2D")
class SpatialDropout2D(_BaseSpatialDropout):
    def __init__(self, rate, data_format=None, seed=None, name=None, dtype=None):
        super().__init__(rate, seed=seed, name=name, dtype=dtype)
        self.data_format = config.standardize_data_format(data_format)
        self.input_spec = InputSpec(ndim=4)

    def _get_noise_shape(self, inputs):
        s = inputs.shape
        return (s[0], s[1], 1, 1) if self.data_format == "channels_first" else (s[0], 1, 1, s[3])

    def get_config(self):
        return {**super().get_config(), "data_format": self.data_format}


@keras_export("keras.layers.SpatialDropout3D")
class SpatialDropout3D(_BaseSpatialDropout):
    def __init__(self, rate, data_format=None, seed=None, name=None, dtype=None):
        super().__init__(rate, seed=seed, name=name, dtype=dtype)
        self.data_format = config.standardize_data_format(data_format)
        self.input_spec = InputSpec(ndim=5)

    def _get_noise_shape(self, inputs):
        s = inputs.shape
        return (s[0], s[1], 1, 1, 1) if self.data_format == "channels_first" else (s[0], 1, 1, 1, s[4])

    def get_config(self):
        return {**super().get_config(), "data_format": self.data_format}


@keras_export("keras.layers.GaussianDropout")
class GaussianDropout(Layer):
    def __init__(self, rate, seed=None, **kwargs):
        super().__init__(**kwargs)
        if not 0 <= rate <= 1:
            raise ValueError(f"Invalid value received for argument `rate`. Expected a float value between 0 and 1. Received: rate={rate}")
        self.rate, self.seed = rate, seed
        if rate > 0:
            self.seed_generator = SeedGenerator(seed)
        self.supports_masking = True
        self.built = True

    def call(self, inputs, training=False):
        if training and self.rate > 0:
            stddev = math.sqrt(self.rate / (1.0 - self.rate))
            noise = _random.normal(tuple(inputs.shape), mean=1.0, stddev=stddev, dtype=self.compute_dtype, seed=self.seed_generator)
            return inputs * noise.to(inputs.device)
        return inputs

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "rate": self.rate, "seed": self.seed}


@keras_export("keras.layers.GaussianNoise")
class GaussianNoise(Layer):
    def __init__(self, stddev, seed=None, **kwargs):
        super().__init__(**kwargs)
        if not 0 <= stddev <= 1:
            raise ValueError(f"Invalid value received for argument `stddev`. Expected a float value between 0 and 1. Received: stddev={stddev}")
        self.stddev, self.seed = stddev, seed
        if stddev > 0:
            self.seed_generator = SeedGenerator(seed)
        self.supports_masking = True
        self.built = True

    def call(self, inputs, training=False):
        if training and self.stddev > 0:
            return inputs + _random.normal(tuple(inputs.shape), mean=0.0, stddev=self.stddev, dtype=self.compute_dtype, seed=self.seed_generator).to(inputs.device)
        return inputs

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "stddev": self.stddev, "seed": self.seed}


@keras_export("keras.layers.AlphaDropout")
class AlphaDropout(Layer):
    def __init__(self, rate, noise_shape=None, seed=None, **kwargs):
        super().__init__(**kwargs)
        if not 0 <= rate <= 1:
            raise ValueError(f"Invalid value received for argument `rate`. Expected a float value between 0 and 1. Received: rate={rate}")
        self.rate, self.seed, self.noise_shape = rate, seed, noise_shape
        if rate > 0:
            self.seed_generator = SeedGenerator(seed)
        self.supports_masking = True
        self.built = True

    def call(self, inputs, training=False):
        if training and self.rate > 0:
            shape = tuple(inputs.shape) if self.noise_shape is None else tuple(inputs.shape[i] if s is None else s for i, s in enumerate(self.noise_shape))
            alpha = 1.6732632423543772848170429916717
            scale = 1.0507009873554804934193349852946
            alpha_p = -alpha * scale
            kept = _random.uniform(shape, seed=self.seed_generator).to(inputs.device) >= self.rate
            kept = kept.to(inputs.dtype)
            a = ((1 - self.rate) * (1 + self.rate * alpha_p ** 2)) ** -0.5
            b = -a * alpha_p * self.rate
            x = inputs * kept + alpha_p * (1 - kept)
            return a * x + b
        return inputs

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        return {**super().get_config(), "rate": self.rate, "seed": self.seed, "noise_shape": self.noise_shape}


@keras_export("keras.layers.ActivityRegularization")
class ActivityRegularization(Layer):
    def __init__(self, l1=0.0, l2=0.0, **kwargs):
        super().__init__(activity_regularizer=regularizers.L1L2(l1=l1, l2=l2), **kwargs)
        self.supports_masking = True
        self.l1, self.l2 = l1, l2
        self.built = True

    def call(self, inputs):
        return inputs

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        cfg = super().get_config()
        cfg.pop("activity_regularizer", None)
        return {**cfg, "l1": self.l1, "l2": self.l2}
