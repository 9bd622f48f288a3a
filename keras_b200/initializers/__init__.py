"""Weight initializers (``keras.initializers``).

Formulas follow keras/src/initializers/random_initializers.py:207-330,663-699 and
constant_initializers.py: VarianceScaling ``scale/=fan``; truncated normal stddev corrected by
0.87962566103423978; uniform limit ``sqrt(3*scale)``; fans: 2-D ``(in,out)``, conv
``(receptive*in, receptive*out)``.
"""

import math

import numpy as np
import torch

from keras_b200.core import config
from keras_b200.core.dtypes import standardize_dtype, to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor, get_device
from keras_b200.random import random as _random
from keras_b200.random.seed_generator import SeedGenerator, make_default_seed
from keras_b200.utils.registry import build_lookup


@keras_export(["keras.Initializer", "keras.initializers.Initializer"])
class Initializer:
    def __call__(self, shape, dtype=None):
        raise NotImplementedError("Initializer subclasses must implement the `__call__()` method.")

    def get_config(self):
        return {}

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def clone(self):
        return self.__class__.from_config(self.get_config())


@keras_export(["keras.initializers.Zeros", "keras.initializers.zeros"])
class Zeros(Initializer):
    def __call__(self, shape, dtype=None):
        return torch.zeros(tuple(shape), dtype=to_torch_dtype(dtype or config.floatx()), device=get_device())


@keras_export(["keras.initializers.Ones", "keras.initializers.ones"])
class Ones(Initializer):
    def __call__(self, shape, dtype=None):
        return torch.ones(tuple(shape), dtype=to_torch_dtype(dtype or config.floatx()), device=get_device())


@keras_export(["keras.initializers.Constant", "keras.initializers.constant"])
class Constant(Initializer):
    def __init__(self, value=0.0):
        self.value = value

    def __call__(self, shape, dtype=None):
        td = to_torch_dtype(dtype or config.floatx())
        v = convert_to_tensor(self.value, dtype=td)
        return torch.broadcast_to(v, tuple(shape)).clone()

    def get_config(self):
        from keras_b200.saving import serialization_lib

        return {"value": serialization_lib.serialize_keras_object(self.value)}

    @classmethod
    def from_config(cls, config):
        from keras_b200.saving import serialization_lib

        value = serialization_lib.deserialize_keras_object(config["value"])
        return cls(value)


@keras_export(["keras.initializers.Identity", "keras.initializers.identity", "keras.initializers.IdentityInitializer"])
class Identity(Initializer):
    def __init__(self, gain=1.0):
        self.gain = gain

    def __call__(self, shape, dtype=None):
        if len(shape) != 2:
            raise ValueError(f"Identity matrix initializer can only be used for 2D matrices. Received: shape={shape} of rank {len(shape)}.")
        return self.gain * torch.eye(shape[0], shape[1], dtype=to_torch_dtype(dtype or config.floatx()), device=get_device())

    def get_config(self):
        return {"gain": self.gain}


class RandomInitializer(Initializer):
    def __init__(self, seed=None):
        self._init_seed = seed
        if seed is None:
            seed = make_default_seed()
        elif isinstance(seed, dict):
            from keras_b200.saving import serialization_lib

            seed = serialization_lib.deserialize_keras_object(seed)
        elif not isinstance(seed, (int, SeedGenerator)):
            raise ValueError(f"`seed` argument should be an instance of `keras.random.SeedGenerator()` or an integer. Received: seed={seed}")
        self.seed = seed

    def get_config(self):
        from keras_b200.saving import serialization_lib

        return {"seed": serialization_lib.serialize_keras_object(self._init_seed)}


@keras_export(["keras.initializers.RandomNormal", "keras.initializers.random_normal"])
class RandomNormal(RandomInitializer):
    def __init__(self, mean=0.0, stddev=0.05, seed=None):
        self.mean, self.stddev = mean, stddev
        super().__init__(seed=seed)

    def __call__(self, shape, dtype=None):
        return _random.normal(shape, mean=self.mean, stddev=self.stddev, seed=self.seed, dtype=dtype)

    def get_config(self):
        return {"mean": self.mean, "stddev": self.stddev, **super().get_config()}


@keras_export(["keras.initializers.TruncatedNormal", "keras.initializers.truncated_normal"])
class TruncatedNormal(RandomInitializer):
    def __init__(self, mean=0.0, stddev=0.05, seed=None):
        self.mean, self.stddev = mean, stddev
        super().__init__(seed=seed)

    def __call__(self, shape, dtype=None):
        return _random.truncated_normal(shape, mean=self.mean, stddev=self.stddev, seed=self.seed, dtype=dtype)

    def get_config(self):
        return {"mean": self.mean, "stddev": self.stddev, **super().get_config()}


@keras_export(["keras.initializers.RandomUniform", "keras.initializers.random_uniform"])
class RandomUniform(RandomInitializer):
    def __init__(self, minval=-0.05, maxval=0.05, seed=None):
        self.minval, self.maxval = minval, maxval
        super().__init__(seed=seed)

    def __call__(self, shape, dtype=None):
        return _random.uniform(shape, minval=self.minval, maxval=self.maxval, seed=self.seed, dtype=dtype)

    def get_config(self):
        return {"minval": self.minval, "maxval": self.maxval, **super().get_config()}


def compute_fans(shape, input_axes=None, output_axes=None):
    shape = tuple(shape)
    if input_axes is not None or output_axes is not None:
        fan_in = int(np.prod([shape[a] for a in (input_axes or [])])) if input_axes else 1
        fan_out = int(np.prod([shape[a] for a in (output_axes or [])])) if output_axes else 1
        return fan_in, fan_out
    if len(shape) < 1:
        return 1, 1
    if len(shape) == 1:
        return shape[0], shape[0]
    if len(shape) == 2:
        return shape[0], shape[1]
    receptive = int(np.prod(shape[:-2]))
    return shape[-2] * receptive, shape[-1] * receptive


@keras_export(["keras.initializers.VarianceScaling", "keras.initializers.variance_scaling"])
class VarianceScaling(RandomInitializer):
    def __init__(self, scale=1.0, mode="fan_in", distribution="truncated_normal", seed=None, input_axes=None, output_axes=None):
        if scale <= 0.0:
            raise ValueError(f"Argument `scale` must be positive float. Received: scale={scale}")
        if mode not in {"fan_in", "fan_out", "fan_avg"}:
            raise ValueError(f"Invalid `mode` argument: {mode}. Please use one of {{'fan_in', 'fan_out', 'fan_avg'}}")
        distribution = distribution.lower()
        if distribution == "normal":
            distribution = "truncated_normal"
        if distribution not in {"uniform", "truncated_normal", "untruncated_normal"}:
            raise ValueError(f"Invalid `distribution` argument: {distribution}.Please use one of {{'uniform', 'truncated_normal', 'untruncated_normal'}}")
        self.scale, self.mode, self.distribution = scale, mode, distribution
        # which axes of the weight count as inputs / outputs when fans are computed (EinsumDense kernels); None: the
        # usual convention (last axis out, the one before in, leading axes a receptive field)
        self.input_axes, self.output_axes = input_axes, output_axes
        super().__init__(seed=seed)

    def __call__(self, shape, dtype=None, input_axes=None, output_axes=None):
        fan_in, fan_out = compute_fans(shape, input_axes if input_axes is not None else self.input_axes,
                                       output_axes if output_axes is not None else self.output_axes)
        scale = self.scale
        if self.mode == "fan_in":
            scale /= max(1.0, fan_in)
        elif self.mode == "fan_out":
            scale /= max(1.0, fan_out)
        else:
            scale /= max(1.0, (fan_in + fan_out) / 2.0)
        if self.distribution == "truncated_normal":
            stddev = math.sqrt(scale) / 0.87962566103423978
            return _random.truncated_normal(shape, mean=0.0, stddev=stddev, dtype=dtype, seed=self.seed)
        if self.distribution == "untruncated_normal":
            return _random.normal(shape, mean=0.0, stddev=math.sqrt(scale), dtype=dtype, seed=self.seed)
        limit = math.sqrt(3.0 * scale)
        return _random.uniform(shape, minval=-limit, maxval=limit, dtype=dtype, seed=self.seed)

    def get_config(self):
        return {"scale": self.scale, "mode": self.mode, "distribution": self.distribution, **super().get_config(), "input_axes": self.input_axes,
                "output_axes": self.output_axes}


def _vs_subclass(name, exports, scale, mode, distribution):
    def __init__(self, seed=None, input_axes=None, output_axes=None):
        VarianceScaling.__init__(self, scale=scale, mode=mode, distribution=distribution, seed=seed, input_axes=input_axes, output_axes=output_axes)

    def get_config(self):
        return {"seed": RandomInitializer.get_config(self)["seed"], "input_axes": self.input_axes, "output_axes": self.output_axes}

    cls = type(name, (VarianceScaling,), {"__init__": __init__, "get_config": get_config})
    cls.__module__ = __name__
    return keras_export(exports)(cls)


GlorotUniform = _vs_subclass("GlorotUniform", ["keras.initializers.GlorotUniform", "keras.initializers.glorot_uniform"], 1.0, "fan_avg", "uniform")
GlorotNormal = _vs_subclass("GlorotNormal", ["keras.initializers.GlorotNormal", "keras.initializers.glorot_normal"], 1.0, "fan_avg", "truncated_normal")
LecunNormal = _vs_subclass("LecunNormal", ["keras.initializers.LecunNormal", "keras.initializers.lecun_normal"], 1.0, "fan_in", "truncated_normal")
LecunUniform = _vs_subclass("LecunUniform", ["keras.initializers.LecunUniform", "keras.initializers.lecun_uniform"], 1.0, "fan_in", "uniform")
HeNormal = _vs_subclass("HeNormal", ["keras.initializers.HeNormal", "keras.initializers.he_normal"], 2.0, "fan_in", "truncated_normal")
HeUniform = _vs_subclass("HeUniform", ["keras.initializers.HeUniform", "keras.initializers.he_uniform"], 2.0, "fan_in", "uniform")


@keras_export(["keras.initializers.Orthogonal", "keras.initializers.orthogonal", "keras.initializers.OrthogonalInitializer"])
class Orthogonal(RandomInitializer):
    def __init__(self, gain=1.0, seed=None):
        self.gain = gain
        super().__init__(seed=seed)

    def __call__(self, shape, dtype=None):
        if len(shape) < 2:
            raise ValueError(f"The tensor to initialize must be at least two-dimensional. Received: shape={shape} of rank {len(shape)}.")
        rows = int(np.prod(shape[:-1]))
        cols = shape[-1]
        flat = (max(cols, rows), min(cols, rows))
        a = _random.normal(flat, seed=self.seed, dtype="float32")
        q, r = torch.linalg.qr(a)
        d = torch.diagonal(r)
        q = q * torch.sign(d)
        if rows < cols:
            q = q.t()
        return (self.gain * q.reshape(tuple(shape))).to(to_torch_dtype(dtype or config.floatx()))

    def get_config(self):
        return {"gain": self.gain, **super().get_config()}


@keras_export(["keras.initializers.STFT", "keras.initializers.stft", "keras.initializers.STFTInitializer"])
class STFT(Initializer):
    def __init__(self, side="real", window="hann", scaling="density", periodic=False):
        if side not in ("real", "imag"):
            raise ValueError(f"side should be 'real' or 'imag', not {side}")
        if isinstance(window, str) and window not in ("hann", "hamming"):
            raise ValueError("If a string is passed to `window`, it must be one of 'hann', 'hamming'.")
        if scaling is not None and scaling not in ("density", "spectrum"):
            raise ValueError("Scaling is invalid, it must be `None`, 'density' or 'spectrum'. " f"Received scaling={scaling}")
        self.side, self.window, self.scaling, self.periodic = side, window, scaling, periodic

    def __call__(self, shape, dtype=None):
        td = to_torch_dtype(dtype or config.floatx())
        frame_length, input_channels, fft_length = shape
        win = None
        scaling = 1.0
        if self.window:
            n = frame_length + 1 if self.periodic else frame_length
            if self.window == "hann":
                win = torch.hann_window(n, periodic=False, dtype=torch.float64)
            elif self.window == "hamming":
                win = torch.hamming_window(n, periodic=False, dtype=torch.float64)
            else:
                win = convert_to_tensor(self.window).double().cpu()
            win = win[:frame_length]
            if self.scaling == "density":
                scaling = torch.sqrt(torch.sum(win ** 2))
            elif self.scaling == "spectrum":
                scaling = torch.sum(torch.abs(win))
        t = torch.arange(frame_length, dtype=torch.float64)[:, None, None]
        f = torch.arange(fft_length, dtype=torch.float64)[None, None, :]
        args = -2 * math.pi * t * f / ((fft_length - 1) * 2)
        kernel = torch.cos(args) if self.side == "real" else torch.sin(args)
        kernel = kernel.expand(frame_length, input_channels, fft_length).clone()
        if win is not None:
            kernel = kernel * win[:, None, None]
        kernel = kernel / scaling
        return kernel.to(td).to(get_device())

    def get_config(self):
        return {"side": self.side, "window": self.window, "periodic": self.periodic, "scaling": self.scaling}


ALL_OBJECTS = [Initializer, Constant, Identity, Ones, STFT, Zeros, GlorotNormal, GlorotUniform, HeNormal, HeUniform,
               LecunNormal, LecunUniform, Orthogonal, RandomNormal, RandomUniform, TruncatedNormal, VarianceScaling]
_LOOKUP = build_lookup(ALL_OBJECTS, {"uniform": RandomUniform, "normal": RandomNormal, "orthogonal": Orthogonal,
                                     "Orthogonal": Orthogonal, "one": Ones, "zero": Zeros,
                                     "IdentityInitializer": Identity, "OrthogonalInitializer": Orthogonal, "STFTInitializer": STFT})
zeros, ones, constant, identity = Zeros, Ones, Constant, Identity
random_normal, random_uniform, truncated_normal, variance_scaling = RandomNormal, RandomUniform, TruncatedNormal, VarianceScaling
glorot_uniform, glorot_normal, lecun_normal, lecun_uniform, he_normal, he_uniform = GlorotUniform, GlorotNormal, LecunNormal, LecunUniform, HeNormal, HeUniform
orthogonal, stft = Orthogonal, STFT
IdentityInitializer, OrthogonalInitializer, STFTInitializer = Identity, Orthogonal, STFT


@keras_export("keras.initializers.serialize")
def serialize(initializer):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(initializer)


@keras_export("keras.initializers.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(config, module_objects=_LOOKUP, custom_objects=custom_objects)


@keras_export("keras.initializers.get")
def get(identifier):
    if identifier is None:
        return None
    if isinstance(identifier, dict):
        obj = deserialize(identifier)
    elif isinstance(identifier, str):
        obj = _LOOKUP.get(identifier)
        if obj is None:
            raise ValueError(f"Could not interpret initializer identifier: {identifier}")
    elif isinstance(identifier, (torch.Tensor, np.ndarray)) or hasattr(identifier, "__array__"):
        def init_from_value(shape, dtype=None, _v=identifier):
            return convert_to_tensor(_v, dtype=dtype)

        return init_from_value
    else:
        obj = identifier
    if callable(obj):
        if isinstance(obj, type):
            obj = obj()
        return obj
    raise ValueError(f"Could not interpret initializer identifier: {identifier}")
