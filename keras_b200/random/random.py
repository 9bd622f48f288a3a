"""Stateless random ops (``keras.random``): every call is a function of its seed.

Semantics follow keras/src/random/random.py and keras/src/backend/torch/random.py:18-253: a
fresh ``torch.Generator`` seeded with ``(seed + counter) & 0xFFFFFFFF`` per call.
"""

import math

import torch
import torch.nn.functional as F

from keras_b200.core import config
from keras_b200.core.dtypes import to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor, get_device
from keras_b200.random.seed_generator import SeedGenerator, draw_seed

_GENERATORS = {}


def _generator(seed, device):
    """Per-device generator re-seeded for this call (object reuse avoids allocation)."""
    dev = torch.device(device)
    if dev.type == "meta":
        return None
    key = (dev.type, dev.index)
    g = _GENERATORS.get(key)
    if g is None:
        g = torch.Generator(device=dev)
        _GENERATORS[key] = g
    g.manual_seed(draw_seed(seed))
    return g


def _shape(shape):
    return tuple(int(s) for s in shape) if not isinstance(shape, int) else (shape,)


@keras_export("keras.random.normal")
def normal(shape, mean=0.0, stddev=1.0, dtype=None, seed=None):
    td = to_torch_dtype(dtype or config.floatx())
    dev = get_device()
    g = _generator(seed, dev)
    if isinstance(mean, (int, float)) and isinstance(stddev, (int, float)):
        # one kernel that scales and shifts before it rounds to the output type (keras/src/backend/torch/random.py:31-47)
        return torch.normal(float(mean), float(stddev), size=_shape(shape), generator=g, dtype=td, device=dev)
    out = torch.randn(_shape(shape), generator=g, dtype=td, device=dev)
    return out * stddev + mean


@keras_export("keras.random.uniform")
def uniform(shape, minval=0.0, maxval=1.0, dtype=None, seed=None):
    td = to_torch_dtype(dtype or config.floatx())
    if not td.is_floating_point:
        raise ValueError(f"`keras.random.uniform` requires a floating point `dtype`. Received: dtype={dtype}")
    dev = get_device()
    g = _generator(seed, dev)
    out = torch.rand(_shape(shape), generator=g, dtype=td, device=dev)
    if maxval != 1.0 or minval != 0.0:
        out = out * (maxval - minval) + minval
    return out


@keras_export("keras.random.randint")
def randint(shape, minval, maxval, dtype="int32", seed=None):
    td = to_torch_dtype(dtype)
    if td.is_floating_point:
        raise ValueError(f"`keras.random.randint` requires an integer `dtype`. Received: dtype={dtype}")
    dev = get_device()
    g = _generator(seed, dev)
    return torch.randint(int(minval), int(maxval), _shape(shape), generator=g, dtype=td, device=dev)


@keras_export("keras.random.truncated_normal")
def truncated_normal(shape, mean=0.0, stddev=1.0, dtype=None, seed=None):
    """Normal samples within two standard deviations.  Four candidates are drawn per element and the first inside the range
    is taken, which is the reference's rule (keras/src/backend/torch/random.py:114-124), so a seeded initializer gives the
    same weights in both frameworks."""
    td = to_torch_dtype(dtype or config.floatx())
    shape = _shape(shape)
    candidates = normal(shape + (4,), mean=0.0, stddev=1.0, dtype=dtype, seed=seed)
    inside = (candidates > -2) & (candidates < 2)
    first = inside.max(-1, keepdim=True)[1]
    out = candidates.gather(-1, first).squeeze(-1)
    return (out * stddev + mean).to(td)


@keras_export("keras.random.categorical")
def categorical(logits, num_samples, dtype="int32", seed=None):
    logits = convert_to_tensor(logits)
    if logits.ndim != 2:
        raise ValueError(f"`logits` should be a 2-D tensor with shape [batch_size, num_classes]. Received: logits={logits}")
    g = _generator(seed, logits.device)
    probs = torch.softmax(logits.float(), dim=-1)
    return torch.multinomial(probs, num_samples, replacement=True, generator=g).to(to_torch_dtype(dtype))


@keras_export("keras.random.dropout")
def dropout(inputs, rate, noise_shape=None, seed=None):
    """Inverted dropout.  A seeded call (an integer, or a ``SeedGenerator`` that was given a seed) or a ``noise_shape``
    draws a Bernoulli keep-mask from a generator seeded for this call, which reproduces the reference's stream
    (keras/src/backend/torch/random.py:140-175); an unseeded call uses the library's fused dropout."""
    x = convert_to_tensor(inputs)
    if rate >= 1.0:
        return torch.zeros_like(x)
    if rate == 0.0:
        return x
    seeded = seed is not None and not (isinstance(seed, SeedGenerator) and seed._initial_seed is None)
    if not seeded and noise_shape is None:
        return torch.nn.functional.dropout(x, p=rate, training=True)
    keep = 1.0 - rate
    shape = tuple(x.shape) if noise_shape is None else tuple(x.shape[i] if s is None else s for i, s in enumerate(noise_shape))
    g = _generator(seed, x.device)
    probs = torch.full(shape, keep, device=x.device)
    mask = (torch.bernoulli(probs) if g is None else torch.bernoulli(probs, generator=g)).bool()
    if mask.shape != x.shape:
        mask = torch.broadcast_to(mask, x.shape)
    return torch.where(mask, x / keep, torch.zeros((), dtype=x.dtype, device=x.device))


@keras_export("keras.random.shuffle")
def shuffle(x, axis=0, seed=None):
    # Ranks of uniform draws, as keras/src/backend/torch/random.py:177-203 does it: the same seed gives the same order, and
    # for axis > 0 every leading index gets its own permutation.
    x = convert_to_tensor(x)
    axis = axis % x.ndim
    g = _generator(seed, x.device)
    order = torch.rand(tuple(x.shape[: axis + 1]), generator=g, device=x.device).argsort(axis)
    order = order.reshape(tuple(order.shape) + (1,) * (x.ndim - axis - 1)).expand(x.shape)
    return torch.gather(x, axis, order)


@keras_export("keras.random.gamma")
def gamma(shape, alpha, dtype=None, seed=None):
    td = to_torch_dtype(dtype or config.floatx())
    dev = get_device()
    torch_state = torch.random.get_rng_state()
    try:
        torch.manual_seed(draw_seed(seed))
        a = torch.broadcast_to(convert_to_tensor(alpha, dtype="float32").cpu(), _shape(shape))
        out = torch.distributions.Gamma(a, torch.ones_like(a)).sample()
    finally:
        torch.random.set_rng_state(torch_state)
    return out.to(device=dev, dtype=td)


@keras_export("keras.random.binomial")
def binomial(shape, counts, probabilities, dtype=None, seed=None):
    td = to_torch_dtype(dtype or config.floatx())
    dev = get_device()
    torch_state = torch.random.get_rng_state()
    try:
        torch.manual_seed(draw_seed(seed))
        c = torch.broadcast_to(convert_to_tensor(counts, dtype="float32").cpu(), _shape(shape))
        p = torch.broadcast_to(convert_to_tensor(probabilities, dtype="float32").cpu(), _shape(shape))
        out = torch.distributions.Binomial(total_count=c, probs=p).sample()
    finally:
        torch.random.set_rng_state(torch_state)
    return out.to(device=dev, dtype=td)


@keras_export("keras.random.beta")
def beta(shape, alpha, beta, dtype=None, seed=None):
    td = to_torch_dtype(dtype or config.floatx())
    dev = get_device()
    torch_state = torch.random.get_rng_state()
    try:
        torch.manual_seed(draw_seed(seed))
        a = torch.broadcast_to(convert_to_tensor(alpha, dtype="float32").cpu(), _shape(shape))
        b = torch.broadcast_to(convert_to_tensor(beta, dtype="float32").cpu(), _shape(shape))
        out = torch.distributions.Beta(a, b).sample()
    finally:
        torch.random.set_rng_state(torch_state)
    return out.to(device=dev, dtype=td)
