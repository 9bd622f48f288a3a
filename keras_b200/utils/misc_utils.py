"""Small public utilities: ``set_random_seed``, ``to_categorical``, ``normalize``, ``pad_sequences``."""

import random

import numpy as np
import torch

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export


@keras_export("keras.utils.set_random_seed")
def set_random_seed(seed):
    """Seed Python, NumPy and the framework RNGs (keras/src/utils/rng_utils.py:15-79)."""
    if not isinstance(seed, int):
        raise ValueError(f"Expected `seed` argument to be an integer. Received: seed={seed} (of type {type(seed)})")
    global_state.set_global_attribute("global_random_seed", seed)
    global_state.set_global_attribute("global_seed_generator", None)
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)


def get_random_seed():
    return global_state.get_global_attribute("global_random_seed")


@keras_export("keras.utils.to_categorical")
def to_categorical(x, num_classes=None):
    if isinstance(x, torch.Tensor):
        # a tensor stays a tensor (the torch one-hot without a dtype is int64: keras/src/backend/torch/nn.py:872-886);
        # anything else gives a float64 NumPy array (keras/src/utils/numerical_utils.py:77-103)
        from keras_b200 import ops

        if x.ndim > 1 and x.shape[-1] == 1:
            x = x.reshape(tuple(x.shape[:-1]))
        return ops.one_hot(x, num_classes, dtype="int64")
    x = np.array(x, dtype="int64")
    input_shape = x.shape
    if input_shape and input_shape[-1] == 1 and len(input_shape) > 1:
        input_shape = tuple(input_shape[:-1])
    x = x.reshape(-1)
    if not num_classes:
        num_classes = np.max(x) + 1
    out = np.zeros((x.shape[0], num_classes))
    out[np.arange(x.shape[0]), x] = 1
    return out.reshape(input_shape + (num_classes,))


@keras_export("keras.utils.normalize")
def normalize(x, axis=-1, order=2):
    from keras_b200 import ops

    if isinstance(x, np.ndarray):
        x = x.astype("float32")
        norm = np.atleast_1d(np.linalg.norm(x, order, axis))
        norm[norm == 0] = 1
        return x / np.expand_dims(norm, axis)
    return ops.normalize(x, axis=axis, order=order)


@keras_export(["keras.utils.pad_sequences", "keras.preprocessing.sequence.pad_sequences"])
def pad_sequences(sequences, maxlen=None, dtype="int32", padding="pre", truncating="pre", value=0.0):
    if not hasattr(sequences, "__len__"):
        raise ValueError("`sequences` must be iterable.")
    num_samples = len(sequences)
    lengths, sample_shape, flag = [], (), True
    for x in sequences:
        try:
            lengths.append(len(x))
            if flag and len(x):
                sample_shape = np.asarray(x).shape[1:]
                flag = False
        except TypeError as e:
            raise ValueError(f"`sequences` must be a list of iterables. Found non-iterable: {str(x)}") from e
    if maxlen is None:
        maxlen = np.max(lengths) if lengths else 0
    is_dtype_str = np.issubdtype(dtype, np.str_) or np.issubdtype(dtype, np.str_)
    if isinstance(value, str) and dtype is not object and not is_dtype_str:
        raise ValueError(f"`dtype` {dtype} is not compatible with `value`'s type: {type(value)}\nYou should set `dtype=object` for variable length strings.")
    x = np.full((num_samples, maxlen) + sample_shape, value, dtype=dtype)
    for idx, s in enumerate(sequences):
        if not len(s):
            continue
        if truncating == "pre":
            trunc = s[-maxlen:]
        elif truncating == "post":
            trunc = s[:maxlen]
        else:
            raise ValueError(f'Truncating type "{truncating}" not understood')
        trunc = np.asarray(trunc, dtype=dtype)
        if trunc.shape[1:] != sample_shape:
            raise ValueError(f"Shape of sample {trunc.shape[1:]} of sequence at position {idx} is different from expected shape {sample_shape}")
        if padding == "post":
            x[idx, : len(trunc)] = trunc
        elif padding == "pre":
            x[idx, -len(trunc):] = trunc
        else:
            raise ValueError(f'Padding type "{padding}" not understood')
    return x
