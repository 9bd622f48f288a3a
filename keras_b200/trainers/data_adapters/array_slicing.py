"""Train/validation splitting of array-like inputs (keras/src/trainers/data_adapters/array_slicing.py)."""

import math

import numpy as np
import torch

from keras_b200 import tree


def train_validation_split(arrays, validation_split):
    """Split every array at the same index: the *last* fraction becomes validation data."""
    flat = [a for a in tree.flatten(arrays) if a is not None]

    def ok(a):
        return isinstance(a, (np.ndarray, torch.Tensor)) or hasattr(a, "__array__") or hasattr(a, "to_numpy")

    bad = [type(a) for a in flat if not ok(a)]
    if bad:
        raise ValueError(f"Argument `validation_split` is only supported for tensors or NumPy arrays. Found incompatible type in the input: {bad}")
    if not flat:
        return arrays, arrays
    batch_dim = int(flat[0].shape[0])
    split_at = int(math.floor(batch_dim * (1.0 - validation_split)))
    if split_at == 0 or split_at == batch_dim:
        raise ValueError(f"Training data contains {batch_dim} samples, which is not sufficient to split it into a validation and training set as specified by `validation_split={validation_split}`. Either provide more data, or a different value for the `validation_split` argument.")

    def take(a, lo, hi):
        if a is None:
            return None
        if hasattr(a, "iloc"):
            return a.iloc[lo:hi]
        return a[lo:hi]

    train = tree.map_structure(lambda a: take(a, 0, split_at), arrays)
    val = tree.map_structure(lambda a: take(a, split_at, batch_dim), arrays)
    return train, val
