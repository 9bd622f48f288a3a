"""Helpers shared by the data adapters (keras/src/trainers/data_adapters/data_adapter_utils.py)."""

import numpy as np
import torch

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export

NUM_BATCHES_FOR_TENSOR_SPEC = 2


@keras_export("keras.utils.unpack_x_y_sample_weight")
def unpack_x_y_sample_weight(data):
    if isinstance(data, list):
        data = tuple(data)
    if not isinstance(data, tuple):
        return (data, None, None)
    if len(data) == 1:
        return (data[0], None, None)
    if len(data) == 2:
        return (data[0], data[1], None)
    if len(data) == 3:
        return (data[0], data[1], data[2])
    raise ValueError(f"Data is expected to be in format `x`, `(x,)`, `(x, y)`, or `(x, y, sample_weight)`, found: {data}")


@keras_export("keras.utils.pack_x_y_sample_weight")
def pack_x_y_sample_weight(x, y=None, sample_weight=None):
    if y is None:
        if not isinstance(x, (tuple, list)):
            return x
        return (x,)
    if sample_weight is None:
        return (x, y)
    return (x, y, sample_weight)


def list_to_tuple(maybe_list):
    if isinstance(maybe_list, list):
        return tuple(maybe_list)
    return maybe_list


def check_data_cardinality(data):
    num_samples = set(int(i.shape[0]) for i in tree.flatten(data))
    if len(num_samples) > 1:
        msg = "Data cardinality is ambiguous. Make sure all arrays contain the same number of samples."
        for label, single_data in zip(["x", "y", "sample_weight"], data):
            sizes = ", ".join(str(i.shape[0]) for i in tree.flatten(single_data))
            msg += f"'{label}' sizes: {sizes}\n"
        raise ValueError(msg)


def class_weight_to_sample_weights(y, class_weight):
    y_numpy = np.asarray(y.cpu() if isinstance(y, torch.Tensor) else y)
    sample_weight = np.ones(shape=(y_numpy.shape[0],), dtype="float32")
    if len(y_numpy.shape) > 1:
        if y_numpy.shape[-1] != 1:
            y_numpy = np.argmax(y_numpy, axis=-1)
        else:
            y_numpy = np.squeeze(y_numpy, axis=-1)
    y_numpy = np.round(y_numpy).astype("int32")
    for i in range(y_numpy.shape[0]):
        sample_weight[i] = class_weight.get(int(y_numpy[i]), 1.0)
    return sample_weight


def is_tensor_like(x):
    return isinstance(x, (np.ndarray, torch.Tensor)) or hasattr(x, "__array__")
