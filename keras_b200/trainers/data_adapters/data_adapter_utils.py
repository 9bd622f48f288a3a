"""Small helpers shared by the data adapters and the training loops
(behaviour of keras/src/trainers/data_adapters/data_adapter_utils.py)."""

import numpy as np
import torch

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export

NUM_BATCHES_FOR_TENSOR_SPEC = 2

_PARTS = ("x", "y", "sample_weight")


@keras_export("keras.utils.unpack_x_y_sample_weight")
def unpack_x_y_sample_weight(data):
    """A batch in any accepted form (``x``, ``(x,)``, ``(x, y)``, ``(x, y, w)``; lists count as tuples) -> ``(x, y, w)``
    with ``None`` for what is absent."""
    if isinstance(data, list):
        data = tuple(data)
    if not isinstance(data, tuple):
        return data, None, None
    if not 1 <= len(data) <= 3:
        raise ValueError(f"Data is expected to be in format `x`, `(x,)`, `(x, y)`, or `(x, y, sample_weight)`, found: {data}")
    return data + (None,) * (3 - len(data))


@keras_export("keras.utils.pack_x_y_sample_weight")
def pack_x_y_sample_weight(x, y=None, sample_weight=None):
    """Inverse of ``unpack_x_y_sample_weight``: trailing ``None`` parts are dropped; a lone ``x`` stays bare unless it is
    itself a tuple or list (then it is wrapped so that it is not mistaken for ``(x, y)``)."""
    if y is not None:
        return (x, y) if sample_weight is None else (x, y, sample_weight)
    return (x,) if isinstance(x, (tuple, list)) else x


def list_to_tuple(maybe_list):
    return tuple(maybe_list) if isinstance(maybe_list, list) else maybe_list


def check_data_cardinality(data):
    """Every array of ``(x, y, sample_weight)`` must have the same number of samples."""
    counts = {int(leaf.shape[0]) for leaf in tree.flatten(data)}
    if len(counts) <= 1:
        return
    lines = ["Data cardinality is ambiguous. Make sure all arrays contain the same number of samples."]
    for label, part in zip(_PARTS, data):
        lines.append(f"'{label}' sizes: " + ", ".join(str(leaf.shape[0]) for leaf in tree.flatten(part)) + "\n")
    raise ValueError("".join(lines))


def class_weight_to_sample_weights(y, class_weight):
    """Per-sample weights from a ``{class index: weight}`` table (1.0 for classes that are not listed).  ``y`` holds class
    indices, possibly with a trailing axis of 1, or one-hot / probability rows (the arg-max is the class)."""
    labels = np.asarray(y.cpu() if isinstance(y, torch.Tensor) else y)
    if labels.ndim > 1:
        labels = np.argmax(labels, axis=-1) if labels.shape[-1] != 1 else labels[..., 0]
    labels = np.round(labels).astype("int32")
    table = {int(k): float(v) for k, v in class_weight.items()}
    return np.fromiter((table.get(int(c), 1.0) for c in labels), dtype="float32", count=labels.shape[0])


def is_tensor_like(x):
    return isinstance(x, (np.ndarray, torch.Tensor)) or hasattr(x, "__array__")
