"""ImageNet helpers (keras/src/applications/imagenet_utils.py): preprocessing modes, input-shape rules."""

import json
import os
import warnings

import numpy as np
import torch

from keras_b200 import activations
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor

CLASS_INDEX = None


@keras_export("keras.applications.imagenet_utils.preprocess_input")
def preprocess_input(x, data_format=None, mode="caffe"):
    if mode not in {"caffe", "tf", "torch"}:
        raise ValueError(f"Expected mode to be one of `caffe`, `tf` or `torch`. Received: mode={mode}")
    data_format = config.standardize_data_format(data_format)
    if isinstance(x, KerasTensor):
        return x
    is_np = isinstance(x, np.ndarray)
    t = torch.as_tensor(x.astype("float32") if is_np and not np.issubdtype(x.dtype, np.floating) else x)
    t = t.to(torch.float32) if not t.dtype.is_floating_point else t.clone()
    ch = -1 if data_format == "channels_last" else (0 if t.ndim == 3 else 1)
    if mode == "tf":
        t = t / 127.5 - 1.0
    else:
        if mode == "torch":
            t = t / 255.0
            mean, std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
        else:
            t = torch.flip(t, dims=(ch % t.ndim,))
            mean, std = [103.939, 116.779, 123.68], None
        shape = [1] * t.ndim
        shape[ch] = 3
        t = t - torch.tensor(mean, dtype=t.dtype, device=t.device).reshape(shape)
        if std is not None:
            t = t / torch.tensor(std, dtype=t.dtype, device=t.device).reshape(shape)
    return t.numpy() if is_np else t


@keras_export("keras.applications.imagenet_utils.decode_predictions")
def decode_predictions(preds, top=5):
    global CLASS_INDEX
    preds = np.asarray(preds.cpu() if isinstance(preds, torch.Tensor) else preds)
    if preds.ndim != 2 or preds.shape[1] != 1000:
        raise ValueError(f"`decode_predictions` expects a batch of predictions (i.e. a 2D array of shape (samples, 1000)). Received array with shape: {preds.shape}")
    if CLASS_INDEX is None:
        path = os.path.join(config.keras_home(), "models", "imagenet_class_index.json")
        if os.path.exists(path):
            with open(path) as f:
                CLASS_INDEX = json.load(f)
        else:
            CLASS_INDEX = {str(i): [f"n{i:08d}", f"class_{i}"] for i in range(1000)}
    results = []
    for pred in preds:
        top_indices = pred.argsort()[-top:][::-1]
        result = [tuple(CLASS_INDEX[str(i)]) + (pred[i],) for i in top_indices]
        result.sort(key=lambda x: x[2], reverse=True)
        results.append(result)
    return results


def obtain_input_shape(input_shape, default_size, min_size, data_format, require_flatten, weights=None):
    if weights != "imagenet" and input_shape and len(input_shape) == 3:
        if data_format == "channels_first":
            if input_shape[0] not in {1, 3}:
                warnings.warn(f"This model usually expects 1 or 3 input channels. However, it was passed an input_shape with {input_shape[0]} input channels.", stacklevel=2)
            default_shape = (input_shape[0], default_size, default_size)
        else:
            if input_shape[-1] not in {1, 3}:
                warnings.warn(f"This model usually expects 1 or 3 input channels. However, it was passed an input_shape with {input_shape[-1]} input channels.", stacklevel=2)
            default_shape = (default_size, default_size, input_shape[-1])
    else:
        default_shape = (3, default_size, default_size) if data_format == "channels_first" else (default_size, default_size, 3)
    if input_shape is not None:
        if len(input_shape) != 3:
            raise ValueError("`input_shape` must be a tuple of three integers.")
        spatial = input_shape[1:] if data_format == "channels_first" else input_shape[:2]
        if any(d is not None and d < min_size for d in spatial):
            raise ValueError(f"Input size must be at least {min_size}x{min_size}; Received: input_shape={input_shape}")
    elif require_flatten:
        input_shape = default_shape
    else:
        input_shape = (3, None, None) if data_format == "channels_first" else (None, None, 3)
    if require_flatten and None in input_shape:
        raise ValueError(f"If `include_top` is True, you should specify a static `input_shape`. Received: input_shape={input_shape}")
    return tuple(input_shape)


def validate_activation(classifier_activation, weights):
    if weights is None:
        return
    classifier_activation = activations.get(classifier_activation)
    if classifier_activation not in {activations.get("softmax"), activations.get(None)}:
        raise ValueError(f"Only `None` and `softmax` activations are allowed for the `classifier_activation` argument when using pretrained weights, with `include_top=True`; Received: classifier_activation={classifier_activation}")
