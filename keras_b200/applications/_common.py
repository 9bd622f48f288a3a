"""Plumbing shared by the ``keras.applications`` builders: argument checks, input tensor, classifier head, weights."""

import os

from keras_b200 import layers
from keras_b200.applications import imagenet_utils
from keras_b200.core import config
from keras_b200.models.functional import Functional
from keras_b200.ops.operation_utils import get_source_inputs


def channel_axis():
    return 3 if config.image_data_format() == "channels_last" else 1


def check_weights(weights, include_top=True, classes=1000):
    """``weights`` is ``None`` or a file path; ImageNet checkpoints need a download that this environment lacks."""
    if weights == "imagenet":
        raise ValueError("Pre-trained ImageNet weights need a download, which is not available here; pass `weights=None` or the path of a weights file.")
    if weights is not None and not os.path.exists(str(weights)):
        raise ValueError("The `weights` argument should be either `None` (random initialization), `imagenet` (pre-training on ImageNet), "
                         f"or the path to the weights file to be loaded. Received: weights={weights}")


def model_input(input_shape, input_tensor, default_size, min_size, include_top, weights):
    """Returns ``(img_input, model_inputs)``."""
    input_shape = imagenet_utils.obtain_input_shape(input_shape, default_size=default_size, min_size=min_size,
                                                    data_format=config.image_data_format(), require_flatten=include_top, weights=weights)
    if input_tensor is None:
        img_input = layers.Input(shape=input_shape)
        return img_input, img_input
    if hasattr(input_tensor, "_keras_history"):
        return input_tensor, get_source_inputs(input_tensor)
    img_input = layers.Input(tensor=input_tensor, shape=input_shape)
    return img_input, img_input


def head(x, include_top, pooling, classes, classifier_activation, weights, dropout=None, pool_name="avg_pool", dense_name="predictions",
         dropout_name="top_dropout", **dense_kwargs):
    if include_top:
        x = layers.GlobalAveragePooling2D(name=pool_name)(x)
        if dropout:
            x = layers.Dropout(dropout, name=dropout_name)(x)
        imagenet_utils.validate_activation(classifier_activation, weights)
        return layers.Dense(classes, activation=classifier_activation, name=dense_name, **dense_kwargs)(x)
    if pooling == "avg":
        return layers.GlobalAveragePooling2D(name=pool_name)(x)
    if pooling == "max":
        return layers.GlobalMaxPooling2D(name="max_pool")(x)
    return x


def finish(inputs, x, name, weights):
    model = Functional(inputs, x, name=name)
    if weights is not None:
        model.load_weights(weights)
    return model


def make_divisible(v, divisor=8, min_value=None):
    if min_value is None:
        min_value = divisor
    new_v = max(min_value, int(v + divisor / 2) // divisor * divisor)
    if new_v < 0.9 * v:
        new_v += divisor
    return new_v


def correct_pad(inputs, kernel_size):
    """Zero padding that makes a stride-2 'valid' convolution behave like TF 'same' (odd/even sizes)."""
    img_dim = 2 if config.image_data_format() == "channels_first" else 1
    input_size = inputs.shape[img_dim:(img_dim + 2)]
    if isinstance(kernel_size, int):
        kernel_size = (kernel_size, kernel_size)
    if input_size[0] is None:
        adjust = (1, 1)
    else:
        adjust = (1 - input_size[0] % 2, 1 - input_size[1] % 2)
    correct = (kernel_size[0] // 2, kernel_size[1] // 2)
    return ((correct[0] - adjust[0], correct[0]), (correct[1] - adjust[1], correct[1]))


def preprocess_fn(mode, *names):
    from keras_b200.core.export_registry import keras_export

    def preprocess_input(x, data_format=None):
        if mode is None:
            return x
        return imagenet_utils.preprocess_input(x, data_format=data_format, mode=mode)

    def decode_predictions(preds, top=5):
        return imagenet_utils.decode_predictions(preds, top=top)

    keras_export([f"keras.applications.{n}.preprocess_input" for n in names])(preprocess_input)
    keras_export([f"keras.applications.{n}.decode_predictions" for n in names])(decode_predictions)
    return preprocess_input, decode_predictions
