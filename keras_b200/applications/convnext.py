"""ConvNeXt Tiny/Small/Base/Large/XLarge (keras/src/applications/convnext.py): patchify stem (4x4/4 conv + LN), four
stages of ``7x7 depthwise → LN → 4x MLP (GELU) → layer-scale → stochastic depth`` residual blocks separated by
``LN → 2x2/2 conv`` down-sampling, and an ``avg-pool → LN → Dense`` head."""

import numpy as np

from keras_b200 import initializers, layers, ops, random
from keras_b200.applications import _common as c
from keras_b200.applications import imagenet_utils
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.core.naming import get_uid
from keras_b200.layers.layer import Layer
from keras_b200.models.sequential import Sequential

_VARIANTS = {
    "tiny": ([3, 3, 9, 3], [96, 192, 384, 768]), "small": ([3, 3, 27, 3], [96, 192, 384, 768]), "base": ([3, 3, 27, 3], [128, 256, 512, 1024]),
    "large": ([3, 3, 27, 3], [192, 384, 768, 1536]), "xlarge": ([3, 3, 27, 3], [256, 512, 1024, 2048]),
}


class StochasticDepth(Layer):
    """Drop the whole residual branch of a sample with probability ``drop_path_rate`` (training only)."""

    def __init__(self, drop_path_rate, **kwargs):
        super().__init__(**kwargs)
        self.drop_path_rate = drop_path_rate

    def call(self, x, training=None):
        if training:
            keep = 1 - self.drop_path_rate
            shape = (ops.shape(x)[0],) + (1,) * (len(ops.shape(x)) - 1)
            mask = ops.floor(keep + random.uniform(shape, 0, 1))
            return (x / keep) * ops.cast(mask, x.dtype)
        return x

    def get_config(self):
        return {**super().get_config(), "drop_path_rate": self.drop_path_rate}


class LayerScale(Layer):
    """Per-channel learnable scale initialised to a small constant."""

    def __init__(self, init_values, projection_dim, **kwargs):
        super().__init__(**kwargs)
        self.init_values, self.projection_dim = init_values, projection_dim

    def build(self, _):
        self.gamma = self.add_weight(shape=(self.projection_dim,), initializer=initializers.Constant(self.init_values), trainable=True)

    def call(self, x):
        return x * self.gamma

    def get_config(self):
        return {**super().get_config(), "init_values": self.init_values, "projection_dim": self.projection_dim}


def _block(x, dim, drop_path_rate, layer_scale_init_value, name):
    inputs = x
    x = layers.Conv2D(filters=dim, kernel_size=7, padding="same", groups=dim, name=f"{name}_depthwise_conv")(x)
    x = layers.LayerNormalization(epsilon=1e-6, name=f"{name}_layernorm")(x)
    x = layers.Dense(4 * dim, name=f"{name}_pointwise_conv_1")(x)
    x = layers.Activation("gelu", name=f"{name}_gelu")(x)
    x = layers.Dense(dim, name=f"{name}_pointwise_conv_2")(x)
    if layer_scale_init_value is not None:
        x = LayerScale(layer_scale_init_value, dim, name=f"{name}_layer_scale")(x)
    branch = StochasticDepth(drop_path_rate, name=f"{name}_stochastic_depth") if drop_path_rate else layers.Activation("linear", name=f"{name}_identity")
    return inputs + branch(x)


def ConvNeXt(depths, projection_dims, drop_path_rate=0.0, layer_scale_init_value=1e-6, default_size=224, name="convnext", include_preprocessing=True,
             include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax",
             weights_name=None):
    if config.image_data_format() == "channels_first":
        raise ValueError("ConvNeXt does not support the `channels_first` image data format. Switch to `channels_last` by editing your local config file at ~/.keras/keras.json")
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, default_size, 32, include_top, weights)
    if isinstance(inputs, list):
        inputs = inputs[0]
    x = img_input
    if include_preprocessing and img_input.shape[-1] == 3:
        x = layers.Normalization(mean=[0.485 * 255, 0.456 * 255, 0.406 * 255], variance=[(0.229 * 255) ** 2, (0.224 * 255) ** 2, (0.225 * 255) ** 2],
                                 name=f"{name}_prestem_normalization")(x)
    down = [Sequential([layers.Conv2D(projection_dims[0], kernel_size=4, strides=4, name=f"{name}_stem_conv"),
                        layers.LayerNormalization(epsilon=1e-6, name=f"{name}_stem_layernorm")], name=f"{name}_stem")]
    for i in range(3):
        down.append(Sequential([layers.LayerNormalization(epsilon=1e-6, name=f"{name}_downsampling_layernorm_{i}"),
                                layers.Conv2D(projection_dims[i + 1], kernel_size=2, strides=2, name=f"{name}_downsampling_conv_{i}")],
                               name=f"{name}_downsampling_block_{i}"))
    rates = [float(r) for r in np.linspace(0.0, drop_path_rate, sum(depths))]
    cur = 0
    for i in range(4):
        x = down[i](x)
        for j in range(depths[i]):
            x = _block(x, projection_dims[i], rates[cur + j], layer_scale_init_value, f"{name}_stage_{i}_block_{j}")
        cur += depths[i]
    if include_top:
        imagenet_utils.validate_activation(classifier_activation, weights)
        x = layers.GlobalAveragePooling2D(name=f"{name}_head_gap")(x)
        x = layers.LayerNormalization(epsilon=1e-6, name=f"{name}_head_layernorm")(x)
        x = layers.Dense(classes, activation=classifier_activation, name=f"{name}_head_dense")(x)
    else:
        if pooling == "avg":
            x = layers.GlobalAveragePooling2D()(x)
        elif pooling == "max":
            x = layers.GlobalMaxPooling2D()(x)
        x = layers.LayerNormalization(epsilon=1e-6)(x)
    return c.finish(inputs, x, name, weights)


def _make(name, key):
    depths, dims = _VARIANTS[key]

    def build(include_top=True, include_preprocessing=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000,
              classifier_activation="softmax", name=f"convnext_{key}"):
        return ConvNeXt(depths, dims, 0.0, 1e-6, 224, name, include_preprocessing, include_top, weights, input_tensor, input_shape, pooling, classes,
                        classifier_activation)

    build.__name__ = name
    return keras_export([f"keras.applications.convnext.{name}", f"keras.applications.{name}"])(build)


ConvNeXtTiny = _make("ConvNeXtTiny", "tiny")
ConvNeXtSmall = _make("ConvNeXtSmall", "small")
ConvNeXtBase = _make("ConvNeXtBase", "base")
ConvNeXtLarge = _make("ConvNeXtLarge", "large")
ConvNeXtXLarge = _make("ConvNeXtXLarge", "xlarge")
preprocess_input, decode_predictions = c.preprocess_fn(None, "convnext")
