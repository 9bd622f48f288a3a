"""DenseNet-121/169/201 (keras/src/applications/densenet.py): dense blocks of BN-ReLU-1x1(4k)-BN-ReLU-3x3(k) units
with channel concatenation (growth rate 32) and 0.5-compression transitions."""

from keras_b200 import layers
from keras_b200.applications import _common as c
from keras_b200.core.export_registry import keras_export

_EPS = 1.001e-5


def _conv_unit(x, growth_rate, name):
    ax = c.channel_axis()
    y = layers.BatchNormalization(axis=ax, epsilon=_EPS, name=name + "_0_bn")(x)
    y = layers.Activation("relu", name=name + "_0_relu")(y)
    y = layers.Conv2D(4 * growth_rate, 1, use_bias=False, name=name + "_1_conv")(y)
    y = layers.BatchNormalization(axis=ax, epsilon=_EPS, name=name + "_1_bn")(y)
    y = layers.Activation("relu", name=name + "_1_relu")(y)
    y = layers.Conv2D(growth_rate, 3, padding="same", use_bias=False, name=name + "_2_conv")(y)
    return layers.Concatenate(axis=ax, name=name + "_concat")([x, y])


def _transition(x, reduction, name):
    ax = c.channel_axis()
    x = layers.BatchNormalization(axis=ax, epsilon=_EPS, name=name + "_bn")(x)
    x = layers.Activation("relu", name=name + "_relu")(x)
    x = layers.Conv2D(int(x.shape[ax] * reduction), 1, use_bias=False, name=name + "_conv")(x)
    return layers.AveragePooling2D(2, strides=2, name=name + "_pool")(x)


def DenseNet(blocks, include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax",
             name="densenet"):
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, 224, 32, include_top, weights)
    ax = c.channel_axis()
    x = layers.ZeroPadding2D(padding=((3, 3), (3, 3)))(img_input)
    x = layers.Conv2D(64, 7, strides=2, use_bias=False, name="conv1_conv")(x)
    x = layers.BatchNormalization(axis=ax, epsilon=_EPS, name="conv1_bn")(x)
    x = layers.Activation("relu", name="conv1_relu")(x)
    x = layers.ZeroPadding2D(padding=((1, 1), (1, 1)))(x)
    x = layers.MaxPooling2D(3, strides=2, name="pool1")(x)
    for stage, n in enumerate(blocks, start=2):
        for i in range(n):
            x = _conv_unit(x, 32, name=f"conv{stage}_block{i + 1}")
        if stage - 2 < len(blocks) - 1:
            x = _transition(x, 0.5, name=f"pool{stage}")
    x = layers.BatchNormalization(axis=ax, epsilon=_EPS, name="bn")(x)
    x = layers.Activation("relu", name="relu")(x)
    x = c.head(x, include_top, pooling, classes, classifier_activation, weights)
    return c.finish(inputs, x, name, weights)


def _make(name, blocks):
    def build(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax",
              name=name.lower()):
        return DenseNet(blocks, include_top, weights, input_tensor, input_shape, pooling, classes, classifier_activation, name=name)

    build.__name__ = name
    return keras_export([f"keras.applications.densenet.{name}", f"keras.applications.{name}"])(build)


DenseNet121 = _make("DenseNet121", [6, 12, 24, 16])
DenseNet169 = _make("DenseNet169", [6, 12, 32, 32])
DenseNet201 = _make("DenseNet201", [6, 12, 48, 32])
preprocess_input, decode_predictions = c.preprocess_fn("torch", "densenet")
