"""Xception (keras/src/applications/xception.py): entry flow (2 convs + 3 residual separable blocks), middle flow
(8 x 3 separable convs at 728 channels), exit flow (1024 → 1536 → 2048)."""

from keras_b200 import layers
from keras_b200.applications import _common as c
from keras_b200.core.export_registry import keras_export


def _sep(x, filters, name, relu_first=True):
    ax = c.channel_axis()
    if relu_first:
        x = layers.Activation("relu", name=name + "_act")(x)
    x = layers.SeparableConv2D(filters, (3, 3), padding="same", use_bias=False, name=name)(x)
    return layers.BatchNormalization(axis=ax, name=name + "_bn")(x)


@keras_export(["keras.applications.xception.Xception", "keras.applications.Xception"])
def Xception(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax",
             name="xception"):
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, 299, 71, include_top, weights)
    ax = c.channel_axis()
    x = layers.Conv2D(32, (3, 3), strides=(2, 2), use_bias=False, name="block1_conv1")(img_input)
    x = layers.BatchNormalization(axis=ax, name="block1_conv1_bn")(x)
    x = layers.Activation("relu", name="block1_conv1_act")(x)
    x = layers.Conv2D(64, (3, 3), use_bias=False, name="block1_conv2")(x)
    x = layers.BatchNormalization(axis=ax, name="block1_conv2_bn")(x)
    x = layers.Activation("relu", name="block1_conv2_act")(x)
    for b, f in ((2, 128), (3, 256), (4, 728)):
        residual = layers.Conv2D(f, (1, 1), strides=(2, 2), padding="same", use_bias=False)(x)
        residual = layers.BatchNormalization(axis=ax)(residual)
        x = _sep(x, f, f"block{b}_sepconv1", relu_first=b != 2)
        x = _sep(x, f, f"block{b}_sepconv2")
        x = layers.MaxPooling2D((3, 3), strides=(2, 2), padding="same", name=f"block{b}_pool")(x)
        x = layers.Add()([x, residual])
    for i in range(8):
        residual = x
        for j in (1, 2, 3):
            x = _sep(x, 728, f"block{i + 5}_sepconv{j}")
        x = layers.Add()([x, residual])
    residual = layers.Conv2D(1024, (1, 1), strides=(2, 2), padding="same", use_bias=False)(x)
    residual = layers.BatchNormalization(axis=ax)(residual)
    x = _sep(x, 728, "block13_sepconv1")
    x = _sep(x, 1024, "block13_sepconv2")
    x = layers.MaxPooling2D((3, 3), strides=(2, 2), padding="same", name="block13_pool")(x)
    x = layers.Add()([x, residual])
    x = _sep(x, 1536, "block14_sepconv1", relu_first=False)
    x = layers.Activation("relu", name="block14_sepconv1_act")(x)
    x = _sep(x, 2048, "block14_sepconv2", relu_first=False)
    x = layers.Activation("relu", name="block14_sepconv2_act")(x)
    x = c.head(x, include_top, pooling, classes, classifier_activation, weights)
    return c.finish(inputs, x, name, weights)


preprocess_input, decode_predictions = c.preprocess_fn("tf", "xception")
