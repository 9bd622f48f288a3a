"""InceptionV3 and Inception-ResNet-v2 (keras/src/applications/inception_v3.py, inception_resnet_v2.py).

Inception modules are written as tables of branches; a branch is a sequence of ``(filters, kernel[, stride, padding])``
conv-BN-ReLU units, optionally preceded by a pooling step.
"""

from keras_b200 import layers
from keras_b200.applications import _common as c
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.layer import Layer


def _cbr(x, filters, kernel, strides=1, padding="same", activation="relu", use_bias=False, name=None):
    """Conv → BatchNorm(scale=False) → activation."""
    x = layers.Conv2D(filters, kernel, strides=strides, padding=padding, use_bias=use_bias, name=name)(x)
    if not use_bias:
        x = layers.BatchNormalization(axis=c.channel_axis(), scale=False, name=None if name is None else f"{name}_bn")(x)
    if activation is not None:
        x = layers.Activation(activation, name=None if name is None else f"{name}_ac")(x)
    return x


def _branch(x, units):
    for u in units:
        if u[0] == "avg":
            x = layers.AveragePooling2D(3, strides=1, padding="same")(x)
        elif u[0] == "max":
            x = layers.MaxPooling2D(3, strides=2)(x)
        else:
            f, k = u[0], u[1]
            s = u[2] if len(u) > 2 else 1
            p = u[3] if len(u) > 3 else "same"
            x = _cbr(x, f, k, strides=s, padding=p)
    return x


def _module(x, branches, name):
    return layers.Concatenate(axis=c.channel_axis(), name=name)([_branch(x, b) for b in branches])


# ------------------------------------------------------------------------------------ InceptionV3
def _v3_conv(x, filters, rows, cols, padding="same", strides=(1, 1), name=None):
    x = layers.Conv2D(filters, (rows, cols), strides=strides, padding=padding, use_bias=False, name=None if name is None else name + "_conv")(x)
    x = layers.BatchNormalization(axis=c.channel_axis(), scale=False, name=None if name is None else name + "_bn")(x)
    return layers.Activation("relu", name=name)(x)


def _v3_branch(x, units):
    for u in units:
        if u == "avg":
            x = layers.AveragePooling2D((3, 3), strides=(1, 1), padding="same")(x)
        elif u == "max":
            x = layers.MaxPooling2D((3, 3), strides=(2, 2))(x)
        else:
            f, r, cc = u[0], u[1], u[2]
            kw = {"strides": (2, 2), "padding": "valid"} if len(u) > 3 else {}
            x = _v3_conv(x, f, r, cc, **kw)
    return x


@keras_export(["keras.applications.inception_v3.InceptionV3", "keras.applications.InceptionV3"])
def InceptionV3(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax",
                name="inception_v3"):
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, 299, 75, include_top, weights)
    ax = c.channel_axis()
    x = _v3_conv(img_input, 32, 3, 3, strides=(2, 2), padding="valid")
    x = _v3_conv(x, 32, 3, 3, padding="valid")
    x = _v3_conv(x, 64, 3, 3)
    x = layers.MaxPooling2D((3, 3), strides=(2, 2))(x)
    x = _v3_conv(x, 80, 1, 1, padding="valid")
    x = _v3_conv(x, 192, 3, 3, padding="valid")
    x = layers.MaxPooling2D((3, 3), strides=(2, 2))(x)

    def cat(branches, name):
        return layers.Concatenate(axis=ax, name=name)(branches)

    for i, pool_f in enumerate((32, 64, 64)):  # mixed 0-2: 35 x 35
        x = cat([_v3_branch(x, [(64, 1, 1)]), _v3_branch(x, [(48, 1, 1), (64, 5, 5)]), _v3_branch(x, [(64, 1, 1), (96, 3, 3), (96, 3, 3)]),
                 _v3_branch(x, ["avg", (pool_f, 1, 1)])], f"mixed{i}")
    x = cat([_v3_branch(x, [(384, 3, 3, "s2")]), _v3_branch(x, [(64, 1, 1), (96, 3, 3), (96, 3, 3, "s2")]), _v3_branch(x, ["max"])], "mixed3")
    for i, f in enumerate((128, 160, 160, 192)):  # mixed 4-7: 17 x 17
        x = cat([_v3_branch(x, [(192, 1, 1)]), _v3_branch(x, [(f, 1, 1), (f, 1, 7), (192, 7, 1)]),
                 _v3_branch(x, [(f, 1, 1), (f, 7, 1), (f, 1, 7), (f, 7, 1), (192, 1, 7)]), _v3_branch(x, ["avg", (192, 1, 1)])], f"mixed{4 + i}")
    x = cat([_v3_branch(x, [(192, 1, 1), (320, 3, 3, "s2")]), _v3_branch(x, [(192, 1, 1), (192, 1, 7), (192, 7, 1), (192, 3, 3, "s2")]),
             _v3_branch(x, ["max"])], "mixed8")
    for i in range(2):  # mixed 9-10: 8 x 8
        b1 = _v3_conv(x, 320, 1, 1)
        b3 = _v3_conv(x, 384, 1, 1)
        b3 = layers.Concatenate(axis=ax, name=f"mixed9_{i}")([_v3_conv(b3, 384, 1, 3), _v3_conv(b3, 384, 3, 1)])
        bd = _v3_conv(_v3_conv(x, 448, 1, 1), 384, 3, 3)
        bd = layers.Concatenate(axis=ax)([_v3_conv(bd, 384, 1, 3), _v3_conv(bd, 384, 3, 1)])
        bp = _v3_branch(x, ["avg", (192, 1, 1)])
        x = cat([b1, b3, bd, bp], f"mixed{9 + i}")
    x = c.head(x, include_top, pooling, classes, classifier_activation, weights)
    return c.finish(inputs, x, name, weights)


# ---------------------------------------------------------------------------- Inception-ResNet-v2
class CustomScaleLayer(Layer):
    """``inputs[0] + inputs[1] * scale``: the scaled residual of an Inception-ResNet block."""

    def __init__(self, scale, **kwargs):
        super().__init__(**kwargs)
        self.scale = scale

    def get_config(self):
        return {**super().get_config(), "scale": self.scale}

    def call(self, inputs):
        return inputs[0] + inputs[1] * self.scale

    def compute_output_shape(self, input_shape):
        return input_shape[0]


_RES_BRANCHES = {
    "block35": [[(32, 1)], [(32, 1), (32, 3)], [(32, 1), (48, 3), (64, 3)]],
    "block17": [[(192, 1)], [(128, 1), (160, [1, 7]), (192, [7, 1])]],
    "block8": [[(192, 1)], [(192, 1), (224, [1, 3]), (256, [3, 1])]],
}


def _res_block(x, scale, block_type, block_idx, activation="relu"):
    if block_type not in _RES_BRANCHES:
        raise ValueError(f'Unknown Inception-ResNet block type. Expects "block35", "block17" or "block8", but got: {block_type}')
    name = f"{block_type}_{block_idx}"
    mixed = _module(x, _RES_BRANCHES[block_type], f"{name}_mixed")
    up = _cbr(mixed, x.shape[c.channel_axis()], 1, activation=None, use_bias=True, name=f"{name}_conv")
    x = CustomScaleLayer(scale)([x, up])
    if activation is not None:
        x = layers.Activation(activation, name=f"{name}_ac")(x)
    return x


@keras_export(["keras.applications.inception_resnet_v2.InceptionResNetV2", "keras.applications.InceptionResNetV2"])
def InceptionResNetV2(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax",
                      name="inception_resnet_v2"):
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, 299, 75, include_top, weights)
    x = _branch(img_input, [(32, 3, 2, "valid"), (32, 3, 1, "valid"), (64, 3)])
    x = layers.MaxPooling2D(3, strides=2)(x)
    x = _branch(x, [(80, 1, 1, "valid"), (192, 3, 1, "valid")])
    x = layers.MaxPooling2D(3, strides=2)(x)
    x = _module(x, [[(96, 1)], [(48, 1), (64, 5)], [(64, 1), (96, 3), (96, 3)], [("avg",), (64, 1)]], "mixed_5b")
    for i in range(1, 11):
        x = _res_block(x, 0.17, "block35", i)
    x = layers.Concatenate(axis=c.channel_axis(), name="mixed_6a")([
        _branch(x, [(384, 3, 2, "valid")]), _branch(x, [(256, 1), (256, 3), (384, 3, 2, "valid")]), layers.MaxPooling2D(3, strides=2, padding="valid")(x)])
    for i in range(1, 21):
        x = _res_block(x, 0.1, "block17", i)
    x = layers.Concatenate(axis=c.channel_axis(), name="mixed_7a")([
        _branch(x, [(256, 1), (384, 3, 2, "valid")]), _branch(x, [(256, 1), (288, 3, 2, "valid")]),
        _branch(x, [(256, 1), (288, 3), (320, 3, 2, "valid")]), layers.MaxPooling2D(3, strides=2, padding="valid")(x)])
    for i in range(1, 10):
        x = _res_block(x, 0.2, "block8", i)
    x = _res_block(x, 1.0, "block8", 10, activation=None)
    x = _cbr(x, 1536, 1, name="conv_7b")
    x = c.head(x, include_top, pooling, classes, classifier_activation, weights)
    return c.finish(inputs, x, name, weights)


preprocess_input, decode_predictions = c.preprocess_fn("tf", "inception_v3", "inception_resnet_v2")
