"""EfficientNet B0–B7 and EfficientNetV2 B0–B3/S/M/L (keras/src/applications/efficientnet.py, efficientnet_v2.py).

Both generations are compound-scaled stacks of mobile inverted bottlenecks; one builder ``_mbconv`` covers the
depthwise (``MBConv``) and the fused (``FusedMBConv``, v2 early stages) variants.  Stage tables are
``(kernel, repeats, in, out, expand, se_ratio, stride, fused)``.
"""

import math

from keras_b200 import layers
from keras_b200.applications import _common as c
from keras_b200.core.export_registry import keras_export

_CONV_INIT = {"class_name": "VarianceScaling", "config": {"scale": 2.0, "mode": "fan_out", "distribution": "truncated_normal"}}
_DENSE_INIT = {"class_name": "VarianceScaling", "config": {"scale": 1.0 / 3.0, "mode": "fan_out", "distribution": "uniform"}}

_V1_STAGES = [(3, 1, 32, 16, 1, 0.25, 1, 0), (3, 2, 16, 24, 6, 0.25, 2, 0), (5, 2, 24, 40, 6, 0.25, 2, 0), (3, 3, 40, 80, 6, 0.25, 2, 0),
              (5, 3, 80, 112, 6, 0.25, 1, 0), (5, 4, 112, 192, 6, 0.25, 2, 0), (3, 1, 192, 320, 6, 0.25, 1, 0)]
_V2_B = [(3, 1, 32, 16, 1, 0, 1, 1), (3, 2, 16, 32, 4, 0, 2, 1), (3, 2, 32, 48, 4, 0, 2, 1), (3, 3, 48, 96, 4, 0.25, 2, 0), (3, 5, 96, 112, 6, 0.25, 1, 0),
         (3, 8, 112, 192, 6, 0.25, 2, 0)]
_V2_STAGES = {
    "efficientnetv2-b0": _V2_B, "efficientnetv2-b1": _V2_B, "efficientnetv2-b2": _V2_B, "efficientnetv2-b3": _V2_B,
    "efficientnetv2-s": [(3, 2, 24, 24, 1, 0, 1, 1), (3, 4, 24, 48, 4, 0, 2, 1), (3, 4, 48, 64, 4, 0, 2, 1), (3, 6, 64, 128, 4, 0.25, 2, 0),
                         (3, 9, 128, 160, 6, 0.25, 1, 0), (3, 15, 160, 256, 6, 0.25, 2, 0)],
    "efficientnetv2-m": [(3, 3, 24, 24, 1, 0, 1, 1), (3, 5, 24, 48, 4, 0, 2, 1), (3, 5, 48, 80, 4, 0, 2, 1), (3, 7, 80, 160, 4, 0.25, 2, 0),
                         (3, 14, 160, 176, 6, 0.25, 1, 0), (3, 18, 176, 304, 6, 0.25, 2, 0), (3, 5, 304, 512, 6, 0.25, 1, 0)],
    "efficientnetv2-l": [(3, 4, 32, 32, 1, 0, 1, 1), (3, 7, 32, 64, 4, 0, 2, 1), (3, 7, 64, 96, 4, 0, 2, 1), (3, 10, 96, 192, 4, 0.25, 2, 0),
                         (3, 19, 192, 224, 6, 0.25, 1, 0), (3, 25, 224, 384, 6, 0.25, 2, 0), (3, 7, 384, 640, 6, 0.25, 1, 0)],
}


def _round_filters(filters, width, divisor=8, min_depth=None):
    filters *= width
    floor = divisor if min_depth is None else min_depth
    new = max(floor, int(filters + divisor / 2) // divisor * divisor)
    if min_depth is None and new < 0.9 * filters:  # the v1 rule keeps at least 90% of the scaled width; v2 does not
        new += divisor
    return int(new)


def _squeeze_excite(x, filters, filters_se, activation, name):
    ax = c.channel_axis()
    se = layers.GlobalAveragePooling2D(name=name + "se_squeeze")(x)
    se = layers.Reshape((filters, 1, 1) if ax == 1 else (1, 1, filters), name=name + "se_reshape")(se)
    se = layers.Conv2D(filters_se, 1, padding="same", activation=activation, kernel_initializer=_CONV_INIT, name=name + "se_reduce")(se)
    se = layers.Conv2D(filters, 1, padding="same", activation="sigmoid", kernel_initializer=_CONV_INIT, name=name + "se_expand")(se)
    return layers.multiply([x, se], name=name + "se_excite")


def _mbconv(x, name, f_in, f_out, kernel, stride, expand, se_ratio, fused, drop, activation, bn, v2):
    """One (fused) mobile inverted bottleneck.  ``v2`` selects the v2 conventions ('same' padding, ``dwconv2`` name)."""
    inputs = x
    filters = f_in * expand
    if expand != 1:
        if fused:
            x = layers.Conv2D(filters, kernel, strides=stride, padding="same", use_bias=False, kernel_initializer=_CONV_INIT, name=name + "expand_conv")(x)
        else:
            x = layers.Conv2D(filters, 1, padding="same", use_bias=False, kernel_initializer=_CONV_INIT, name=name + "expand_conv")(x)
        x = layers.BatchNormalization(name=name + "expand_bn", **bn)(x)
        x = layers.Activation(activation, name=name + "expand_activation")(x)
    if not fused:
        if stride == 2 and not v2:
            x = layers.ZeroPadding2D(padding=c.correct_pad(x, kernel), name=name + "dwconv_pad")(x)
            pad = "valid"
        else:
            pad = "same"
        x = layers.DepthwiseConv2D(kernel, strides=stride, padding=pad, use_bias=False, depthwise_initializer=_CONV_INIT,
                                   name=name + ("dwconv2" if v2 else "dwconv"))(x)
        x = layers.BatchNormalization(name=name + "bn", **bn)(x)
        x = layers.Activation(activation, name=name + "activation")(x)
    if 0 < se_ratio <= 1:
        x = _squeeze_excite(x, filters, max(1, int(f_in * se_ratio)), activation, name)
    if fused and expand == 1:
        x = layers.Conv2D(f_out, kernel, strides=stride, padding="same", use_bias=False, kernel_initializer=_CONV_INIT, name=name + "project_conv")(x)
    else:
        x = layers.Conv2D(f_out, 1, padding="same", use_bias=False, kernel_initializer=_CONV_INIT, name=name + "project_conv")(x)
    x = layers.BatchNormalization(name=name + "project_bn", **bn)(x)
    if fused and expand == 1:
        x = layers.Activation(activation, name=name + "project_activation")(x)
    if stride == 1 and f_in == f_out:
        if drop > 0:
            x = layers.Dropout(drop, noise_shape=(None, 1, 1, 1), name=name + "drop")(x)
        x = layers.add([x, inputs], name=name + "add")
    return x


def _efficientnet(stages, width, depth, default_size, dropout_rate, name, include_top, weights, input_tensor, input_shape, pooling, classes,
                  classifier_activation, v2, include_preprocessing=True, drop_connect_rate=0.2, activation="swish"):
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, default_size, 32, include_top, weights)
    ax = c.channel_axis()
    bn = {"axis": ax, "momentum": 0.9} if v2 else {"axis": ax}
    min_depth = 8 if v2 else None
    x = img_input
    if not v2:
        x = layers.Rescaling(1.0 / 255.0)(x)
        x = layers.Normalization(axis=ax)(x)
        x = layers.ZeroPadding2D(padding=c.correct_pad(x, 3), name="stem_conv_pad")(x)
        x = layers.Conv2D(_round_filters(32, width), 3, strides=2, padding="valid", use_bias=False, kernel_initializer=_CONV_INIT, name="stem_conv")(x)
    else:
        if include_preprocessing:
            if name.split("-")[-1].startswith("b") and img_input.shape[ax] == 3:
                x = layers.Rescaling(scale=1.0 / 255)(x)
                x = layers.Normalization(mean=[0.485, 0.456, 0.406], variance=[0.229 ** 2, 0.224 ** 2, 0.225 ** 2], axis=ax)(x)
            else:
                x = layers.Rescaling(scale=1.0 / 128.0, offset=-1)(x)
        x = layers.Conv2D(_round_filters(stages[0][2], width, min_depth=min_depth), 3, strides=2, padding="same", use_bias=False,
                          kernel_initializer=_CONV_INIT, name="stem_conv")(x)
    x = layers.BatchNormalization(name="stem_bn", **bn)(x)
    x = layers.Activation(activation, name="stem_activation")(x)
    repeats = [int(math.ceil(depth * s[1])) for s in stages]
    total = float(sum(repeats)) if not v2 else float(sum(s[1] for s in stages))
    b = 0
    for i, ((kernel, _, f_in, f_out, expand, se, stride, fused), n) in enumerate(zip(stages, repeats)):
        f_in = _round_filters(f_in, width, min_depth=min_depth)
        f_out = _round_filters(f_out, width, min_depth=min_depth)
        for j in range(n):
            x = _mbconv(x, f"block{i + 1}{chr(j + 97)}_", f_in if j == 0 else f_out, f_out, kernel, stride if j == 0 else 1, expand, se, fused,
                        drop_connect_rate * b / total, activation, bn, v2)
            b += 1
    x = layers.Conv2D(_round_filters(1280, width, min_depth=min_depth), 1, padding="same", use_bias=False, kernel_initializer=_CONV_INIT, name="top_conv")(x)
    x = layers.BatchNormalization(name="top_bn", **bn)(x)
    x = layers.Activation(activation, name="top_activation")(x)
    dense_kwargs = {"kernel_initializer": _DENSE_INIT}
    if v2:
        dense_kwargs["bias_initializer"] = {"class_name": "Constant", "config": {"value": 0.0}}
    x = c.head(x, include_top, pooling, classes, classifier_activation, weights, dropout=dropout_rate if dropout_rate > 0 else None, **dense_kwargs)
    return c.finish(inputs, x, name, weights)


def _v1(name, width, depth, size, dropout):
    def build(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax",
              name=name.lower()):
        return _efficientnet(_V1_STAGES, width, depth, size, dropout, name, include_top, weights, input_tensor, input_shape, pooling, classes,
                             classifier_activation, v2=False)

    build.__name__ = name
    return keras_export([f"keras.applications.efficientnet.{name}", f"keras.applications.{name}"])(build)


def _v2(name, key, width, depth, size, dropout=0.2):
    def build(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax",
              include_preprocessing=True, name=key):
        return _efficientnet(_V2_STAGES[key], width, depth, size, dropout, name, include_top, weights, input_tensor, input_shape, pooling, classes,
                             classifier_activation, v2=True, include_preprocessing=include_preprocessing)

    build.__name__ = name
    return keras_export([f"keras.applications.efficientnet_v2.{name}", f"keras.applications.{name}"])(build)


EfficientNetB0 = _v1("EfficientNetB0", 1.0, 1.0, 224, 0.2)
EfficientNetB1 = _v1("EfficientNetB1", 1.0, 1.1, 240, 0.2)
EfficientNetB2 = _v1("EfficientNetB2", 1.1, 1.2, 260, 0.3)
EfficientNetB3 = _v1("EfficientNetB3", 1.2, 1.4, 300, 0.3)
EfficientNetB4 = _v1("EfficientNetB4", 1.4, 1.8, 380, 0.4)
EfficientNetB5 = _v1("EfficientNetB5", 1.6, 2.2, 456, 0.4)
EfficientNetB6 = _v1("EfficientNetB6", 1.8, 2.6, 528, 0.5)
EfficientNetB7 = _v1("EfficientNetB7", 2.0, 3.1, 600, 0.5)
EfficientNetV2B0 = _v2("EfficientNetV2B0", "efficientnetv2-b0", 1.0, 1.0, 224)
EfficientNetV2B1 = _v2("EfficientNetV2B1", "efficientnetv2-b1", 1.0, 1.1, 240)
EfficientNetV2B2 = _v2("EfficientNetV2B2", "efficientnetv2-b2", 1.1, 1.2, 260)
EfficientNetV2B3 = _v2("EfficientNetV2B3", "efficientnetv2-b3", 1.2, 1.4, 300)
EfficientNetV2S = _v2("EfficientNetV2S", "efficientnetv2-s", 1.0, 1.0, 384)
EfficientNetV2M = _v2("EfficientNetV2M", "efficientnetv2-m", 1.0, 1.0, 480)
EfficientNetV2L = _v2("EfficientNetV2L", "efficientnetv2-l", 1.0, 1.0, 480)
preprocess_input, decode_predictions = c.preprocess_fn(None, "efficientnet", "efficientnet_v2")
