"""MobileNet v1, v2 and v3 (keras/src/applications/{mobilenet,mobilenet_v2,mobilenet_v3}.py).

v1: depthwise-separable stacks with ReLU6.  v2: inverted residual bottlenecks (expand x6, linear projection).
v3: bottlenecks with squeeze-excite and hard-swish, described here by per-block tables.
"""

from keras_b200 import layers
from keras_b200.applications import _common as c
from keras_b200.applications import imagenet_utils
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export


def _default_size(input_shape, sizes):
    if input_shape is None:
        return 224
    rows, cols = (input_shape[1], input_shape[2]) if config.image_data_format() == "channels_first" else (input_shape[0], input_shape[1])
    return rows if rows == cols and rows in sizes else 224


def _rows(img_input):
    return img_input.shape[2 if config.image_data_format() == "channels_first" else 1]


# -------------------------------------------------------------------------------------------- v1
_V1_BLOCKS = [(64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2), (512, 1), (512, 1), (512, 1), (512, 1), (512, 1), (1024, 2), (1024, 1)]


@keras_export(["keras.applications.mobilenet.MobileNet", "keras.applications.MobileNet"])
def MobileNet(input_shape=None, alpha=1.0, depth_multiplier=1, dropout=1e-3, include_top=True, weights=None, input_tensor=None, pooling=None,
              classes=1000, classifier_activation="softmax", name=None):
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, _default_size(input_shape, (128, 160, 192, 224)), 32, include_top, weights)
    ax = c.channel_axis()
    x = layers.Conv2D(int(32 * alpha), (3, 3), padding="same", use_bias=False, strides=(2, 2), name="conv1")(img_input)
    x = layers.BatchNormalization(axis=ax, name="conv1_bn")(x)
    x = layers.ReLU(6.0, name="conv1_relu")(x)
    for i, (filters, stride) in enumerate(_V1_BLOCKS, start=1):
        if stride == 2:
            x = layers.ZeroPadding2D(((0, 1), (0, 1)), name=f"conv_pad_{i}")(x)
        x = layers.DepthwiseConv2D((3, 3), padding="same" if stride == 1 else "valid", depth_multiplier=depth_multiplier, strides=(stride, stride),
                                   use_bias=False, name=f"conv_dw_{i}")(x)
        x = layers.BatchNormalization(axis=ax, name=f"conv_dw_{i}_bn")(x)
        x = layers.ReLU(6.0, name=f"conv_dw_{i}_relu")(x)
        x = layers.Conv2D(int(filters * alpha), (1, 1), padding="same", use_bias=False, strides=(1, 1), name=f"conv_pw_{i}")(x)
        x = layers.BatchNormalization(axis=ax, name=f"conv_pw_{i}_bn")(x)
        x = layers.ReLU(6.0, name=f"conv_pw_{i}_relu")(x)
    if include_top:
        x = layers.GlobalAveragePooling2D(keepdims=True)(x)
        x = layers.Dropout(dropout, name="dropout")(x)
        x = layers.Conv2D(classes, (1, 1), padding="same", name="conv_preds")(x)
        x = layers.Reshape((classes,), name="reshape_2")(x)
        imagenet_utils.validate_activation(classifier_activation, weights)
        x = layers.Activation(activation=classifier_activation, name="predictions")(x)
    elif pooling == "avg":
        x = layers.GlobalAveragePooling2D()(x)
    elif pooling == "max":
        x = layers.GlobalMaxPooling2D()(x)
    return c.finish(inputs, x, name or f"mobilenet_{alpha:0.2f}_{_rows(img_input)}", weights)


# -------------------------------------------------------------------------------------------- v2
_V2_BLOCKS = [(16, 1, 1, 1), (24, 6, 2, 2), (32, 6, 2, 3), (64, 6, 2, 4), (96, 6, 1, 3), (160, 6, 2, 3), (320, 6, 1, 1)]  # filters, expansion, stride, repeats


def _v2_block(x, expansion, stride, alpha, filters, block_id):
    ax = c.channel_axis()
    in_ch = x.shape[ax]
    out_ch = c.make_divisible(int(filters * alpha), 8)
    inputs = x
    prefix = f"block_{block_id}_" if block_id else "expanded_conv_"
    if block_id:
        x = layers.Conv2D(expansion * in_ch, 1, padding="same", use_bias=False, name=prefix + "expand")(x)
        x = layers.BatchNormalization(axis=ax, epsilon=1e-3, momentum=0.999, name=prefix + "expand_BN")(x)
        x = layers.ReLU(6.0, name=prefix + "expand_relu")(x)
    if stride == 2:
        x = layers.ZeroPadding2D(padding=c.correct_pad(x, 3), name=prefix + "pad")(x)
    x = layers.DepthwiseConv2D(3, strides=stride, use_bias=False, padding="same" if stride == 1 else "valid", name=prefix + "depthwise")(x)
    x = layers.BatchNormalization(axis=ax, epsilon=1e-3, momentum=0.999, name=prefix + "depthwise_BN")(x)
    x = layers.ReLU(6.0, name=prefix + "depthwise_relu")(x)
    x = layers.Conv2D(out_ch, 1, padding="same", use_bias=False, name=prefix + "project")(x)
    x = layers.BatchNormalization(axis=ax, epsilon=1e-3, momentum=0.999, name=prefix + "project_BN")(x)
    if in_ch == out_ch and stride == 1:
        return layers.Add(name=prefix + "add")([inputs, x])
    return x


@keras_export(["keras.applications.mobilenet_v2.MobileNetV2", "keras.applications.MobileNetV2"])
def MobileNetV2(input_shape=None, alpha=1.0, include_top=True, weights=None, input_tensor=None, pooling=None, classes=1000,
                classifier_activation="softmax", name=None):
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, _default_size(input_shape, (96, 128, 160, 192, 224)), 32, include_top, weights)
    ax = c.channel_axis()
    x = layers.Conv2D(c.make_divisible(32 * alpha, 8), 3, strides=(2, 2), padding="same", use_bias=False, name="Conv1")(img_input)
    x = layers.BatchNormalization(axis=ax, epsilon=1e-3, momentum=0.999, name="bn_Conv1")(x)
    x = layers.ReLU(6.0, name="Conv1_relu")(x)
    block_id = 0
    for filters, expansion, stride, repeats in _V2_BLOCKS:
        for r in range(repeats):
            x = _v2_block(x, expansion, stride if r == 0 else 1, alpha, filters, block_id)
            block_id += 1
    last = c.make_divisible(1280 * alpha, 8) if alpha > 1.0 else 1280
    x = layers.Conv2D(last, 1, use_bias=False, name="Conv_1")(x)
    x = layers.BatchNormalization(axis=ax, epsilon=1e-3, momentum=0.999, name="Conv_1_bn")(x)
    x = layers.ReLU(6.0, name="out_relu")(x)
    if include_top:
        x = layers.GlobalAveragePooling2D()(x)
        imagenet_utils.validate_activation(classifier_activation, weights)
        x = layers.Dense(classes, activation=classifier_activation, name="predictions")(x)
    elif pooling == "avg":
        x = layers.GlobalAveragePooling2D()(x)
    elif pooling == "max":
        x = layers.GlobalMaxPooling2D()(x)
    return c.finish(inputs, x, name or f"mobilenetv2_{alpha:0.2f}_{_rows(img_input)}", weights)


# -------------------------------------------------------------------------------------------- v3
# (expansion, filters, kernel [None: 3 or 5 by variant], stride, squeeze-excite?, activation: "re" relu / "hs" variant activation)
_V3_SMALL = [(1, 16, 3, 2, True, "re"), (72.0 / 16, 24, 3, 2, False, "re"), (88.0 / 24, 24, 3, 1, False, "re"), (4, 40, None, 2, True, "hs"),
             (6, 40, None, 1, True, "hs"), (6, 40, None, 1, True, "hs"), (3, 48, None, 1, True, "hs"), (3, 48, None, 1, True, "hs"),
             (6, 96, None, 2, True, "hs"), (6, 96, None, 1, True, "hs"), (6, 96, None, 1, True, "hs")]
_V3_LARGE = [(1, 16, 3, 1, False, "re"), (4, 24, 3, 2, False, "re"), (3, 24, 3, 1, False, "re"), (3, 40, None, 2, True, "re"), (3, 40, None, 1, True, "re"),
             (3, 40, None, 1, True, "re"), (6, 80, 3, 2, False, "hs"), (2.5, 80, 3, 1, False, "hs"), (2.3, 80, 3, 1, False, "hs"), (2.3, 80, 3, 1, False, "hs"),
             (6, 112, 3, 1, True, "hs"), (6, 112, 3, 1, True, "hs"), (6, 160, None, 2, True, "hs"), (6, 160, None, 1, True, "hs"), (6, 160, None, 1, True, "hs")]


def _relu(x):
    return layers.ReLU()(x)


def _hard_swish(x):
    return layers.Activation("hard_swish")(x)


def _hard_sigmoid(x):
    return layers.ReLU(6.0)(x + 3.0) * (1.0 / 6.0)


def _v3_block(x, expansion, filters, kernel, stride, se_ratio, act, block_id):
    ax = c.channel_axis()
    shortcut, in_ch = x, x.shape[ax]
    prefix = f"expanded_conv_{block_id}_" if block_id else "expanded_conv_"
    bn = dict(axis=ax, epsilon=1e-3, momentum=0.999)
    if block_id:
        x = layers.Conv2D(c.make_divisible(in_ch * expansion), 1, padding="same", use_bias=False, name=prefix + "expand")(x)
        x = act(layers.BatchNormalization(name=prefix + "expand_bn", **bn)(x))
    if stride == 2:
        x = layers.ZeroPadding2D(padding=c.correct_pad(x, kernel), name=prefix + "depthwise_pad")(x)
    x = layers.DepthwiseConv2D(kernel, strides=stride, padding="same" if stride == 1 else "valid", use_bias=False, name=prefix + "depthwise")(x)
    x = act(layers.BatchNormalization(name=prefix + "depthwise_bn", **bn)(x))
    if se_ratio:
        ch = c.make_divisible(in_ch * expansion)
        s = layers.GlobalAveragePooling2D(keepdims=True, name=prefix + "squeeze_excite_avg_pool")(x)
        s = layers.Conv2D(c.make_divisible(ch * se_ratio), 1, padding="same", name=prefix + "squeeze_excite_conv")(s)
        s = layers.ReLU(name=prefix + "squeeze_excite_relu")(s)
        s = layers.Conv2D(ch, 1, padding="same", name=prefix + "squeeze_excite_conv_1")(s)
        x = layers.Multiply(name=prefix + "squeeze_excite_mul")([x, _hard_sigmoid(s)])
    x = layers.Conv2D(filters, 1, padding="same", use_bias=False, name=prefix + "project")(x)
    x = layers.BatchNormalization(name=prefix + "project_bn", **bn)(x)
    if stride == 1 and in_ch == filters:
        x = layers.Add(name=prefix + "add")([shortcut, x])
    return x


def _mobilenet_v3(table, last_point_ch, input_shape, alpha, minimalistic, include_top, weights, input_tensor, classes, pooling, dropout_rate,
                  classifier_activation, include_preprocessing, name):
    c.check_weights(weights, include_top, classes)
    if input_shape is None and input_tensor is None:
        input_shape = (None, None, 3) if config.image_data_format() == "channels_last" else (3, None, None)
    if input_tensor is None:
        img_input = inputs = layers.Input(shape=input_shape)
    else:
        img_input, inputs = c.model_input(input_shape, input_tensor, 224, 32, include_top, weights)
    ax = c.channel_axis()
    kernel, act, se = (3, _relu, None) if minimalistic else (5, _hard_swish, 0.25)
    x = img_input
    if include_preprocessing:
        x = layers.Rescaling(scale=1.0 / 127.5, offset=-1.0)(x)
    x = layers.Conv2D(16, kernel_size=3, strides=(2, 2), padding="same", use_bias=False, name="conv")(x)
    x = act(layers.BatchNormalization(axis=ax, epsilon=1e-3, momentum=0.999, name="conv_bn")(x))
    for i, (expansion, filters, k, stride, use_se, a) in enumerate(table):
        x = _v3_block(x, expansion, c.make_divisible(filters * alpha), k or kernel, stride, se if use_se else None, _relu if a == "re" else act, i)
    last_conv_ch = c.make_divisible(x.shape[ax] * 6)
    if alpha > 1.0:
        last_point_ch = c.make_divisible(last_point_ch * alpha)
    x = layers.Conv2D(last_conv_ch, kernel_size=1, padding="same", use_bias=False, name="conv_1")(x)
    x = act(layers.BatchNormalization(axis=ax, epsilon=1e-3, momentum=0.999, name="conv_1_bn")(x))
    if include_top:
        x = layers.GlobalAveragePooling2D(keepdims=True)(x)
        x = act(layers.Conv2D(last_point_ch, kernel_size=1, padding="same", use_bias=True, name="conv_2")(x))
        if dropout_rate > 0:
            x = layers.Dropout(dropout_rate)(x)
        x = layers.Conv2D(classes, kernel_size=1, padding="same", name="logits")(x)
        x = layers.Flatten()(x)
        imagenet_utils.validate_activation(classifier_activation, weights)
        x = layers.Activation(activation=classifier_activation, name="predictions")(x)
    elif pooling == "avg":
        x = layers.GlobalAveragePooling2D(name="avg_pool")(x)
    elif pooling == "max":
        x = layers.GlobalMaxPooling2D(name="max_pool")(x)
    return c.finish(inputs, x, name, weights)


@keras_export("keras.applications.MobileNetV3Small")
def MobileNetV3Small(input_shape=None, alpha=1.0, minimalistic=False, include_top=True, weights=None, input_tensor=None, classes=1000, pooling=None,
                     dropout_rate=0.2, classifier_activation="softmax", include_preprocessing=True, name="MobileNetV3Small"):
    return _mobilenet_v3(_V3_SMALL, 1024, input_shape, alpha, minimalistic, include_top, weights, input_tensor, classes, pooling, dropout_rate,
                         classifier_activation, include_preprocessing, name)


@keras_export("keras.applications.MobileNetV3Large")
def MobileNetV3Large(input_shape=None, alpha=1.0, minimalistic=False, include_top=True, weights=None, input_tensor=None, classes=1000, pooling=None,
                     dropout_rate=0.2, classifier_activation="softmax", include_preprocessing=True, name="MobileNetV3Large"):
    return _mobilenet_v3(_V3_LARGE, 1280, input_shape, alpha, minimalistic, include_top, weights, input_tensor, classes, pooling, dropout_rate,
                         classifier_activation, include_preprocessing, name)


preprocess_input, decode_predictions = c.preprocess_fn("tf", "mobilenet", "mobilenet_v2")
preprocess_input_v3, decode_predictions_v3 = c.preprocess_fn(None, "mobilenet_v3")
