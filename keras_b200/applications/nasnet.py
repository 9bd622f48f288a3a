"""NASNet-A Mobile / Large (keras/src/applications/nasnet.py): a stem, then three groups of ``num_blocks`` normal cells
separated by reduction cells.  Each cell combines the current and the previous feature maps through five two-input
blocks; the operands are described here as small tables (``sep5`` = two stacked 5x5 separable convs, etc.)."""

import warnings

from keras_b200 import layers
from keras_b200.applications import _common as c
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export

_BN = dict(momentum=0.9997, epsilon=1e-3)


def _sep(ip, filters, kernel=(3, 3), strides=(1, 1), block_id=None):
    """ReLU → separable conv → BN → ReLU → separable conv → BN."""
    ax = -1 if config.image_data_format() == "channels_last" else 1
    x = layers.Activation("relu")(ip)
    if strides == (2, 2):
        x = layers.ZeroPadding2D(padding=c.correct_pad(x, kernel), name=f"separable_conv_1_pad_{block_id}")(x)
        pad = "valid"
    else:
        pad = "same"
    x = layers.SeparableConv2D(filters, kernel, strides=strides, name=f"separable_conv_1_{block_id}", padding=pad, use_bias=False)(x)
    x = layers.BatchNormalization(axis=ax, name=f"separable_conv_1_bn_{block_id}", **_BN)(x)
    x = layers.Activation("relu")(x)
    x = layers.SeparableConv2D(filters, kernel, name=f"separable_conv_2_{block_id}", padding="same", use_bias=False)(x)
    return layers.BatchNormalization(axis=ax, name=f"separable_conv_2_bn_{block_id}", **_BN)(x)


def _adjust(p, ip, filters, block_id=None):
    """Bring the previous cell's output ``p`` to the spatial size and width of the current input."""
    ax = -1 if config.image_data_format() == "channels_last" else 1
    img_dim = -2 if config.image_data_format() == "channels_last" else 2
    if p is None:
        return ip
    if p.shape[img_dim] != ip.shape[img_dim]:
        p = layers.Activation("relu", name=f"adjust_relu_1_{block_id}")(p)
        p1 = layers.AveragePooling2D((1, 1), strides=(2, 2), padding="valid", name=f"adjust_avg_pool_1_{block_id}")(p)
        p1 = layers.Conv2D(filters // 2, (1, 1), padding="same", use_bias=False, name=f"adjust_conv_1_{block_id}", kernel_initializer="he_normal")(p1)
        p2 = layers.ZeroPadding2D(padding=((0, 1), (0, 1)))(p)
        p2 = layers.Cropping2D(cropping=((1, 0), (1, 0)))(p2)
        p2 = layers.AveragePooling2D((1, 1), strides=(2, 2), padding="valid", name=f"adjust_avg_pool_2_{block_id}")(p2)
        p2 = layers.Conv2D(filters // 2, (1, 1), padding="same", use_bias=False, name=f"adjust_conv_2_{block_id}", kernel_initializer="he_normal")(p2)
        p = layers.concatenate([p1, p2], axis=ax)
        return layers.BatchNormalization(axis=ax, name=f"adjust_bn_{block_id}", **_BN)(p)
    if p.shape[ax] != filters:
        p = layers.Activation("relu")(p)
        p = layers.Conv2D(filters, (1, 1), strides=(1, 1), padding="same", name=f"adjust_conv_projection_{block_id}", use_bias=False,
                          kernel_initializer="he_normal")(p)
        return layers.BatchNormalization(axis=ax, name=f"adjust_bn_{block_id}", **_BN)(p)
    return p


def _squeeze(ip, filters, kind, block_id):
    ax = -1 if config.image_data_format() == "channels_last" else 1
    h = layers.Activation("relu")(ip)
    h = layers.Conv2D(filters, (1, 1), strides=(1, 1), padding="same", name=f"{kind}_conv_1_{block_id}", use_bias=False, kernel_initializer="he_normal")(h)
    return layers.BatchNormalization(axis=ax, name=f"{kind}_bn_1_{block_id}", **_BN)(h)


def _normal_cell(ip, p, filters, block_id):
    ax = -1 if config.image_data_format() == "channels_last" else 1
    p = _adjust(p, ip, filters, block_id)
    h = _squeeze(ip, filters, "normal", block_id)
    avg = lambda t, nm: layers.AveragePooling2D((3, 3), strides=(1, 1), padding="same", name=f"{nm}_{block_id}")(t)
    x1 = layers.add([_sep(h, filters, (5, 5), block_id=f"normal_left1_{block_id}"), _sep(p, filters, block_id=f"normal_right1_{block_id}")],
                    name=f"normal_add_1_{block_id}")
    x2 = layers.add([_sep(p, filters, (5, 5), block_id=f"normal_left2_{block_id}"), _sep(p, filters, (3, 3), block_id=f"normal_right2_{block_id}")],
                    name=f"normal_add_2_{block_id}")
    x3 = layers.add([avg(h, "normal_left3"), p], name=f"normal_add_3_{block_id}")
    x4 = layers.add([avg(p, "normal_left4"), avg(p, "normal_right4")], name=f"normal_add_4_{block_id}")
    x5 = layers.add([_sep(h, filters, block_id=f"normal_left5_{block_id}"), h], name=f"normal_add_5_{block_id}")
    return layers.concatenate([p, x1, x2, x3, x4, x5], axis=ax, name=f"normal_concat_{block_id}"), ip


def _reduction_cell(ip, p, filters, block_id):
    ax = -1 if config.image_data_format() == "channels_last" else 1
    p = _adjust(p, ip, filters, block_id)
    h = _squeeze(ip, filters, "reduction", block_id)
    h3 = layers.ZeroPadding2D(padding=c.correct_pad(h, 3), name=f"reduction_pad_1_{block_id}")(h)
    s2 = (2, 2)
    x1 = layers.add([_sep(h, filters, (5, 5), strides=s2, block_id=f"reduction_left1_{block_id}"),
                     _sep(p, filters, (7, 7), strides=s2, block_id=f"reduction_right1_{block_id}")], name=f"reduction_add_1_{block_id}")
    x2 = layers.add([layers.MaxPooling2D((3, 3), strides=s2, padding="valid", name=f"reduction_left2_{block_id}")(h3),
                     _sep(p, filters, (7, 7), strides=s2, block_id=f"reduction_right2_{block_id}")], name=f"reduction_add_2_{block_id}")
    x3 = layers.add([layers.AveragePooling2D((3, 3), strides=s2, padding="valid", name=f"reduction_left3_{block_id}")(h3),
                     _sep(p, filters, (5, 5), strides=s2, block_id=f"reduction_right3_{block_id}")], name=f"reduction_add3_{block_id}")
    x4 = layers.add([x2, layers.AveragePooling2D((3, 3), strides=(1, 1), padding="same", name=f"reduction_left4_{block_id}")(x1)])
    x5 = layers.add([_sep(x1, filters, (3, 3), block_id=f"reduction_left4_{block_id}"),
                     layers.MaxPooling2D((3, 3), strides=s2, padding="valid", name=f"reduction_right5_{block_id}")(h3)], name=f"reduction_add4_{block_id}")
    return layers.concatenate([x2, x3, x4, x5], axis=ax, name=f"reduction_concat_{block_id}"), ip


def NASNet(input_shape=None, penultimate_filters=4032, num_blocks=6, stem_block_filters=96, skip_reduction=True, filter_multiplier=2, include_top=True,
           weights=None, input_tensor=None, pooling=None, classes=1000, default_size=None, classifier_activation="softmax", name="NASNet"):
    if config.image_data_format() == "channels_first":
        raise ValueError("NASNet does not support the `channels_first` image data format. Switch to `channels_last` by editing your local config file at ~/.keras/keras.json")
    c.check_weights(weights, include_top, classes)
    if isinstance(input_shape, tuple) and None in input_shape and weights == "imagenet":
        raise ValueError(f"When specifying the input shape of a NASNet and loading `ImageNet` weights, the input_shape argument must be static (no None entries). Got: `input_shape={input_shape}`.")
    img_input, inputs = c.model_input(input_shape, input_tensor, default_size or 331, 32, include_top, weights)
    if penultimate_filters % (24 * (filter_multiplier ** 2)) != 0:
        raise ValueError(f"For NASNet-A models, the `penultimate_filters` must be a multiple of 24 * (`filter_multiplier` ** 2). Current value: {penultimate_filters}")
    filters = penultimate_filters // 24
    x = layers.Conv2D(stem_block_filters, (3, 3), strides=(2, 2), padding="valid", use_bias=False, name="stem_conv1", kernel_initializer="he_normal")(img_input)
    x = layers.BatchNormalization(axis=-1, name="stem_bn1", **_BN)(x)
    p = None
    x, p = _reduction_cell(x, p, filters // (filter_multiplier ** 2), block_id="stem_1")
    x, p = _reduction_cell(x, p, filters // filter_multiplier, block_id="stem_2")
    for i in range(num_blocks):
        x, p = _normal_cell(x, p, filters, block_id=f"{i}")
    x, p0 = _reduction_cell(x, p, filters * filter_multiplier, block_id=f"reduce_{num_blocks}")
    p = p0 if not skip_reduction else p
    for i in range(num_blocks):
        x, p = _normal_cell(x, p, filters * filter_multiplier, block_id=f"{num_blocks + i + 1}")
    x, p0 = _reduction_cell(x, p, filters * filter_multiplier ** 2, block_id=f"reduce_{2 * num_blocks}")
    p = p0 if not skip_reduction else p
    for i in range(num_blocks):
        x, p = _normal_cell(x, p, filters * filter_multiplier ** 2, block_id=f"{2 * num_blocks + i + 1}")
    x = layers.Activation("relu")(x)
    if include_top:
        from keras_b200.applications import imagenet_utils

        x = layers.GlobalAveragePooling2D()(x)
        imagenet_utils.validate_activation(classifier_activation, weights)
        x = layers.Dense(classes, activation=classifier_activation, name="predictions")(x)
    elif pooling == "avg":
        x = layers.GlobalAveragePooling2D()(x)
    elif pooling == "max":
        x = layers.GlobalMaxPooling2D()(x)
    return c.finish(inputs, x, name, weights)


@keras_export(["keras.applications.nasnet.NASNetMobile", "keras.applications.NASNetMobile"])
def NASNetMobile(input_shape=None, include_top=True, weights=None, input_tensor=None, pooling=None, classes=1000, classifier_activation="softmax",
                 name="nasnet_mobile"):
    if input_shape is None and input_tensor is None and not include_top:
        warnings.warn("`input_shape` is undefined; the NASNetMobile default of (224, 224, 3) is used.", stacklevel=2)
    return NASNet(input_shape, penultimate_filters=1056, num_blocks=4, stem_block_filters=32, skip_reduction=False, filter_multiplier=2,
                  include_top=include_top, weights=weights, input_tensor=input_tensor, pooling=pooling, classes=classes, default_size=224,
                  classifier_activation=classifier_activation, name=name)


@keras_export(["keras.applications.nasnet.NASNetLarge", "keras.applications.NASNetLarge"])
def NASNetLarge(input_shape=None, include_top=True, weights=None, input_tensor=None, pooling=None, classes=1000, classifier_activation="softmax",
                name="nasnet_large"):
    return NASNet(input_shape, penultimate_filters=4032, num_blocks=6, stem_block_filters=96, skip_reduction=True, filter_multiplier=2,
                  include_top=include_top, weights=weights, input_tensor=input_tensor, pooling=pooling, classes=classes, default_size=331,
                  classifier_activation=classifier_activation, name=name)


preprocess_input, decode_predictions = c.preprocess_fn("tf", "nasnet")
