"""ResNet v1 / v2 architectures (``keras.applications.ResNet50`` …).

Graph follows keras/src/applications/resnet.py:48-428: ``ZeroPadding2D(3)`` → 7×7/2 conv →
BN(eps 1.001e-5) → ReLU → ``ZeroPadding2D(1)`` → 3×3/2 max-pool → bottleneck stacks (stride on the
first 1×1 conv of a stack for v1) → global average pool → softmax ``Dense``.  Layer names match the
reference so weight files interchange.  Pre-trained ImageNet weights cannot be downloaded here
(``weights`` accepts ``None`` or a path to a weights file).
"""

from keras_b200 import layers
from keras_b200.applications import imagenet_utils
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.models.functional import Functional

_BN_EPS = 1.001e-5


def _bn_axis():
    return 3 if config.image_data_format() == "channels_last" else 1


def _block_v1(x, filters, kernel_size=3, stride=1, conv_shortcut=True, name=None):
    axis = _bn_axis()
    if conv_shortcut:
        shortcut = layers.Conv2D(4 * filters, 1, strides=stride, name=name + "_0_conv")(x)
        shortcut = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name=name + "_0_bn")(shortcut)
    else:
        shortcut = x
    y = layers.Conv2D(filters, 1, strides=stride, name=name + "_1_conv")(x)
    y = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name=name + "_1_bn")(y)
    y = layers.Activation("relu", name=name + "_1_relu")(y)
    y = layers.Conv2D(filters, kernel_size, padding="SAME", name=name + "_2_conv")(y)
    y = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name=name + "_2_bn")(y)
    y = layers.Activation("relu", name=name + "_2_relu")(y)
    y = layers.Conv2D(4 * filters, 1, name=name + "_3_conv")(y)
    y = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name=name + "_3_bn")(y)
    y = layers.Add(name=name + "_add")([shortcut, y])
    return layers.Activation("relu", name=name + "_out")(y)


def _stack_v1(x, filters, blocks, stride1=2, name=None):
    x = _block_v1(x, filters, stride=stride1, name=name + "_block1")
    for i in range(2, blocks + 1):
        x = _block_v1(x, filters, conv_shortcut=False, name=f"{name}_block{i}")
    return x


def _block_v2(x, filters, kernel_size=3, stride=1, conv_shortcut=False, name=None):
    axis = _bn_axis()
    preact = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name=name + "_preact_bn")(x)
    preact = layers.Activation("relu", name=name + "_preact_relu")(preact)
    if conv_shortcut:
        shortcut = layers.Conv2D(4 * filters, 1, strides=stride, name=name + "_0_conv")(preact)
    else:
        shortcut = layers.MaxPooling2D(1, strides=stride)(x) if stride > 1 else x
    y = layers.Conv2D(filters, 1, strides=1, use_bias=False, name=name + "_1_conv")(preact)
    y = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name=name + "_1_bn")(y)
    y = layers.Activation("relu", name=name + "_1_relu")(y)
    y = layers.ZeroPadding2D(padding=((1, 1), (1, 1)), name=name + "_2_pad")(y)
    y = layers.Conv2D(filters, kernel_size, strides=stride, use_bias=False, name=name + "_2_conv")(y)
    y = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name=name + "_2_bn")(y)
    y = layers.Activation("relu", name=name + "_2_relu")(y)
    y = layers.Conv2D(4 * filters, 1, name=name + "_3_conv")(y)
    return layers.Add(name=name + "_out")([shortcut, y])


def _stack_v2(x, filters, blocks, stride1=2, name=None):
    x = _block_v2(x, filters, conv_shortcut=True, name=name + "_block1")
    for i in range(2, blocks):
        x = _block_v2(x, filters, name=f"{name}_block{i}")
    return _block_v2(x, filters, stride=stride1, name=f"{name}_block{blocks}")


def ResNet(stack_fn, preact, use_bias, name="resnet", include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None,
           classes=1000, classifier_activation="softmax", weights_name=None):
    if weights == "imagenet":
        raise ValueError("Pre-trained ImageNet weights need a download, which is not available; pass `weights=None` or a file path.")
    if weights is not None:
        import os

        if not os.path.exists(str(weights)):
            raise ValueError(f"The `weights` argument should be either `None` (random initialization) or the path to the weights file to be loaded. Received: weights={weights}")
    input_shape = imagenet_utils.obtain_input_shape(input_shape, default_size=224, min_size=32, data_format=config.image_data_format(),
                                                    require_flatten=include_top, weights=weights)
    if input_tensor is None:
        img_input = layers.Input(shape=input_shape)
    else:
        img_input = input_tensor if hasattr(input_tensor, "_keras_history") else layers.Input(tensor=input_tensor, shape=input_shape)
    axis = _bn_axis()
    x = layers.ZeroPadding2D(padding=((3, 3), (3, 3)), name="conv1_pad")(img_input)
    x = layers.Conv2D(64, 7, strides=2, use_bias=use_bias, name="conv1_conv")(x)
    if not preact:
        x = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name="conv1_bn")(x)
        x = layers.Activation("relu", name="conv1_relu")(x)
    x = layers.ZeroPadding2D(padding=((1, 1), (1, 1)), name="pool1_pad")(x)
    x = layers.MaxPooling2D(3, strides=2, name="pool1_pool")(x)
    x = stack_fn(x)
    if preact:
        x = layers.BatchNormalization(axis=axis, epsilon=_BN_EPS, name="post_bn")(x)
        x = layers.Activation("relu", name="post_relu")(x)
    if include_top:
        x = layers.GlobalAveragePooling2D(name="avg_pool")(x)
        imagenet_utils.validate_activation(classifier_activation, weights)
        x = layers.Dense(classes, activation=classifier_activation, name="predictions")(x)
    elif pooling == "avg":
        x = layers.GlobalAveragePooling2D(name="avg_pool")(x)
    elif pooling == "max":
        x = layers.GlobalMaxPooling2D(name="max_pool")(x)
    model = Functional(img_input, x, name=name)
    if weights is not None:
        model.load_weights(weights)
    return model


def _v1(name, blocks, exports):
    def build(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000,
              classifier_activation="softmax", name=name.lower()):
        def stack_fn(x):
            x = _stack_v1(x, 64, blocks[0], stride1=1, name="conv2")
            x = _stack_v1(x, 128, blocks[1], name="conv3")
            x = _stack_v1(x, 256, blocks[2], name="conv4")
            return _stack_v1(x, 512, blocks[3], name="conv5")

        return ResNet(stack_fn, False, True, name=name, include_top=include_top, weights=weights, input_tensor=input_tensor,
                      input_shape=input_shape, pooling=pooling, classes=classes, classifier_activation=classifier_activation)

    build.__name__ = name
    return keras_export(exports)(build)


def _v2(name, blocks, exports):
    def build(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000,
              classifier_activation="softmax", name=name.lower()):
        def stack_fn(x):
            x = _stack_v2(x, 64, blocks[0], name="conv2")
            x = _stack_v2(x, 128, blocks[1], name="conv3")
            x = _stack_v2(x, 256, blocks[2], name="conv4")
            return _stack_v2(x, 512, blocks[3], stride1=1, name="conv5")

        return ResNet(stack_fn, True, True, name=name, include_top=include_top, weights=weights, input_tensor=input_tensor,
                      input_shape=input_shape, pooling=pooling, classes=classes, classifier_activation=classifier_activation)

    build.__name__ = name
    return keras_export(exports)(build)


ResNet50 = _v1("ResNet50", (3, 4, 6, 3), ["keras.applications.resnet50.ResNet50", "keras.applications.resnet.ResNet50", "keras.applications.ResNet50"])
ResNet101 = _v1("ResNet101", (3, 4, 23, 3), ["keras.applications.resnet.ResNet101", "keras.applications.ResNet101"])
ResNet152 = _v1("ResNet152", (3, 8, 36, 3), ["keras.applications.resnet.ResNet152", "keras.applications.ResNet152"])
ResNet50V2 = _v2("ResNet50V2", (3, 4, 6, 3), ["keras.applications.resnet_v2.ResNet50V2", "keras.applications.ResNet50V2"])
ResNet101V2 = _v2("ResNet101V2", (3, 4, 23, 3), ["keras.applications.resnet_v2.ResNet101V2", "keras.applications.ResNet101V2"])
ResNet152V2 = _v2("ResNet152V2", (3, 8, 36, 3), ["keras.applications.resnet_v2.ResNet152V2", "keras.applications.ResNet152V2"])


@keras_export(["keras.applications.resnet50.preprocess_input", "keras.applications.resnet.preprocess_input"])
def preprocess_input(x, data_format=None):
    return imagenet_utils.preprocess_input(x, data_format=data_format, mode="caffe")


@keras_export(["keras.applications.resnet50.decode_predictions", "keras.applications.resnet.decode_predictions"])
def decode_predictions(preds, top=5):
    return imagenet_utils.decode_predictions(preds, top=top)


@keras_export("keras.applications.resnet_v2.preprocess_input")
def preprocess_input_v2(x, data_format=None):
    return imagenet_utils.preprocess_input(x, data_format=data_format, mode="tf")


@keras_export("keras.applications.resnet_v2.decode_predictions")
def decode_predictions_v2(preds, top=5):
    return imagenet_utils.decode_predictions(preds, top=top)
