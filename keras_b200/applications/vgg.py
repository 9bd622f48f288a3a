"""VGG16 / VGG19 (keras/src/applications/vgg16.py, vgg19.py): five conv blocks of 3x3 convolutions + 2x2 max-pool,
then ``flatten → fc1(4096) → fc2(4096) → predictions``."""

from keras_b200 import layers
from keras_b200.applications import _common as c
from keras_b200.applications import imagenet_utils
from keras_b200.core.export_registry import keras_export


def _vgg(name, convs_per_block, include_top, weights, input_tensor, input_shape, pooling, classes, classifier_activation):
    c.check_weights(weights, include_top, classes)
    img_input, inputs = c.model_input(input_shape, input_tensor, 224, 32, include_top, weights)
    x = img_input
    for b, (n, f) in enumerate(zip(convs_per_block, (64, 128, 256, 512, 512)), start=1):
        for i in range(1, n + 1):
            x = layers.Conv2D(f, (3, 3), activation="relu", padding="same", name=f"block{b}_conv{i}")(x)
        x = layers.MaxPooling2D((2, 2), strides=(2, 2), name=f"block{b}_pool")(x)
    if include_top:
        x = layers.Flatten(name="flatten")(x)
        x = layers.Dense(4096, activation="relu", name="fc1")(x)
        x = layers.Dense(4096, activation="relu", name="fc2")(x)
        imagenet_utils.validate_activation(classifier_activation, weights)
        x = layers.Dense(classes, activation=classifier_activation, name="predictions")(x)
    elif pooling == "avg":
        x = layers.GlobalAveragePooling2D()(x)
    elif pooling == "max":
        x = layers.GlobalMaxPooling2D()(x)
    return c.finish(inputs, x, name, weights)


@keras_export(["keras.applications.vgg16.VGG16", "keras.applications.VGG16"])
def VGG16(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax", name="vgg16"):
    return _vgg(name, (2, 2, 3, 3, 3), include_top, weights, input_tensor, input_shape, pooling, classes, classifier_activation)


@keras_export(["keras.applications.vgg19.VGG19", "keras.applications.VGG19"])
def VGG19(include_top=True, weights=None, input_tensor=None, input_shape=None, pooling=None, classes=1000, classifier_activation="softmax", name="vgg19"):
    return _vgg(name, (2, 2, 4, 4, 4), include_top, weights, input_tensor, input_shape, pooling, classes, classifier_activation)


preprocess_input, decode_predictions = c.preprocess_fn("caffe", "vgg16", "vgg19")
