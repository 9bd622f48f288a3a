"""``keras.applications``: reference architectures (random initialisation or weights from a local file)."""

import sys as _sys
import types as _types

from keras_b200.applications import (  # noqa: F401
    convnext, densenet, efficientnet, imagenet_utils, inception, mobilenet, nasnet, resnet, vgg, xception,
)
from keras_b200.applications.convnext import ConvNeXtBase, ConvNeXtLarge, ConvNeXtSmall, ConvNeXtTiny, ConvNeXtXLarge  # noqa: F401
from keras_b200.applications.densenet import DenseNet121, DenseNet169, DenseNet201  # noqa: F401
from keras_b200.applications.efficientnet import (  # noqa: F401
    EfficientNetB0, EfficientNetB1, EfficientNetB2, EfficientNetB3, EfficientNetB4, EfficientNetB5, EfficientNetB6, EfficientNetB7,
    EfficientNetV2B0, EfficientNetV2B1, EfficientNetV2B2, EfficientNetV2B3, EfficientNetV2L, EfficientNetV2M, EfficientNetV2S,
)
from keras_b200.applications.inception import InceptionResNetV2, InceptionV3  # noqa: F401
from keras_b200.applications.mobilenet import MobileNet, MobileNetV2, MobileNetV3Large, MobileNetV3Small  # noqa: F401
from keras_b200.applications.nasnet import NASNetLarge, NASNetMobile  # noqa: F401
from keras_b200.applications.resnet import ResNet50, ResNet50V2, ResNet101, ResNet101V2, ResNet152, ResNet152V2  # noqa: F401
from keras_b200.applications.vgg import VGG16, VGG19  # noqa: F401
from keras_b200.applications.xception import Xception  # noqa: F401


def _alias(name, source, members, preprocess=None, decode=None):
    """Sub-namespace ``keras.applications.<name>`` exposing ``members`` of ``source`` plus its preprocessing pair."""
    mod = _types.ModuleType(f"{__name__}.{name}")
    for m in members:
        setattr(mod, m, getattr(source, m))
    mod.preprocess_input = preprocess or source.preprocess_input
    mod.decode_predictions = decode or source.decode_predictions
    _sys.modules[mod.__name__] = mod
    globals()[name] = mod
    return mod


_alias("vgg16", vgg, ["VGG16"])
_alias("vgg19", vgg, ["VGG19"])
_alias("resnet50", resnet, ["ResNet50"])
_alias("resnet_v2", resnet, ["ResNet50V2", "ResNet101V2", "ResNet152V2"], preprocess=resnet.preprocess_input_v2)
_alias("mobilenet_v2", mobilenet, ["MobileNetV2"])
_alias("mobilenet_v3", mobilenet, ["MobileNetV3Small", "MobileNetV3Large"], mobilenet.preprocess_input_v3, mobilenet.decode_predictions_v3)
_alias("inception_v3", inception, ["InceptionV3"])
_alias("inception_resnet_v2", inception, ["InceptionResNetV2"])
_alias("efficientnet_v2", efficientnet, ["EfficientNetV2B0", "EfficientNetV2B1", "EfficientNetV2B2", "EfficientNetV2B3", "EfficientNetV2S",
                                         "EfficientNetV2M", "EfficientNetV2L"])
