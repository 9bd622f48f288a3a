from keras_b200.applications import imagenet_utils, resnet  # noqa: F401
from keras_b200.applications.resnet import ResNet50, ResNet50V2, ResNet101, ResNet101V2, ResNet152, ResNet152V2  # noqa: F401

resnet50 = resnet
resnet_v2 = resnet
