from keras_b200.layers.preprocessing.image_preprocessing.base import BaseImagePreprocessingLayer  # noqa: F401
from keras_b200.layers.preprocessing.image_preprocessing.image_layers import *  # noqa: F401,F403
