from keras_b200.layers.preprocessing.data_layer import DataLayer  # noqa: F401
from keras_b200.layers.preprocessing.numerical import (  # noqa: F401
    CategoryEncoding, Discretization, HashedCrossing, Hashing, MelSpectrogram, Normalization, Pipeline, Rescaling, STFTSpectrogram,
)
from keras_b200.layers.preprocessing.lookup import IndexLookup, IntegerLookup, StringLookup, TextVectorization  # noqa: F401
from keras_b200.layers.preprocessing.feature_space import FeatureSpace  # noqa: F401
from keras_b200.layers.preprocessing.image_preprocessing import *  # noqa: F401,F403
from keras_b200.layers.preprocessing.image_preprocessing import BaseImagePreprocessingLayer, image_layers as _il  # noqa: F401

IMAGE_LAYER_NAMES = list(_il.__all__)
