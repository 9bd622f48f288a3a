from keras_b200.layers.preprocessing.data_layer import DataLayer  # noqa: F401
from keras_b200.layers.preprocessing.numerical import (  # noqa: F401
    CategoryEncoding, Discretization, HashedCrossing, Hashing, MelSpectrogram, Normalization, Pipeline, Rescaling, STFTSpectrogram,
)
from keras_b200.layers.preprocessing.lookup import IndexLookup, IntegerLookup, StringLookup, TextVectorization  # noqa: F401
