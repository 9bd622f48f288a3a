from keras_b200.core.export_registry import keras_export
from keras_b200.layers.input_spec import InputSpec  # noqa: F401
from keras_b200.layers.layer import Layer, _late_bind  # noqa: F401

_late_bind()
from keras_b200.layers.core.input_layer import Input, InputLayer  # noqa: E402,F401
from keras_b200.layers.core.wrapper import Wrapper  # noqa: E402,F401
from keras_b200.layers.core.dense import Dense  # noqa: E402,F401
from keras_b200.layers.core.einsum_dense import EinsumDense  # noqa: E402,F401
from keras_b200.layers.core.embedding import Embedding, ReversibleEmbedding  # noqa: E402,F401
from keras_b200.layers.core.misc import Identity, Lambda, Masking  # noqa: E402,F401
from keras_b200.layers.activations.activation_layers import ELU, Activation, LeakyReLU, PReLU, ReLU, Softmax  # noqa: E402,F401
from keras_b200.layers.convolutional.base_conv import (  # noqa: E402,F401
    Conv1D, Conv1DTranspose, Conv2D, Conv2DTranspose, Conv3D, Conv3DTranspose, DepthwiseConv1D, DepthwiseConv2D,
    SeparableConv1D, SeparableConv2D,
)
from keras_b200.layers.merging.merging_layers import (  # noqa: E402,F401
    Add, Average, Concatenate, Dot, Maximum, Minimum, Multiply, Subtract, add, average, concatenate, dot, maximum, minimum,
    multiply, subtract,
)
from keras_b200.layers.normalization.normalization_layers import (  # noqa: E402,F401
    BatchNormalization, GroupNormalization, LayerNormalization, RMSNormalization, SpectralNormalization, UnitNormalization,
)
from keras_b200.layers.pooling.pooling import (  # noqa: E402,F401
    AdaptiveAveragePooling1D, AdaptiveAveragePooling2D, AdaptiveAveragePooling3D, AdaptiveMaxPooling1D, AdaptiveMaxPooling2D,
    AdaptiveMaxPooling3D, AveragePooling1D, AveragePooling2D, AveragePooling3D, GlobalAveragePooling1D, GlobalAveragePooling2D,
    GlobalAveragePooling3D, GlobalMaxPooling1D, GlobalMaxPooling2D, GlobalMaxPooling3D, MaxPooling1D, MaxPooling2D, MaxPooling3D,
)
from keras_b200.layers.regularization.regularization_layers import (  # noqa: E402,F401
    ActivityRegularization, AlphaDropout, Dropout, GaussianDropout, GaussianNoise, SpatialDropout1D, SpatialDropout2D, SpatialDropout3D,
)
from keras_b200.layers.reshaping.reshaping_layers import (  # noqa: E402,F401
    Cropping1D, Cropping2D, Cropping3D, Flatten, Permute, RepeatVector, Reshape, UpSampling1D, UpSampling2D, UpSampling3D,
    ZeroPadding1D, ZeroPadding2D, ZeroPadding3D,
)

Convolution1D, Convolution2D, Convolution3D = Conv1D, Conv2D, Conv3D
Convolution1DTranspose, Convolution2DTranspose, Convolution3DTranspose = Conv1DTranspose, Conv2DTranspose, Conv3DTranspose
SeparableConvolution1D, SeparableConvolution2D = SeparableConv1D, SeparableConv2D
MaxPool1D, MaxPool2D, MaxPool3D = MaxPooling1D, MaxPooling2D, MaxPooling3D
AvgPool1D, AvgPool2D, AvgPool3D = AveragePooling1D, AveragePooling2D, AveragePooling3D
GlobalMaxPool1D, GlobalMaxPool2D, GlobalMaxPool3D = GlobalMaxPooling1D, GlobalMaxPooling2D, GlobalMaxPooling3D
GlobalAvgPool1D, GlobalAvgPool2D, GlobalAvgPool3D = GlobalAveragePooling1D, GlobalAveragePooling2D, GlobalAveragePooling3D


def _optional(module, names):
    import importlib

    try:
        mod = importlib.import_module(module)
    except ImportError:
        return
    for n in names:
        if hasattr(mod, n):
            globals()[n] = getattr(mod, n)


_optional("keras_b200.layers.attention.attention_layers", ["MultiHeadAttention", "GroupedQueryAttention", "GroupQueryAttention", "Attention", "AdditiveAttention"])
_optional("keras_b200.layers.rnn.rnn_layers", ["RNN", "SimpleRNN", "SimpleRNNCell", "LSTM", "LSTMCell", "GRU", "GRUCell", "StackedRNNCells", "Bidirectional", "TimeDistributed", "ConvLSTM1D", "ConvLSTM2D", "ConvLSTM3D"])
_optional("keras_b200.layers.core.torch_module_wrapper", ["TorchModuleWrapper"])
_optional("keras_b200.layers.core.ternary_dense", ["TernaryDense"])
_optional("keras_b200.layers.core.bridge_layers", ["JaxLayer", "FlaxLayer", "TFSMLayer"])
_optional("keras_b200.layers.preprocessing", ["DataLayer", "CategoryEncoding", "Discretization", "HashedCrossing", "Hashing", "MelSpectrogram",
                                               "Normalization", "Pipeline", "Rescaling", "STFTSpectrogram", "IndexLookup", "IntegerLookup",
                                               "StringLookup", "TextVectorization", "AugMix", "AutoContrast", "CenterCrop",
                                               "ContrastLimitedAdaptiveHistogramEqualization", "CutMix", "Equalization", "MaxNumBoundingBoxes",
                                               "MixUp", "RandAugment", "RandomBrightness", "RandomColorDegeneration", "RandomColorJitter",
                                               "RandomContrast", "RandomCrop", "RandomElasticTransform", "RandomErasing", "RandomFlip",
                                               "RandomGaussianBlur", "RandomGrayscale", "RandomHue", "RandomInvert", "RandomPerspective",
                                               "RandomPosterization", "RandomRotation", "RandomSaturation", "RandomSharpness", "RandomShear",
                                               "RandomTranslation", "RandomZoom", "Resizing", "Solarization"])


@keras_export("keras.layers.serialize")
def serialize(layer):
    """Config dict of a layer (keras/src/layers/__init__.py)."""
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(layer)


@keras_export("keras.layers.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    obj = serialization_lib.deserialize_keras_object(config, custom_objects=custom_objects)
    if not isinstance(obj, Layer):
        raise ValueError(f"`keras.layers.deserialize` was passed a `config` object that is not a `keras.layers.Layer`. Received: {config}")
    return obj
