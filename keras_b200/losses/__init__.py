import inspect

from keras_b200.core.export_registry import keras_export
from keras_b200.losses.loss import Loss  # noqa: F401
from keras_b200.losses.losses import *  # noqa: F401,F403
from keras_b200.losses import losses as _l
from keras_b200.losses.losses import LossFunctionWrapper  # noqa: F401

ALL_OBJECTS = {
    Loss, LossFunctionWrapper,
    _l.MeanSquaredError, _l.MeanAbsoluteError, _l.MeanAbsolutePercentageError, _l.MeanSquaredLogarithmicError,
    _l.CosineSimilarity, _l.Huber, _l.LogCosh, _l.Hinge, _l.SquaredHinge, _l.CategoricalHinge, _l.KLDivergence, _l.Poisson,
    _l.BinaryCrossentropy, _l.BinaryFocalCrossentropy, _l.CategoricalCrossentropy, _l.CategoricalFocalCrossentropy,
    _l.SparseCategoricalCrossentropy, _l.CTC, _l.Dice, _l.Tversky, _l.Circle, _l.CategoricalGeneralizedCrossEntropy,
    _l.mean_squared_error, _l.mean_absolute_error, _l.mean_absolute_percentage_error, _l.mean_squared_logarithmic_error,
    _l.cosine_similarity, _l.huber, _l.log_cosh, _l.hinge, _l.squared_hinge, _l.categorical_hinge, _l.kl_divergence,
    _l.poisson, _l.binary_crossentropy, _l.binary_focal_crossentropy, _l.categorical_crossentropy,
    _l.categorical_focal_crossentropy, _l.sparse_categorical_crossentropy, _l.ctc, _l.dice, _l.tversky, _l.circle,
    _l.categorical_generalized_cross_entropy,
}
ALL_OBJECTS_DICT = {cls.__name__: cls for cls in ALL_OBJECTS}
ALL_OBJECTS_DICT.update({
    "bce": _l.binary_crossentropy, "BCE": _l.binary_crossentropy, "kld": _l.kl_divergence, "KLD": _l.kl_divergence,
    "mae": _l.mean_absolute_error, "MAE": _l.mean_absolute_error, "mse": _l.mean_squared_error, "MSE": _l.mean_squared_error,
    "mape": _l.mean_absolute_percentage_error, "MAPE": _l.mean_absolute_percentage_error,
    "msle": _l.mean_squared_logarithmic_error, "MSLE": _l.mean_squared_logarithmic_error, "logcosh": _l.log_cosh,
})
mse = MSE = _l.mean_squared_error
mae = MAE = _l.mean_absolute_error
mape = MAPE = _l.mean_absolute_percentage_error
msle = MSLE = _l.mean_squared_logarithmic_error
kld = KLD = _l.kl_divergence
logcosh = _l.log_cosh


@keras_export("keras.losses.serialize")
def serialize(loss):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(loss)


@keras_export("keras.losses.deserialize")
def deserialize(name, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(name, module_objects=ALL_OBJECTS_DICT, custom_objects=custom_objects)


@keras_export("keras.losses.get")
def get(identifier):
    if identifier is None:
        return None
    if isinstance(identifier, dict):
        obj = deserialize(identifier)
    elif isinstance(identifier, str):
        obj = ALL_OBJECTS_DICT.get(identifier, None)
        if obj is None:
            from keras_b200.saving import object_registration

            obj = object_registration.get_registered_object(identifier)
    else:
        obj = identifier
    if callable(obj):
        if inspect.isclass(obj):
            obj = obj()
        return obj
    raise ValueError(f"Could not interpret loss identifier: {identifier}")
