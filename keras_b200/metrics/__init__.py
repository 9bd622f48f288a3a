import inspect

from keras_b200.core.export_registry import keras_export
from keras_b200.core.naming import to_snake_case
from keras_b200.metrics.metric import Metric  # noqa: F401
from keras_b200.metrics.reduction_metrics import Mean, MeanMetricWrapper, Sum  # noqa: F401
from keras_b200.metrics.simple_metrics import *  # noqa: F401,F403
from keras_b200.metrics import simple_metrics as _s
from keras_b200.metrics.confusion_metrics import *  # noqa: F401,F403
from keras_b200.metrics import confusion_metrics as _c
from keras_b200.metrics.extra_metrics import *  # noqa: F401,F403
from keras_b200.metrics import extra_metrics as _e

ALL_OBJECTS = {Metric, Mean, Sum, MeanMetricWrapper}
for _mod in (_s, _c, _e):
    for _n in dir(_mod):
        _o = getattr(_mod, _n)
        if inspect.isclass(_o) and issubclass(_o, Metric) and _o.__module__ == _mod.__name__:
            ALL_OBJECTS.add(_o)
ALL_OBJECTS_DICT = {cls.__name__: cls for cls in ALL_OBJECTS}
ALL_OBJECTS_DICT.update({to_snake_case(cls.__name__): cls for cls in ALL_OBJECTS})
ALL_OBJECTS_DICT.update({
    "bce": _s.BinaryCrossentropy, "BCE": _s.BinaryCrossentropy, "mse": _s.MeanSquaredError, "MSE": _s.MeanSquaredError,
    "mae": _s.MeanAbsoluteError, "MAE": _s.MeanAbsoluteError, "mape": _s.MeanAbsolutePercentageError, "MAPE": _s.MeanAbsolutePercentageError,
    "msle": _s.MeanSquaredLogarithmicError, "MSLE": _s.MeanSquaredLogarithmicError,
    "binary_accuracy": _s.BinaryAccuracy, "categorical_accuracy": _s.CategoricalAccuracy,
    "sparse_categorical_accuracy": _s.SparseCategoricalAccuracy, "top_k_categorical_accuracy": _s.TopKCategoricalAccuracy,
    "sparse_top_k_categorical_accuracy": _s.SparseTopKCategoricalAccuracy,
})
from keras_b200.losses.losses import (  # noqa: E402,F401
    binary_crossentropy, binary_focal_crossentropy, categorical_crossentropy, categorical_focal_crossentropy,
    categorical_hinge, hinge, huber, kl_divergence, log_cosh, mean_absolute_error, mean_absolute_percentage_error,
    mean_squared_error, mean_squared_logarithmic_error, poisson, sparse_categorical_crossentropy, squared_hinge,
)


@keras_export("keras.metrics.serialize")
def serialize(metric):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(metric)


@keras_export("keras.metrics.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    return serialization_lib.deserialize_keras_object(config, module_objects=ALL_OBJECTS_DICT, custom_objects=custom_objects)


@keras_export("keras.metrics.get")
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
            if obj is None:
                from keras_b200 import losses

                obj = losses.ALL_OBJECTS_DICT.get(identifier)
    else:
        obj = identifier
    if callable(obj):
        if inspect.isclass(obj):
            obj = obj()
        return obj
    raise ValueError(f"Could not interpret metric identifier: {identifier}")
