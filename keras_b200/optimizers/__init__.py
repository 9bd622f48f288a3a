from keras_b200.core.export_registry import keras_export
from keras_b200.optimizers import schedules  # noqa: F401
from keras_b200.optimizers.base_optimizer import BaseOptimizer  # noqa: F401
from keras_b200.optimizers.loss_scale_optimizer import LossScaleOptimizer  # noqa: F401
from keras_b200.optimizers.optimizers import (  # noqa: F401
    SGD, Adadelta, Adafactor, Adagrad, Adam, Adamax, AdamW, Ftrl, Lamb, Lion, Muon, Nadam, Optimizer, RMSprop, ScheduleFreeAdamW,
)

from keras_b200.optimizers.multi_optimizer import MultiOptimizer, OptimizerMap  # noqa: F401,E402
from keras_b200.optimizers import legacy  # noqa: F401,E402

ALL_OBJECTS = {MultiOptimizer, Optimizer, Adam, SGD, RMSprop, Adadelta, AdamW, Adagrad, Adamax, Adafactor, Nadam, Ftrl, Lion, Lamb, Muon, ScheduleFreeAdamW, LossScaleOptimizer}
ALL_OBJECTS_DICT = {cls.__name__.lower(): cls for cls in ALL_OBJECTS}


@keras_export("keras.optimizers.serialize")
def serialize(optimizer):
    from keras_b200.saving import serialization_lib

    return serialization_lib.serialize_keras_object(optimizer)


@keras_export("keras.optimizers.deserialize")
def deserialize(config, custom_objects=None):
    from keras_b200.saving import serialization_lib

    if isinstance(config, dict) and config.get("class_name", "").lower() in ALL_OBJECTS_DICT:
        config = dict(config)
        config["class_name"] = config["class_name"].lower()
    return serialization_lib.deserialize_keras_object(config, module_objects=ALL_OBJECTS_DICT, custom_objects=custom_objects)


@keras_export("keras.optimizers.get")
def get(identifier):
    if identifier is None:
        return None
    if isinstance(identifier, dict):
        obj = deserialize(identifier)
    elif isinstance(identifier, str):
        cls = ALL_OBJECTS_DICT.get(identifier.lower())
        if cls is None:
            raise ValueError(f"Could not interpret optimizer identifier: {identifier}")
        obj = cls()
    else:
        obj = identifier
    if isinstance(obj, BaseOptimizer):
        return obj
    raise ValueError(f"Could not interpret optimizer identifier: {identifier}")
