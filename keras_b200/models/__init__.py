from keras_b200.models.functional import Functional  # noqa: F401
from keras_b200.models.model import Model  # noqa: F401
from keras_b200.models.sequential import Sequential  # noqa: F401
from keras_b200.models.cloning import clone_model  # noqa: F401
from keras_b200.saving.saving_api import load_model, save_model  # noqa: F401
from keras_b200.core.export_registry import keras_export as _keras_export  # noqa: E402


@_keras_export("keras.models.model_from_json")
def model_from_json(json_string, custom_objects=None):
    """Instantiate a model from ``Model.to_json()`` output (keras/src/models/model.py:1060-1080)."""
    import json

    from keras_b200.saving import serialization_lib

    model_config = json.loads(json_string)
    return serialization_lib.deserialize_keras_object(model_config, custom_objects=custom_objects)
