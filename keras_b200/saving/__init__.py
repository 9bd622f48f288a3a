from keras_b200.saving.object_registration import (  # noqa: F401
    CustomObjectScope, custom_object_scope, get_custom_objects, get_registered_name, get_registered_object, register_keras_serializable,
)
from keras_b200.saving.saving_api import load_model, load_weights, save_model, save_weights  # noqa: F401
from keras_b200.saving.serialization_lib import deserialize_keras_object, serialize_keras_object  # noqa: F401

from keras_b200.saving.file_editor import KerasFileEditor  # noqa: F401,E402
