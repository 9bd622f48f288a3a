from keras_b200.utils.io_utils import (  # noqa: F401
    disable_interactive_logging, enable_interactive_logging, is_interactive_logging_enabled,
)
from keras_b200.utils.progbar import Progbar  # noqa: F401
from keras_b200.trainers.data_adapters.adapters import PyDataset  # noqa: F401
from keras_b200.trainers.data_adapters.data_adapter_utils import pack_x_y_sample_weight, unpack_x_y_sample_weight  # noqa: F401
from keras_b200.saving.object_registration import (  # noqa: F401
    CustomObjectScope, custom_object_scope, get_custom_objects, get_registered_name, get_registered_object, register_keras_serializable,
)
from keras_b200.saving.serialization_lib import deserialize_keras_object, serialize_keras_object  # noqa: F401
from keras_b200.core.keras_tensor import is_keras_tensor  # noqa: F401

Sequence = PyDataset


def __getattr__(name):
    import importlib

    if name == "FeatureSpace":
        from keras_b200.layers.preprocessing.feature_space import FeatureSpace

        return FeatureSpace
    if name == "bounding_boxes":
        return importlib.import_module("keras_b200.utils.bounding_boxes")
    if name == "legacy":
        return importlib.import_module("keras_b200.legacy.saving.legacy_serialization_api")
    if name == "clear_session":
        from keras_b200.core.global_state import clear_session

        return clear_session
    if name == "get_source_inputs":
        from keras_b200.ops.operation_utils import get_source_inputs

        return get_source_inputs
    if name == "standardize_dtype":
        from keras_b200.core.dtypes import standardize_dtype

        return standardize_dtype
    for mod in ("keras_b200.utils.misc_utils", "keras_b200.utils.summary_utils", "keras_b200.utils.dataset_utils", "keras_b200.utils.image_utils",
                "keras_b200.utils.file_utils", "keras_b200.utils.config_utils", "keras_b200.utils.model_visualization"):
        try:
            m = importlib.import_module(mod)
        except ImportError:
            continue
        if hasattr(m, name):
            return getattr(m, name)
    raise AttributeError(f"module 'keras_b200.utils' has no attribute {name!r}")
