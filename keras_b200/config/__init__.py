"""``keras.config`` namespace."""

from keras_b200.core.config import (  # noqa: F401
    backend, disable_flash_attention, enable_flash_attention, epsilon, floatx, image_data_format, is_flash_attention_enabled,
    is_nnx_enabled, max_epochs, max_steps_per_epoch, set_backend, set_epsilon, set_floatx, set_image_data_format, set_max_epochs,
    set_max_steps_per_epoch,
)
from keras_b200.dtype_policies import dtype_policy, set_dtype_policy  # noqa: F401
from keras_b200.saving.serialization_lib import enable_unsafe_deserialization  # noqa: F401
from keras_b200.utils.io_utils import (  # noqa: F401
    disable_interactive_logging, enable_interactive_logging, is_interactive_logging_enabled,
)
from keras_b200.utils.traceback_utils import (  # noqa: F401
    disable_traceback_filtering, enable_traceback_filtering, is_traceback_filtering_enabled,
)
