"""``keras.backend`` namespace (public subset: config getters, ``result_type``, ``clear_session``…)."""

from keras_b200.core.config import (  # noqa: F401
    backend, epsilon, floatx, image_data_format, set_epsilon, set_floatx, set_image_data_format, standardize_data_format,
)
from keras_b200.core.dtypes import result_type, standardize_dtype  # noqa: F401
from keras_b200.core.export_registry import keras_export
from keras_b200.core.global_state import clear_session as _clear_session
from keras_b200.core.keras_tensor import KerasTensor, is_keras_tensor  # noqa: F401
from keras_b200.core.naming import get_uid  # noqa: F401
from keras_b200.core.tensor import (  # noqa: F401
    IS_THREAD_SAFE, cast, compute_output_spec, convert_to_numpy, convert_to_tensor, device_scope, is_tensor, shape,
)
from keras_b200.core.variables import Variable  # noqa: F401


@keras_export(["keras.backend.clear_session", "keras.utils.clear_session"])
def clear_session(free_memory=True):
    _clear_session(free_memory)


@keras_export("keras.backend.is_float_dtype")
def is_float_dtype(dtype):
    dtype = standardize_dtype(dtype)
    return dtype.startswith("float") or dtype.startswith("bfloat")


@keras_export("keras.backend.is_int_dtype")
def is_int_dtype(dtype):
    dtype = standardize_dtype(dtype)
    return dtype.startswith("int") or dtype.startswith("uint")


def backend_name():
    return backend()


def rnn(*args, **kwargs):
    from keras_b200.layers.rnn.rnn_loop import rnn as _rnn

    return _rnn(*args, **kwargs)
