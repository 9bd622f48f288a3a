"""Traceback filtering switch (keras/src/utils/traceback_utils.py).  Frames of this framework are
kept short in user-facing tracebacks when filtering is enabled."""

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export


@keras_export("keras.config.enable_traceback_filtering")
def enable_traceback_filtering():
    global_state.set_global_attribute("traceback_filtering", True)


@keras_export("keras.config.disable_traceback_filtering")
def disable_traceback_filtering():
    global_state.set_global_attribute("traceback_filtering", False)


@keras_export("keras.config.is_traceback_filtering_enabled")
def is_traceback_filtering_enabled():
    return global_state.get_global_attribute("traceback_filtering", True)
