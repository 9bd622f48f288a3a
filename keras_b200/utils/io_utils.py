"""Interactive logging switch and message printing (keras/src/utils/io_utils.py:15-113)."""

import sys

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export


@keras_export(["keras.config.enable_interactive_logging", "keras.utils.enable_interactive_logging"])
def enable_interactive_logging():
    global_state.set_global_attribute("interactive_logging", True)


@keras_export(["keras.config.disable_interactive_logging", "keras.utils.disable_interactive_logging"])
def disable_interactive_logging():
    global_state.set_global_attribute("interactive_logging", False)


@keras_export(["keras.config.is_interactive_logging_enabled", "keras.utils.is_interactive_logging_enabled"])
def is_interactive_logging_enabled():
    return global_state.get_global_attribute("interactive_logging", True)


def set_logging_verbosity(level):
    import logging

    valid = {"FATAL": logging.FATAL, "ERROR": logging.ERROR, "WARNING": logging.WARNING, "INFO": logging.INFO, "DEBUG": logging.DEBUG}
    if level not in valid:
        raise ValueError(f"Please pass a valid level for logging verbosity. Expected one of: {set(valid.keys())}. Received: {level}")
    logging.getLogger("keras_b200").setLevel(valid[level])


def print_msg(message, line_break=True):
    message = str(message)
    if is_interactive_logging_enabled():
        message = message + "\n" if line_break else message
        try:
            sys.stdout.write(message)
        except UnicodeEncodeError:
            sys.stdout.write(message.encode("ascii", "ignore").decode())
        sys.stdout.flush()
    else:
        import logging

        logging.getLogger("keras_b200").info(message)


def ask_to_proceed_with_overwrite(filepath):
    overwrite = input(f"[WARNING] {filepath} already exists - overwrite? [y/n]").strip().lower()
    while overwrite not in ("y", "n"):
        overwrite = input('Enter "y" (overwrite) or "n" (cancel).').strip().lower()
    if overwrite == "n":
        return False
    print_msg("[TIP] Next time specify overwrite=True!")
    return True
