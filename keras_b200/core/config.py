"""Framework configuration: floatx, epsilon, image data format, debug caps, switches.

Mirrors the surface of keras/src/backend/config.py:31-460 (``keras.config.*`` and the
``~/.keras/keras.json`` file) for a framework that has exactly one compute layer.  ``backend()``
therefore returns a constant.
"""

import json
import os

from keras_b200.core.export_registry import keras_export

_FLOATX = "float32"
_EPSILON = 1e-7
_IMAGE_DATA_FORMAT = "channels_last"
_BACKEND = "torch"
_MAX_EPOCHS = None
_MAX_STEPS_PER_EPOCH = None
_FLASH_ATTENTION = None
_NNX = False


@keras_export(["keras.config.floatx", "keras.backend.floatx"])
def floatx():
    return _FLOATX


@keras_export(["keras.config.set_floatx", "keras.backend.set_floatx"])
def set_floatx(value):
    global _FLOATX
    allowed = {"bfloat16", "float16", "float32", "float64"}
    if value not in allowed:
        raise ValueError(f"Unknown `floatx` value: {value}. Expected one of {allowed}")
    _FLOATX = str(value)


@keras_export(["keras.config.epsilon", "keras.backend.epsilon"])
def epsilon():
    return _EPSILON


@keras_export(["keras.config.set_epsilon", "keras.backend.set_epsilon"])
def set_epsilon(value):
    global _EPSILON
    _EPSILON = float(value)


@keras_export(["keras.config.image_data_format", "keras.backend.image_data_format"])
def image_data_format():
    return _IMAGE_DATA_FORMAT


@keras_export(["keras.config.set_image_data_format", "keras.backend.set_image_data_format"])
def set_image_data_format(data_format):
    global _IMAGE_DATA_FORMAT
    data_format = str(data_format).lower()
    if data_format not in {"channels_first", "channels_last"}:
        raise ValueError(
            "The `data_format` argument must be one of {'channels_first', 'channels_last'}. "
            f"Received: data_format={data_format}"
        )
    _IMAGE_DATA_FORMAT = data_format


def standardize_data_format(data_format):
    if data_format is None:
        return image_data_format()
    data_format = str(data_format).lower()
    if data_format not in {"channels_first", "channels_last"}:
        raise ValueError(
            "The `data_format` argument must be one of {'channels_first', 'channels_last'}. "
            f"Received: data_format={data_format}"
        )
    return data_format


@keras_export(["keras.config.backend", "keras.backend.backend"])
def backend():
    """Name of the tensor runtime. There is only one; the string is kept for API parity."""
    return _BACKEND


@keras_export("keras.config.set_backend")
def set_backend(name):
    if name != _BACKEND:
        raise ValueError(
            "This framework has a single compute layer (PyTorch tensors + sm_100a kernels); "
            f"`set_backend({name!r})` is not available."
        )


@keras_export("keras.config.enable_flash_attention")
def enable_flash_attention():
    global _FLASH_ATTENTION
    _FLASH_ATTENTION = None


@keras_export("keras.config.disable_flash_attention")
def disable_flash_attention():
    global _FLASH_ATTENTION
    _FLASH_ATTENTION = False


@keras_export("keras.config.is_flash_attention_enabled")
def is_flash_attention_enabled():
    return _FLASH_ATTENTION


@keras_export("keras.config.is_nnx_enabled")
def is_nnx_enabled():
    return _NNX


@keras_export("keras.config.max_epochs")
def max_epochs():
    return _MAX_EPOCHS


@keras_export("keras.config.set_max_epochs")
def set_max_epochs(value):
    global _MAX_EPOCHS
    _MAX_EPOCHS = value


@keras_export("keras.config.max_steps_per_epoch")
def max_steps_per_epoch():
    return _MAX_STEPS_PER_EPOCH


@keras_export("keras.config.set_max_steps_per_epoch")
def set_max_steps_per_epoch(value):
    global _MAX_STEPS_PER_EPOCH
    _MAX_STEPS_PER_EPOCH = value


def keras_home():
    home = os.environ.get("KERAS_HOME")
    if home:
        return home
    base = os.path.expanduser("~")
    if not os.access(base, os.W_OK):
        base = "/tmp"
    return os.path.join(base, ".keras")


def _load_user_config():
    global _MAX_EPOCHS, _MAX_STEPS_PER_EPOCH
    path = os.path.join(keras_home(), "keras.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                cfg = json.load(f)
        except (ValueError, OSError):
            cfg = {}
        if cfg.get("floatx") in {"bfloat16", "float16", "float32", "float64"}:
            set_floatx(cfg["floatx"])
        if "epsilon" in cfg:
            try:
                set_epsilon(cfg["epsilon"])
            except (TypeError, ValueError):
                pass
        if cfg.get("image_data_format") in {"channels_last", "channels_first"}:
            set_image_data_format(cfg["image_data_format"])
    if os.environ.get("KERAS_MAX_EPOCHS"):
        _MAX_EPOCHS = int(os.environ["KERAS_MAX_EPOCHS"])
    if os.environ.get("KERAS_MAX_STEPS_PER_EPOCH"):
        _MAX_STEPS_PER_EPOCH = int(os.environ["KERAS_MAX_STEPS_PER_EPOCH"])


_load_user_config()


# --- framework switches (read once per query; cheap) -------------------------------------

def fused_kernels_enabled():
    """False when ``KERAS_B200_DISABLE_FUSED_KERNELS=1``: every op then runs its library path."""
    return os.environ.get("KERAS_B200_DISABLE_FUSED_KERNELS", "0") != "1"


def comm_mode():
    """``KERAS_B200_COMM`` = ``p2p`` (own kernels over peer memory, default), ``nvls`` or ``nccl``."""
    return os.environ.get("KERAS_B200_COMM", "p2p")
