"""Image files and arrays: ``array_to_img``, ``img_to_array``, ``load_img``, ``save_img`` (through Pillow) and
``smart_resize`` (through ``keras.ops.image``).  Public behaviour of keras/src/utils/image_utils.py.

Arrays are ``(height, width, channels)`` or, with ``data_format="channels_first"``, ``(channels, height, width)``.
"""

import io
import os
import pathlib
import warnings

import numpy as np

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export

try:
    from PIL import Image as pil_image
except ImportError:
    pil_image = None

_RESAMPLING_NAMES = ("nearest", "bilinear", "bicubic", "hamming", "box", "lanczos")


def _resampling_table():
    if pil_image is None:
        return {}
    source = getattr(pil_image, "Resampling", pil_image)  # the enum moved between Pillow versions
    return {name: getattr(source, name.upper()) for name in _RESAMPLING_NAMES}


PIL_INTERPOLATION_METHODS = _resampling_table()

# channels -> (Pillow mode, array dtype); one-channel images that exceed 8 bits go to 32-bit integer mode instead
_MODE_OF_CHANNELS = {4: ("RGBA", "uint8"), 3: ("RGB", "uint8"), 1: ("L", "uint8")}
_ACCEPTED_MODES = {"grayscale": ("L", "I;16", "I"), "rgba": ("RGBA",), "rgb": ("RGB",)}


def _pillow(for_what):
    if pil_image is None:
        raise ImportError(f"Could not import PIL.Image. The use of `{for_what}` requires PIL.")
    return pil_image


def _channels_last(x, data_format):
    return x.transpose(1, 2, 0) if data_format == "channels_first" else x


@keras_export(["keras.utils.array_to_img", "keras.preprocessing.image.array_to_img"])
def array_to_img(x, data_format=None, scale=True, dtype=None):
    """One image array -> ``PIL.Image``.  ``scale`` stretches the values to 0..255 first."""
    data_format = config.standardize_data_format(data_format)
    pil = _pillow("array_to_img")
    pixels = np.asarray(x, dtype=dtype or config.floatx())
    if pixels.ndim != 3:
        raise ValueError(f"Expected image array to have rank 3 (single image). Got array with shape: {pixels.shape}")
    pixels = _channels_last(pixels, data_format)
    if scale:
        pixels = pixels - pixels.min()
        peak = pixels.max()
        if peak != 0:
            pixels = pixels / peak
        pixels = pixels * 255
    channels = pixels.shape[2]
    if channels not in _MODE_OF_CHANNELS:
        raise ValueError(f"Unsupported channel number: {channels}")
    mode, storage = _MODE_OF_CHANNELS[channels]
    if channels == 1:
        pixels = pixels[:, :, 0]
        if pixels.max() > 255:
            mode, storage = "I", "int32"
    return pil.fromarray(pixels.astype(storage), mode)


@keras_export(["keras.utils.img_to_array", "keras.preprocessing.image.img_to_array"])
def img_to_array(img, data_format=None, dtype=None):
    """``PIL.Image`` (or anything array-like of rank 2 or 3) -> array with an explicit channel axis."""
    data_format = config.standardize_data_format(data_format)
    pixels = np.asarray(img, dtype=dtype or config.floatx())
    if pixels.ndim == 2:
        pixels = pixels[:, :, None]
    elif pixels.ndim != 3:
        raise ValueError(f"Unsupported image shape: {pixels.shape}")
    return pixels.transpose(2, 0, 1) if data_format == "channels_first" else pixels


@keras_export(["keras.utils.save_img", "keras.preprocessing.image.save_img"])
def save_img(path, x, data_format=None, file_format=None, scale=True, **kwargs):
    """Write an image array to ``path``; the format comes from ``file_format`` or from the file extension."""
    data_format = config.standardize_data_format(data_format)
    if file_format is None and isinstance(path, (str, pathlib.Path)):
        file_format = os.path.splitext(str(path))[1].lstrip(".").lower()
    file_format = {"jpg": "jpeg"}.get(file_format, file_format)
    img = array_to_img(x, data_format=data_format, scale=scale)
    if file_format == "jpeg" and img.mode == "RGBA":
        warnings.warn("The JPG format does not support RGBA images, converting to RGB.")
        img = img.convert("RGB")
    img.save(path, format=file_format, **kwargs)


def _centre_box(width, height, target_width, target_height):
    """Largest centred window of a ``width x height`` image that has the aspect ratio of the target."""
    box_height = min(height, (width * target_height) // target_width)
    box_width = min(width, (height * target_width) // target_height)
    left, top = (width - box_width) // 2, (height - box_height) // 2
    return [left, top, left + box_width, top + box_height]


@keras_export(["keras.utils.load_img", "keras.preprocessing.image.load_img"])
def load_img(path, color_mode="rgb", target_size=None, interpolation="nearest", keep_aspect_ratio=False):
    """Read an image file (a path, or bytes already in a ``BytesIO``) as a ``PIL.Image`` in the requested colour mode,
    optionally resized to ``target_size = (height, width)``."""
    pil = _pillow("load_img")
    if isinstance(path, io.BytesIO):
        img = pil.open(path)
    elif isinstance(path, (pathlib.Path, bytes, str)):
        location = str(path.resolve()) if isinstance(path, pathlib.Path) else path
        with open(location, "rb") as handle:
            img = pil.open(io.BytesIO(handle.read()))  # decoded from memory: the file is closed when this returns
    else:
        raise TypeError(f"path should be path-like or io.BytesIO, not {type(path)}")
    if color_mode not in _ACCEPTED_MODES:
        raise ValueError('color_mode must be "grayscale", "rgb", or "rgba"')
    accepted = _ACCEPTED_MODES[color_mode]
    if img.mode not in accepted:
        img = img.convert(accepted[0])
    if target_size is None:
        return img
    wanted = (target_size[1], target_size[0])  # Pillow sizes are (width, height)
    if img.size == wanted:
        return img
    if interpolation not in PIL_INTERPOLATION_METHODS:
        raise ValueError(f"Invalid interpolation method {interpolation} specified. Supported methods are {', '.join(PIL_INTERPOLATION_METHODS.keys())}")
    box = _centre_box(*img.size, *wanted) if keep_aspect_ratio else None
    return img.resize(wanted, PIL_INTERPOLATION_METHODS[interpolation], box=box)


@keras_export("keras.preprocessing.image.smart_resize")
def smart_resize(x, size, interpolation="bilinear", data_format="channels_last", backend_module=None):
    """Resize without distortion: the largest centred window with the target aspect ratio is cut out, then resized.
    NumPy in, NumPy out; tensors stay tensors."""
    from keras_b200 import ops
    from keras_b200.core.tensor import convert_to_numpy, convert_to_tensor

    if len(size) != 2:
        raise ValueError(f"Expected `size` to be a tuple of 2 integers, but got: {size}.")
    img = convert_to_tensor(x)
    if img.ndim not in (3, 4):
        raise ValueError("Expected an image array with shape `(height, width, channels)`, or `(batch_size, height, width, channels)`, but got "
                         f"input with incorrect rank, of shape {tuple(img.shape)}.")
    resized = ops.image.resize(img, size, interpolation=interpolation, crop_to_aspect_ratio=True, data_format=data_format)
    return convert_to_numpy(resized) if isinstance(x, np.ndarray) else resized
