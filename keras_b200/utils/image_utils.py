"""PIL-backed image helpers: ``array_to_img``, ``img_to_array``, ``load_img``, ``save_img``, ``smart_resize``
(keras/src/utils/image_utils.py)."""

import io
import pathlib
import warnings

import numpy as np

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export

try:
    from PIL import Image as pil_image

    try:
        pil_image_resampling = pil_image.Resampling
    except AttributeError:
        pil_image_resampling = pil_image
except ImportError:
    pil_image = None
    pil_image_resampling = None

if pil_image_resampling is not None:
    PIL_INTERPOLATION_METHODS = {
        "nearest": pil_image_resampling.NEAREST, "bilinear": pil_image_resampling.BILINEAR, "bicubic": pil_image_resampling.BICUBIC,
        "hamming": pil_image_resampling.HAMMING, "box": pil_image_resampling.BOX, "lanczos": pil_image_resampling.LANCZOS,
    }
else:
    PIL_INTERPOLATION_METHODS = {}


def _need_pil(fn):
    if pil_image is None:
        raise ImportError(f"Could not import PIL.Image. The use of `{fn}` requires PIL.")


@keras_export(["keras.utils.array_to_img", "keras.preprocessing.image.array_to_img"])
def array_to_img(x, data_format=None, scale=True, dtype=None):
    data_format = config.standardize_data_format(data_format)
    if dtype is None:
        dtype = config.floatx()
    _need_pil("array_to_img")
    x = np.asarray(x, dtype=dtype)
    if x.ndim != 3:
        raise ValueError(f"Expected image array to have rank 3 (single image). Got array with shape: {x.shape}")
    if data_format == "channels_first":
        x = x.transpose(1, 2, 0)
    if scale:
        x = x - np.min(x)
        x_max = np.max(x)
        if x_max != 0:
            x /= x_max
        x *= 255
    if x.shape[2] == 4:
        return pil_image.fromarray(x.astype("uint8"), "RGBA")
    if x.shape[2] == 3:
        return pil_image.fromarray(x.astype("uint8"), "RGB")
    if x.shape[2] == 1:
        if np.max(x) > 255:
            return pil_image.fromarray(x[:, :, 0].astype("int32"), "I")
        return pil_image.fromarray(x[:, :, 0].astype("uint8"), "L")
    raise ValueError(f"Unsupported channel number: {x.shape[2]}")


@keras_export(["keras.utils.img_to_array", "keras.preprocessing.image.img_to_array"])
def img_to_array(img, data_format=None, dtype=None):
    data_format = config.standardize_data_format(data_format)
    if dtype is None:
        dtype = config.floatx()
    x = np.asarray(img, dtype=dtype)
    if len(x.shape) == 3:
        if data_format == "channels_first":
            x = x.transpose(2, 0, 1)
    elif len(x.shape) == 2:
        if data_format == "channels_first":
            x = x.reshape((1, x.shape[0], x.shape[1]))
        else:
            x = x.reshape((x.shape[0], x.shape[1], 1))
    else:
        raise ValueError(f"Unsupported image shape: {x.shape}")
    return x


@keras_export(["keras.utils.save_img", "keras.preprocessing.image.save_img"])
def save_img(path, x, data_format=None, file_format=None, scale=True, **kwargs):
    data_format = config.standardize_data_format(data_format)
    if file_format is None and isinstance(path, (str, pathlib.Path)):
        file_format = pathlib.Path(path).suffix[1:].lower()
    if file_format == "jpg":
        file_format = "jpeg"
    img = array_to_img(x, data_format=data_format, scale=scale)
    if img.mode == "RGBA" and file_format == "jpeg":
        warnings.warn("The JPG format does not support RGBA images, converting to RGB.")
        img = img.convert("RGB")
    img.save(path, format=file_format, **kwargs)


@keras_export(["keras.utils.load_img", "keras.preprocessing.image.load_img"])
def load_img(path, color_mode="rgb", target_size=None, interpolation="nearest", keep_aspect_ratio=False):
    _need_pil("load_img")
    if isinstance(path, io.BytesIO):
        img = pil_image.open(path)
    elif isinstance(path, (pathlib.Path, bytes, str)):
        if isinstance(path, pathlib.Path):
            path = str(path.resolve())
        with open(path, "rb") as f:
            img = pil_image.open(io.BytesIO(f.read()))
    else:
        raise TypeError(f"path should be path-like or io.BytesIO, not {type(path)}")
    if color_mode == "grayscale":
        if img.mode not in ("L", "I;16", "I"):
            img = img.convert("L")
    elif color_mode == "rgba":
        if img.mode != "RGBA":
            img = img.convert("RGBA")
    elif color_mode == "rgb":
        if img.mode != "RGB":
            img = img.convert("RGB")
    else:
        raise ValueError('color_mode must be "grayscale", "rgb", or "rgba"')
    if target_size is not None:
        width_height_tuple = (target_size[1], target_size[0])
        if img.size != width_height_tuple:
            if interpolation not in PIL_INTERPOLATION_METHODS:
                raise ValueError(f"Invalid interpolation method {interpolation} specified. Supported methods are {', '.join(PIL_INTERPOLATION_METHODS.keys())}")
            resample = PIL_INTERPOLATION_METHODS[interpolation]
            if keep_aspect_ratio:
                width, height = img.size
                target_width, target_height = width_height_tuple
                crop_height = (width * target_height) // target_width
                crop_width = (height * target_width) // target_height
                crop_height = min(height, crop_height)
                crop_width = min(width, crop_width)
                crop_box_hstart = (height - crop_height) // 2
                crop_box_wstart = (width - crop_width) // 2
                crop_box = [crop_box_wstart, crop_box_hstart, crop_box_wstart + crop_width, crop_box_hstart + crop_height]
                img = img.resize(width_height_tuple, resample, box=crop_box)
            else:
                img = img.resize(width_height_tuple, resample)
    return img


@keras_export("keras.preprocessing.image.smart_resize")
def smart_resize(x, size, interpolation="bilinear", data_format="channels_last", backend_module=None):
    """Resize without aspect distortion: centre-crop to the target aspect ratio, then resize."""
    from keras_b200 import ops
    from keras_b200.core.tensor import convert_to_numpy, convert_to_tensor

    if len(size) != 2:
        raise ValueError(f"Expected `size` to be a tuple of 2 integers, but got: {size}.")
    img = convert_to_tensor(x)
    if img.ndim not in (3, 4):
        raise ValueError(f"Expected an image array with shape `(height, width, channels)`, or `(batch_size, height, width, channels)`, but got input with incorrect rank, of shape {tuple(img.shape)}.")
    out = ops.image.resize(img, size, interpolation=interpolation, crop_to_aspect_ratio=True, data_format=data_format)
    if isinstance(x, np.ndarray):
        return convert_to_numpy(out)
    return out
