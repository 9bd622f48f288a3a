"""Image preprocessing and augmentation layers (keras/src/layers/preprocessing/image_preprocessing/*.py).

Every layer draws per-sample parameters as batched tensors and applies them with batched device ops: geometric
layers build a forward affine / projective map per sample and resample once; colour layers are elementwise.
"""

import math

import torch
import torch.nn.functional as F

from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.layers.preprocessing.image_preprocessing import bounding_boxes as bbx
from keras_b200.layers.preprocessing.image_preprocessing.base import BaseImagePreprocessingLayer
from keras_b200.ops import image as image_ops
from keras_b200.random.seed_generator import SeedGenerator

__all__ = [
    "AugMix", "AutoContrast", "CenterCrop", "ContrastLimitedAdaptiveHistogramEqualization", "CutMix", "Equalization", "MaxNumBoundingBoxes",
    "MixUp", "RandAugment", "RandomBrightness", "RandomColorDegeneration", "RandomColorJitter", "RandomContrast", "RandomCrop",
    "RandomElasticTransform", "RandomErasing", "RandomFlip", "RandomGaussianBlur", "RandomGrayscale", "RandomHue", "RandomInvert",
    "RandomPerspective", "RandomPosterization", "RandomRotation", "RandomSaturation", "RandomSharpness", "RandomShear",
    "RandomTranslation", "RandomZoom", "Resizing", "Solarization",
]


class _Base(BaseImagePreprocessingLayer):
    """Shared plumbing: float cast, ``transform_images`` that honours ``training``."""

    _ALWAYS = False  # deterministic layers run in inference too

    def transform_images(self, images, transformation, training=True):
        images = self._cast(images)
        if training or self._ALWAYS:
            return self._apply(images, transformation)
        return self._inference(images)

    def _cast(self, images):
        images = convert_to_tensor(images)
        td = getattr(torch, self.compute_dtype, torch.float32)
        if not td.is_floating_point:
            td = torch.float32
        return images.to(td) if images.dtype != td else images

    def _apply(self, images, t):
        raise NotImplementedError

    def _inference(self, images):
        return images

    def _seeded(self, seed):
        self.seed = seed
        self.generator = SeedGenerator(seed)

    def _channel_axis(self, ndim=4):
        return ndim - 1 if self.data_format == "channels_last" else ndim - 3

    def _spatial_axes(self, ndim=4):
        return (ndim - 3, ndim - 2) if self.data_format == "channels_last" else (ndim - 2, ndim - 1)

    def _clip(self, x):
        return x.clamp(self.value_range[0], self.value_range[1])

    def _grayscale(self, x):
        return image_ops.rgb_to_grayscale(x, data_format=self.data_format)


def _check_value_range(value_range):
    if not isinstance(value_range, (tuple, list)) or len(value_range) != 2:
        raise ValueError(f"The `value_range` argument should be a list of two numbers. Received: value_range={value_range}")
    return tuple(value_range)


# ------------------------------------------------------------------------------ geometry (fixed)
@keras_export("keras.layers.Resizing")
class Resizing(_Base):
    _USE_BASE_FACTOR = False
    _ALWAYS = True

    def __init__(self, height, width, interpolation="bilinear", crop_to_aspect_ratio=False, pad_to_aspect_ratio=False, fill_mode="constant",
                 fill_value=0.0, antialias=False, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.height, self.width, self.interpolation = height, width, interpolation
        self.crop_to_aspect_ratio, self.pad_to_aspect_ratio = crop_to_aspect_ratio, pad_to_aspect_ratio
        self.fill_mode, self.fill_value, self.antialias = fill_mode, fill_value, bool(antialias)

    def _resize(self, x, interpolation):
        return image_ops.resize(x, (self.height, self.width), interpolation=interpolation, antialias=self.antialias,
                                crop_to_aspect_ratio=self.crop_to_aspect_ratio, pad_to_aspect_ratio=self.pad_to_aspect_ratio,
                                fill_mode=self.fill_mode, fill_value=self.fill_value, data_format=self.data_format)

    def _apply(self, images, t):
        return self._resize(images, self.interpolation)

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        return self._resize(convert_to_tensor(segmentation_masks), "nearest")

    def get_random_transformation(self, data, training=True, seed=None):
        _, h, w = self._batch_hw(self._images_of(data))
        return (h, w)

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        h, w = transformation
        H, W = self.height, self.width
        if self.crop_to_aspect_ratio:
            s = max(H / h, W / w)
            ox, oy = (w * s - W) / 2, (h * s - H) / 2
            fn = lambda b: b * s - torch.tensor([ox, oy, ox, oy], dtype=b.dtype, device=b.device)
        elif self.pad_to_aspect_ratio:
            s = min(H / h, W / w)
            ox, oy = (W - w * s) / 2, (H - h * s) / 2
            fn = lambda b: b * s + torch.tensor([ox, oy, ox, oy], dtype=b.dtype, device=b.device)
        else:
            fn = lambda b: b * torch.tensor([W / w, H / h, W / w, H / h], dtype=b.dtype, device=b.device)
        return self._boxes_io(bounding_boxes, h, w, fn, H, W)

    def compute_output_shape(self, input_shape):
        s = list(input_shape)
        if len(s) == 4:
            if self.data_format == "channels_last":
                s[1], s[2] = self.height, self.width
            else:
                s[2], s[3] = self.height, self.width
        elif self.data_format == "channels_last":
            s[0], s[1] = self.height, self.width
        else:
            s[1], s[2] = self.height, self.width
        return tuple(s)

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"height": self.height, "width": self.width, "interpolation": self.interpolation,
                    "crop_to_aspect_ratio": self.crop_to_aspect_ratio, "pad_to_aspect_ratio": self.pad_to_aspect_ratio,
                    "fill_mode": self.fill_mode, "fill_value": self.fill_value, "antialias": self.antialias})
        return cfg


class _CropBase(_Base):
    _USE_BASE_FACTOR = False
    _ALWAYS = True

    def _crop(self, x, top, left):
        """Crop ``[B,...]`` with scalar or per-sample offsets; falls back to an aspect-preserving resize when the
        image is smaller than the target."""
        _, h, w = self._batch_hw(x)
        if h < self.height or w < self.width:
            return image_ops.resize(x, (self.height, self.width), crop_to_aspect_ratio=True, data_format=self.data_format)
        if isinstance(top, torch.Tensor) and top.numel() > 1:
            rows = []
            for i in range(x.shape[0]):
                rows.append(self._crop(x[i:i + 1], int(top[i]), int(left[i])))
            return torch.cat(rows, dim=0)
        top, left = int(top), int(left)
        if self.data_format == "channels_last":
            return x[:, top:top + self.height, left:left + self.width, :]
        return x[:, :, top:top + self.height, left:left + self.width]

    def compute_output_shape(self, input_shape):
        return Resizing.compute_output_shape(self, input_shape)

    def _box_transform(self, bounding_boxes, h, w, top, left):
        if h < self.height or w < self.width:
            s = max(self.height / h, self.width / w)
            ox, oy = (w * s - self.width) / 2, (h * s - self.height) / 2
            fn = lambda b: b * s - torch.tensor([ox, oy, ox, oy], dtype=b.dtype, device=b.device)
        else:
            def fn(b):
                t = convert_to_tensor(top).to(b.dtype).to(b.device).reshape(-1, 1, 1)
                l = convert_to_tensor(left).to(b.dtype).to(b.device).reshape(-1, 1, 1)
                return b - torch.cat([l, t, l, t], dim=-1)
        return self._boxes_io(bounding_boxes, h, w, fn, self.height, self.width)


@keras_export("keras.layers.CenterCrop")
class CenterCrop(_CropBase):
    def __init__(self, height, width, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.height, self.width = height, width

    def get_random_transformation(self, data, training=True, seed=None):
        _, h, w = self._batch_hw(self._images_of(data))
        return (h, w, max((h - self.height) // 2, 0), max((w - self.width) // 2, 0))

    def _apply(self, images, t):
        return self._crop(images, t[2], t[3])

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        return self._crop(convert_to_tensor(segmentation_masks), transformation[2], transformation[3])

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        h, w, top, left = transformation
        return self._box_transform(bounding_boxes, h, w, top, left)

    def get_config(self):
        return {**super().get_config(), "height": self.height, "width": self.width}


@keras_export("keras.layers.RandomCrop")
class RandomCrop(_CropBase):
    def __init__(self, height, width, seed=None, data_format=None, name=None, **kwargs):
        super().__init__(name=name, data_format=data_format, **kwargs)
        self.height, self.width = height, width
        self._seeded(seed)
        self.supports_masking = False
        self.supports_jit = False

    def get_random_transformation(self, data, training=True, seed=None):
        n, h, w = self._batch_hw(self._images_of(data))
        if training and h > self.height and w > self.width:
            # one window for the whole batch, its corner drawn as two scalars
            # (keras/src/layers/preprocessing/image_preprocessing/random_crop.py:97-116)
            top = self._uniform((), 0.0, float(h - self.height + 1), seed=seed).to(torch.int32).long().clamp(max=h - self.height).cpu().expand(n)
            left = self._uniform((), 0.0, float(w - self.width + 1), seed=seed).to(torch.int32).long().clamp(max=w - self.width).cpu().expand(n)
        else:
            top = torch.full((n,), max((h - self.height) // 2, 0), dtype=torch.long)
            left = torch.full((n,), max((w - self.width) // 2, 0), dtype=torch.long)
        return (h, w, top, left)

    # Outside training the layer passes images, masks and boxes through untouched
    # (keras/src/layers/preprocessing/image_preprocessing/random_crop.py:131-140, 196-280).
    _ALWAYS = False

    def transform_images(self, images, transformation, training=True):
        if not training:
            return convert_to_tensor(images)
        return self._apply(self._cast(images), transformation)

    def _apply(self, images, t):
        return self._crop(images, t[2], t[3])

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        if not training:
            return convert_to_tensor(segmentation_masks)
        return self._crop(convert_to_tensor(segmentation_masks), transformation[2], transformation[3])

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        if not training:
            return bounding_boxes
        h, w, top, left = transformation
        return self._box_transform(bounding_boxes, h, w, top, left)

    def get_config(self):
        return {**super().get_config(), "height": self.height, "width": self.width, "seed": self.seed}


HORIZONTAL, VERTICAL, HORIZONTAL_AND_VERTICAL = "horizontal", "vertical", "horizontal_and_vertical"


@keras_export("keras.layers.RandomFlip")
class RandomFlip(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, mode=HORIZONTAL_AND_VERTICAL, seed=None, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        if mode not in (HORIZONTAL, VERTICAL, HORIZONTAL_AND_VERTICAL):
            raise ValueError(f"RandomFlip layer {self.name} received an unknown mode argument: {mode}")
        self.mode = mode
        self._seeded(seed)
        self.supports_jit = False

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n, h, w = self._batch_hw(images)
        flips = self._uniform((n,), seed=seed) <= 0.5
        flips_v = flips  # one draw decides both directions (keras/src/layers/preprocessing/image_preprocessing/random_flip.py:79-82)
        return {"flips": flips, "flips_v": flips_v, "input_shape": (h, w)}

    def _flip(self, x, t):
        hax, wax = self._spatial_axes(x.ndim)
        fh = self._per_sample(t["flips"].to(x.device), x.ndim)
        fv = self._per_sample(t["flips_v"].to(x.device), x.ndim)
        if self.mode in (HORIZONTAL, HORIZONTAL_AND_VERTICAL):
            x = torch.where(fh, torch.flip(x, dims=(wax,)), x)
        if self.mode in (VERTICAL, HORIZONTAL_AND_VERTICAL):
            x = torch.where(fv, torch.flip(x, dims=(hax,)), x)
        return x

    def _apply(self, images, t):
        return self._flip(images, t)

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        if not training:
            return segmentation_masks
        return self._flip(convert_to_tensor(segmentation_masks), transformation)

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        if not training:
            return bounding_boxes
        h, w = transformation["input_shape"]

        def fn(b):
            fh = transformation["flips"].to(b.device).reshape(-1, 1)
            fv = transformation["flips_v"].to(b.device).reshape(-1, 1)
            x1, y1, x2, y2 = b.unbind(-1)
            if self.mode in (HORIZONTAL, HORIZONTAL_AND_VERTICAL):
                x1, x2 = torch.where(fh, w - x2, x1), torch.where(fh, w - x1, x2)
            if self.mode in (VERTICAL, HORIZONTAL_AND_VERTICAL):
                y1, y2 = torch.where(fv, h - y2, y1), torch.where(fv, h - y1, y2)
            return torch.stack([x1, y1, x2, y2], dim=-1)

        return self._boxes_io(bounding_boxes, h, w, fn)

    def get_config(self):
        return {**super().get_config(), "seed": self.seed, "mode": self.mode}


# --------------------------------------------------------------------------- geometry (resampled)
class _AffineBase(_Base):
    """Random affine layers: ``_params`` returns per-sample (angle°, tx px, ty px, scale_x, scale_y, shear_x°, shear_y°)."""

    _USE_BASE_FACTOR = False

    def _init_sampling(self, fill_mode, interpolation, fill_value, seed):
        if fill_mode not in ("reflect", "wrap", "constant", "nearest"):
            raise NotImplementedError(f"Unknown `fill_mode` {fill_mode}. Expected of one {{'reflect', 'wrap', 'constant', 'nearest'}}.")
        if interpolation not in ("nearest", "bilinear"):
            raise NotImplementedError(f"Unknown `interpolation` {interpolation}. Expected of one {{'nearest', 'bilinear'}}.")
        self.fill_mode, self.interpolation, self.fill_value = fill_mode, interpolation, fill_value
        self._seeded(seed)
        self.supports_jit = False

    def _params(self, n, h, w, seed):
        raise NotImplementedError

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        n, h, w = self._batch_hw(self._images_of(data))
        p = self._params(n, h, w, seed)
        z = torch.zeros(n)
        o = torch.ones(n)
        angle, tx, ty = p.get("angle", z), p.get("tx", z), p.get("ty", z)
        sx, sy = p.get("sx", o), p.get("sy", o)
        shx, shy = p.get("shx", z), p.get("shy", z)
        a0, a1, a2, b0, b1, b2 = self.forward_affine(angle, tx, ty, o, shx, shy, float(h), float(w))
        # anisotropic scale about the centre composes on the left
        cx, cy = 0.5 * (w - 1), 0.5 * (h - 1)
        a0, a1, a2 = sx * a0, sx * a1, sx * (a2 - cx) + cx
        b0, b1, b2 = sy * b0, sy * b1, sy * (b2 - cy) + cy
        return {"forward": (a0, a1, a2, b0, b1, b2), "input_shape": (h, w), **p}

    def _apply(self, images, t):
        return self._apply_affine(images, t["forward"], self.interpolation, self.fill_mode, self.fill_value)

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        if not training:
            return segmentation_masks
        return self._apply_affine(convert_to_tensor(segmentation_masks), transformation["forward"], "nearest", self.fill_mode, self.fill_value)

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        if not training:
            return bounding_boxes
        h, w = transformation["input_shape"]
        return self._boxes_io(bounding_boxes, h, w, lambda b: self._box_hull(b, transformation["forward"]))

    def _sampling_config(self):
        return {"fill_mode": self.fill_mode, "interpolation": self.interpolation, "seed": self.seed, "fill_value": self.fill_value}


@keras_export("keras.layers.RandomRotation")
class RandomRotation(_AffineBase):
    def __init__(self, factor, fill_mode="reflect", interpolation="bilinear", seed=None, fill_value=0.0, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.factor = self._check_factor(factor, (-1, 1))
        self._factor_arg = factor
        self._init_sampling(fill_mode, interpolation, fill_value, seed)

    def _params(self, n, h, w, seed):
        lo, hi = self.factor
        return {"angle": self._uniform((n,), lo * 360.0, hi * 360.0, seed=seed).cpu()}

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, **self._sampling_config()}


def _pair_factor(value, name, bounds=(-1, 1)):
    if isinstance(value, (tuple, list)):
        if len(value) != 2:
            raise ValueError(f"`{name}` must be a number or a pair of numbers. Received: {name}={value}")
        lo, hi = sorted(value)
    else:
        lo, hi = -abs(value), abs(value)
    if lo < bounds[0] or hi > bounds[1]:
        raise ValueError(f"`{name}` argument must have values between [{bounds[0]}, {bounds[1]}]. Received: {name}={value}")
    return lo, hi


@keras_export("keras.layers.RandomTranslation")
class RandomTranslation(_AffineBase):
    def __init__(self, height_factor, width_factor, fill_mode="reflect", interpolation="bilinear", seed=None, fill_value=0.0, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.height_factor, self.width_factor = height_factor, width_factor
        self.height_lower, self.height_upper = _pair_factor(height_factor, "height_factor")
        self.width_lower, self.width_upper = _pair_factor(width_factor, "width_factor")
        self._init_sampling(fill_mode, interpolation, fill_value, seed)

    def _params(self, n, h, w, seed):
        ty = self._uniform((n,), self.height_lower, self.height_upper, seed=seed).cpu() * h
        tx = self._uniform((n,), self.width_lower, self.width_upper, seed=seed).cpu() * w
        return {"tx": tx, "ty": ty}

    def get_config(self):
        return {**super().get_config(), "height_factor": self.height_factor, "width_factor": self.width_factor, **self._sampling_config()}


@keras_export("keras.layers.RandomZoom")
class RandomZoom(_AffineBase):
    def __init__(self, height_factor, width_factor=None, fill_mode="reflect", interpolation="bilinear", seed=None, fill_value=0.0,
                 data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.height_factor, self.width_factor = height_factor, width_factor
        self.height_lower, self.height_upper = _pair_factor(height_factor, "height_factor", (-1.0, 1.0))
        if width_factor is not None:
            self.width_lower, self.width_upper = _pair_factor(width_factor, "width_factor", (-1.0, 1.0))
        self._init_sampling(fill_mode, interpolation, fill_value, seed)

    def _params(self, n, h, w, seed):
        # a positive factor zooms out (content shrinks): forward scale = 1 / (1 + factor)
        zy = 1.0 + self._uniform((n,), self.height_lower, self.height_upper, seed=seed).cpu()
        zx = 1.0 + self._uniform((n,), self.width_lower, self.width_upper, seed=seed).cpu() if self.width_factor is not None else zy
        return {"sx": 1.0 / zx, "sy": 1.0 / zy}

    def get_config(self):
        return {**super().get_config(), "height_factor": self.height_factor, "width_factor": self.width_factor, **self._sampling_config()}


@keras_export("keras.layers.RandomShear")
class RandomShear(_AffineBase):
    def __init__(self, x_factor=0.0, y_factor=0.0, interpolation="bilinear", fill_mode="reflect", fill_value=0.0, data_format=None, seed=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.x_factor = self._shear_factor(x_factor, "x_factor")
        self.y_factor = self._shear_factor(y_factor, "y_factor")
        self._init_sampling(fill_mode, interpolation, fill_value, seed)

    @staticmethod
    def _shear_factor(f, name):
        if isinstance(f, (tuple, list)):
            if len(f) != 2:
                raise ValueError(f"`{name}` must be a pair of numbers. Received: {f}")
            lo, hi = sorted(f)
            if lo < 0 or hi > 1:
                raise ValueError(f"`{name}` must be in the range [0, 1]. Received: {f}")
        else:
            if f < 0 or f > 1:
                raise ValueError(f"`{name}` must be in the range [0, 1]. Received: {f}")
            lo, hi = -abs(f), abs(f)  # a single number draws from (-f, f)
        return lo, hi

    def get_random_transformation(self, data, training=True, seed=None):
        """Output pixel (x, y) reads input pixel (x + sx*y, sy*x + y): a shear about the top-left corner, with one random sign for
        both factors of an image (keras/src/layers/preprocessing/image_preprocessing/random_shear.py:141-225)."""
        if not training:
            return None
        n, h, w = self._batch_hw(self._images_of(data))
        sign = torch.where(self._uniform((n, 1), seed=seed).cpu() > 0.5, -1.0, 1.0)
        shy = self._uniform((n, 1), self.y_factor[0], self.y_factor[1], seed=seed).cpu()
        shx = self._uniform((n, 1), self.x_factor[0], self.x_factor[1], seed=seed).cpu()
        factor = torch.cat([shx, shy], dim=1) * sign
        sx, sy = factor[:, 0], factor[:, 1]
        det = 1.0 - sx * sy
        z = torch.zeros(n)
        forward = (1.0 / det, -sx / det, z, -sy / det, 1.0 / det, z)  # the inverse of the read map
        return {"forward": forward, "input_shape": (h, w), "shear_factor": factor}

    def get_config(self):
        return {**super().get_config(), "x_factor": self.x_factor, "y_factor": self.y_factor, **self._sampling_config()}


@keras_export("keras.layers.RandomPerspective")
class RandomPerspective(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, factor=1.0, scale=1.0, interpolation="bilinear", fill_value=0.0, seed=None, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.factor = self._check_factor(factor, (0, 1))
        if self.factor[0] < 0:
            self.factor = (0.0, self.factor[1])
        if not 0.0 <= scale <= 1.0:
            raise ValueError(f"`scale` must be in the range [0, 1]. Received: scale={scale}")
        self.scale, self.interpolation, self.fill_value = scale, interpolation, fill_value
        self._seeded(seed)
        self.supports_jit = False

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        n, h, w = self._batch_hw(self._images_of(data))
        apply = (self._uniform((n,), seed=seed).cpu() < self._uniform((n,), self.factor[0], self.factor[1], seed=seed).cpu())
        corners = torch.tensor([[0.0, 0.0], [w - 1.0, 0.0], [0.0, h - 1.0], [w - 1.0, h - 1.0]]).expand(n, 4, 2)
        jitter = (self._uniform((n, 4, 2), -0.5, 0.5, seed=seed).cpu() * self.scale) * torch.tensor([float(w), float(h)])
        jitter = jitter * apply.reshape(n, 1, 1)
        return {"start": corners, "end": corners + jitter, "input_shape": (h, w)}

    def _warp(self, x, t, interpolation):
        return image_ops.perspective_transform(x, t["start"].to(x.device), t["end"].to(x.device), interpolation=interpolation,
                                               fill_value=self.fill_value, data_format=self.data_format)

    def _apply(self, images, t):
        return self._warp(images, t, self.interpolation)

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        if not training:
            return segmentation_masks
        return self._warp(convert_to_tensor(segmentation_masks), transformation, "nearest")

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        if not training:
            return bounding_boxes
        h, w = transformation["input_shape"]
        from keras_b200.ops.image import _perspective_coeffs

        def fn(b):
            coeffs = _perspective_coeffs(transformation["start"].to(b.dtype), transformation["end"].to(b.dtype)).to(b.device)  # start -> end
            x1, y1, x2, y2 = b.unbind(-1)
            xs = torch.stack([x1, x2, x1, x2], dim=-1)
            ys = torch.stack([y1, y1, y2, y2], dim=-1)
            c = [coeffs[:, i].reshape(-1, 1, 1) for i in range(8)]
            k = c[6] * xs + c[7] * ys + 1.0
            nx = (c[0] * xs + c[1] * ys + c[2]) / k
            ny = (c[3] * xs + c[4] * ys + c[5]) / k
            return torch.stack([nx.amin(-1), ny.amin(-1), nx.amax(-1), ny.amax(-1)], dim=-1)

        return self._boxes_io(bounding_boxes, h, w, fn)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "scale": self.scale, "interpolation": self.interpolation,
                "fill_value": self.fill_value, "seed": self.seed}


@keras_export("keras.layers.RandomElasticTransform")
class RandomElasticTransform(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, factor=1.0, scale=1.0, interpolation="bilinear", fill_mode="reflect", fill_value=0.0, value_range=(0, 255), seed=None,
                 data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.factor = self._check_factor(factor, (0, 1))
        if self.factor[0] < 0:
            self.factor = (0.0, self.factor[1])
        self.scale = self._check_factor(scale, (0, float("inf")), "scale") if not isinstance(scale, (int, float)) else (0.0, float(scale))
        self.interpolation, self.fill_mode, self.fill_value = interpolation, fill_mode, fill_value
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)
        self.supports_jit = False

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        n, _, _ = self._batch_hw(self._images_of(data))
        # per image: a probability, then a threshold; one distortion factor for the batch
        # (keras/src/layers/preprocessing/image_preprocessing/random_elastic_transform.py:170-260)
        probability = self._uniform((n,), self.factor[0], self.factor[1], seed=seed)
        apply = self._uniform((n,), seed=seed) < probability
        distortion = float(self._uniform((), self.scale[0], self.scale[1], seed=seed))
        return {"apply_transform": apply, "distortion_factor": distortion, "seed": seed if seed is not None else self._get_seed_generator()}

    def _apply(self, images, t):
        _, h, w = self._batch_hw(images)
        alpha, sigma = max(h, w) * 0.1 * t["distortion_factor"], min(h, w) * 0.05 * t["distortion_factor"]
        out = image_ops.elastic_transform(images, alpha=alpha, sigma=sigma, interpolation=self.interpolation, fill_mode=self.fill_mode,
                                          fill_value=self.fill_value, seed=t["seed"], data_format=self.data_format)
        return self._clip(torch.where(self._per_sample(t["apply_transform"].to(images.device), images.ndim), out, images))

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "scale": self.scale, "interpolation": self.interpolation,
                "fill_mode": self.fill_mode, "fill_value": self.fill_value, "value_range": self.value_range, "seed": self.seed}


# ----------------------------------------------------------------------------------- colour
@keras_export("keras.layers.RandomBrightness")
class RandomBrightness(_Base):
    _FACTOR_BOUNDS = (-1, 1)

    def __init__(self, factor, value_range=(0, 255), seed=None, **kwargs):
        super().__init__(factor=factor, **kwargs)
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        return {"rgb_delta": self._uniform((n,), self.factor[0], self.factor[1], seed=seed) * (self.value_range[1] - self.value_range[0])}

    def _apply(self, images, t):
        d = self._per_sample(t["rgb_delta"].to(images.device).to(images.dtype))
        return self._clip(images + d)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.RandomContrast")
class RandomContrast(_Base):
    _FACTOR_BOUNDS = (0, 1)

    def __init__(self, factor, value_range=(0, 255), seed=None, **kwargs):
        super().__init__(factor=factor, **kwargs)
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def _set_factor(self, factor):
        # the shared rule: a single number f means the range (max(-f, 0), f) = (0, f), so the contrast is only ever raised
        super()._set_factor(factor)
        self.lower, self.upper = self.factor

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        return {"contrast_factor": self._uniform((n,), 1.0 - self.lower, 1.0 + self.upper, seed=seed)}

    def _apply(self, images, t):
        f = self._per_sample(t["contrast_factor"].to(images.device).to(images.dtype))
        mean = images.mean(dim=self._spatial_axes(), keepdim=True)
        return self._clip((images - mean) * f + mean)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "value_range": self.value_range, "seed": self.seed}


class _HSVBase(_Base):
    _FACTOR_BOUNDS = (0, 1)

    def _hsv(self, images):
        x = self._transform_value_range(images, self.value_range, (0, 1))
        return image_ops.rgb_to_hsv(x, data_format=self.data_format)

    def _rgb(self, hsv, dtype):
        x = image_ops.hsv_to_rgb(hsv, data_format=self.data_format).clamp(0, 1)
        return self._transform_value_range(x, (0, 1), self.value_range).to(dtype)

    def _channels(self, hsv):
        ax = self._channel_axis()
        return [hsv.narrow(ax, i, 1) for i in range(3)], ax


@keras_export("keras.layers.RandomSaturation")
class RandomSaturation(_HSVBase):
    """The saturation channel of the images, as they come (no rescaling to 0..1), is multiplied by ``f / (1 - f)`` and clipped to
    ``value_range``; a single number ``f`` draws from ``(-f, f)``
    (keras/src/layers/preprocessing/image_preprocessing/random_saturation.py)."""

    _FACTOR_BOUNDS = (-1, 1)

    def __init__(self, factor, value_range=(0, 255), data_format=None, seed=None, **kwargs):
        super().__init__(factor=factor, data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        f = self._uniform((n,), self.factor[0], self.factor[1], seed=seed)
        return {"factor": f / (1 - f + 1e-7)}

    def _apply(self, images, t):
        (h, s, v), ax = self._channels(image_ops.rgb_to_hsv(images, data_format=self.data_format))
        s = (s * self._per_sample(t["factor"].to(images.device).to(s.dtype))).clamp(self.value_range[0], self.value_range[1])
        return image_ops.hsv_to_rgb(torch.cat([h, s, v], dim=ax), data_format=self.data_format).to(images.dtype)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.RandomHue")
class RandomHue(_HSVBase):
    def __init__(self, factor, value_range=(0, 255), data_format=None, seed=None, **kwargs):
        super().__init__(factor=factor, data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        sign = torch.where(self._uniform((n,), seed=seed) > 0.5, -1.0, 1.0)
        # a factor of 1 turns the hue by half the circle, either way (random_hue.py: ``invert * factor * 0.5``)
        return {"factor": self._uniform((n,), self.factor[0], self.factor[1], seed=seed) * sign * 0.5}

    def _apply(self, images, t):
        (h, s, v), ax = self._channels(self._hsv(images))
        h = h + self._per_sample(t["factor"].to(images.device).to(h.dtype))
        h = torch.where(h > 1.0, h - 1.0, h)
        h = torch.where(h < 0.0, h + 1.0, h)
        return self._rgb(torch.cat([h, s, v], dim=ax), images.dtype)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.RandomColorDegeneration")
class RandomColorDegeneration(_Base):
    _FACTOR_BOUNDS = (-1, 1)  # the shared rule: a single number f draws from (-f, f)

    def __init__(self, factor, value_range=(0, 255), data_format=None, seed=None, **kwargs):
        super().__init__(factor=factor, data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        return self._uniform((n,), self.factor[0], self.factor[1], seed=seed)

    def _apply(self, images, t):
        f = self._per_sample(t.to(images.device).to(images.dtype))
        gray = self._grayscale(images)
        return self._clip(images + (gray - images) * f)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.RandomGrayscale")
class RandomGrayscale(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, factor=0.5, data_format=None, seed=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        if factor < 0 or factor > 1:
            raise ValueError(f"`factor` should be between 0 and 1. Received: factor={factor}")
        self.factor = factor
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        return self._uniform((n,), seed=seed) < self.factor

    def _apply(self, images, t):
        ax = self._channel_axis()
        gray = self._grayscale(images)
        reps = [1] * images.ndim
        reps[ax] = images.shape[ax]
        return torch.where(self._per_sample(t.to(images.device)), gray.repeat(*reps), images)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "seed": self.seed}


@keras_export("keras.layers.RandomInvert")
class RandomInvert(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, factor=1.0, value_range=(0, 255), seed=None, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.factor = self._check_factor(factor, (0, 1))
        if self.factor[0] < 0:
            self.factor = (0.0, self.factor[1])
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        probability = self._uniform((n,), self.factor[0], self.factor[1], seed=seed)  # drawn first, then the threshold
        return self._uniform((n,), seed=seed) < probability

    def _apply(self, images, t):
        inv = self.value_range[1] + self.value_range[0] - images
        return torch.where(self._per_sample(t.to(images.device)), inv, images)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.RandomPosterization")
class RandomPosterization(_Base):
    """Keeps the top ``factor`` bits of every 8-bit channel value.  ``factor`` is a number or a pair in 1..8; a single number f
    means the range (1, f), and a range draws one integer per image, upper bound excluded
    (keras/src/layers/preprocessing/image_preprocessing/random_posterization.py)."""

    _USE_BASE_FACTOR = False
    _FACTOR_BOUNDS = (1, 8)
    _MAX_FACTOR = 8

    def __init__(self, factor, value_range=(0, 255), data_format=None, seed=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self._set_factor(factor)
        self.value_range = tuple(sorted(_check_value_range(value_range)))
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        if self.factor[0] != self.factor[1]:
            from keras_b200 import random

            bits = random.randint((n,), minval=self.factor[0], maxval=self.factor[1], seed=seed if seed is not None else self._get_seed_generator(), dtype="uint8")
        else:
            bits = torch.full((n,), self.factor[0], dtype=torch.uint8)
        return {"shift_factor": self._MAX_FACTOR - bits}

    def _apply(self, images, t):
        x = self._transform_value_range(images, self.value_range, (0, 255)).to(torch.uint8)
        shift = self._per_sample(t["shift_factor"].to(images.device))
        x = torch.bitwise_left_shift(torch.bitwise_right_shift(x, shift), shift)
        return self._transform_value_range(x.to(images.dtype), (0, 255), self.value_range).to(images.dtype)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.Solarization")
class Solarization(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, addition_factor=0.0, threshold_factor=0.0, value_range=(0, 255), seed=None, **kwargs):
        super().__init__(**kwargs)
        self.addition_factor = self._check_factor(addition_factor, (0, 1), "addition_factor") if not isinstance(addition_factor, (int, float)) else (0.0, float(addition_factor))
        self.threshold_factor = self._check_factor(threshold_factor, (0, 1), "threshold_factor") if not isinstance(threshold_factor, (int, float)) else (0.0, float(threshold_factor))
        for nm, v in (("addition_factor", self.addition_factor), ("threshold_factor", self.threshold_factor)):
            if v[0] < 0 or v[1] > 1:
                raise ValueError(f"The `{nm}` argument should be a number (or a list of two numbers) in the range [0, 1]. Received: {nm}={v}")
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        return {"additions": self._uniform((n,), self.addition_factor[0] * 255, self.addition_factor[1] * 255, seed=seed),
                "thresholds": self._uniform((n,), self.threshold_factor[0] * 255, self.threshold_factor[1] * 255, seed=seed)}

    def _apply(self, images, t):
        x = self._transform_value_range(images, self.value_range, (0, 255))
        x = (x + self._per_sample(t["additions"].to(x.device).to(x.dtype))).clamp(0, 255)
        thr = self._per_sample(t["thresholds"].to(x.device).to(x.dtype))
        x = torch.where(x < thr, x, 255 - x)
        return self._transform_value_range(x, (0, 255), self.value_range).to(images.dtype)

    def get_config(self):
        return {**super().get_config(), "value_range": self.value_range, "addition_factor": self.addition_factor,
                "threshold_factor": self.threshold_factor, "seed": self.seed}


def _depthwise_filter(x_bchw, kernel2d, mode="replicate"):
    c = x_bchw.shape[1]
    k = kernel2d.to(x_bchw.dtype).to(x_bchw.device).expand(c, 1, *kernel2d.shape[-2:])
    ph, pw = kernel2d.shape[-2] // 2, kernel2d.shape[-1] // 2
    if mode == "zeros":
        return F.conv2d(x_bchw, k, padding=(ph, pw), groups=c)
    return F.conv2d(F.pad(x_bchw, (pw, pw, ph, ph), mode=mode), k, groups=c)


@keras_export("keras.layers.RandomSharpness")
class RandomSharpness(_Base):
    _FACTOR_BOUNDS = (0, 1)

    def __init__(self, factor, value_range=(0, 255), data_format=None, seed=None, **kwargs):
        super().__init__(factor=factor, data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        return self._uniform((n,), self.factor[0], self.factor[1], seed=seed) * 2.0  # 0: blurred, 1: unchanged, 2: sharpened

    def _apply(self, images, t):
        x = self._to_bchw(images)
        kernel = torch.tensor([[1.0, 1.0, 1.0], [1.0, 5.0, 1.0], [1.0, 1.0, 1.0]]) / 13.0
        blurred = _depthwise_filter(x, kernel, mode="zeros")  # "same" padding with zeros, as the reference's depthwise convolution
        a = t.to(x.device).to(x.dtype).reshape(-1, 1, 1, 1)
        return self._clip(self._from_bchw(blurred + a * (x - blurred)))

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.RandomGaussianBlur")
class RandomGaussianBlur(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, factor=1.0, kernel_size=3, sigma=1.0, value_range=(0, 255), data_format=None, seed=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.factor = self._check_factor(factor, (0, 1))
        if self.factor[0] < 0:
            self.factor = (0.0, self.factor[1])
        self.kernel_size = (kernel_size, kernel_size) if isinstance(kernel_size, int) else tuple(kernel_size)
        self.sigma = (0.0, float(sigma)) if isinstance(sigma, (int, float)) else tuple(sorted(sigma))
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        probability = self._uniform((n,), self.factor[0], self.factor[1], seed=seed)  # drawn first, then the threshold
        apply = self._uniform((n,), seed=seed) < probability
        sigma = self._uniform((2,), self.sigma[0], self.sigma[1], seed=seed) + 1e-6
        return {"apply": apply, "sigma": (float(sigma[0]), float(sigma[1]))}

    def _apply(self, images, t):
        blurred = image_ops.gaussian_blur(images, kernel_size=self.kernel_size, sigma=t["sigma"], data_format=self.data_format)
        return self._clip(torch.where(self._per_sample(t["apply"].to(images.device)), blurred, images))

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "kernel_size": self.kernel_size, "sigma": self.sigma,
                "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.RandomErasing")
class RandomErasing(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, factor=1.0, scale=(0.02, 0.33), fill_value=None, value_range=(0, 255), seed=None, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.factor = self._check_factor(factor, (0, 1))
        if self.factor[0] < 0:
            self.factor = (0.0, self.factor[1])
        self.scale = self._check_factor(scale, (0, 1), "scale") if not isinstance(scale, (int, float)) else (0.0, float(scale))
        self.fill_value = fill_value
        self.value_range = _check_value_range(value_range)
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        n, h, w = self._batch_hw(self._images_of(data))
        apply = self._uniform((n,), seed=seed) < self._uniform((n,), self.factor[0], self.factor[1], seed=seed)
        area = self._uniform((n,), self.scale[0], self.scale[1], seed=seed) * h * w
        log_ratio = self._uniform((n,), math.log(0.3), math.log(1 / 0.3), seed=seed)
        ratio = torch.exp(log_ratio)
        eh = torch.sqrt(area * ratio).round().clamp(1, h)
        ew = torch.sqrt(area / ratio).round().clamp(1, w)
        top = (self._uniform((n,), seed=seed) * (h - eh + 1)).floor()
        left = (self._uniform((n,), seed=seed) * (w - ew + 1)).floor()
        return {"apply": apply, "box": (top, left, eh, ew), "input_shape": (h, w)}

    def _apply(self, images, t):
        h, w = t["input_shape"]
        dev = images.device
        top, left, eh, ew = [v.to(dev).reshape(-1, 1, 1) for v in t["box"]]
        ys = torch.arange(h, device=dev).reshape(1, h, 1)
        xs = torch.arange(w, device=dev).reshape(1, 1, w)
        mask = (ys >= top) & (ys < top + eh) & (xs >= left) & (xs < left + ew) & t["apply"].to(dev).reshape(-1, 1, 1)
        mask = mask.unsqueeze(self._channel_axis())
        if self.fill_value is None:
            fill = self._uniform(tuple(images.shape), self.value_range[0], self.value_range[1], like=images).to(images.dtype)
        else:
            fill = torch.full_like(images, float(self.fill_value))
        return torch.where(mask, fill, images)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "scale": self.scale, "fill_value": self.fill_value,
                "value_range": self.value_range, "seed": self.seed}


@keras_export("keras.layers.AutoContrast")
class AutoContrast(_Base):
    _USE_BASE_FACTOR = False
    _ALWAYS = True

    def __init__(self, value_range=(0, 255), **kwargs):
        super().__init__(**kwargs)
        self.value_range = _check_value_range(value_range)

    def _apply(self, images, t):
        x = self._transform_value_range(images, self.value_range, (0, 255))
        ax = self._spatial_axes()
        lo, hi = x.amin(dim=ax, keepdim=True), x.amax(dim=ax, keepdim=True)
        scale = 255.0 / (hi - lo)
        out = torch.where(torch.isfinite(scale), (x - lo) * scale, x).clamp(0, 255)
        return self._transform_value_range(out, (0, 255), self.value_range).to(images.dtype)

    def get_config(self):
        return {**super().get_config(), "value_range": self.value_range}


@keras_export("keras.layers.Equalization")
class Equalization(_Base):
    """Histogram equalisation of every channel.  As in keras/src/layers/preprocessing/image_preprocessing/equalization.py:88-200
    one histogram is taken per channel over everything else in the tensor (a batch shares it), levels are truncated into bins,
    the look-up table always spans 0..255, and outside training the input passes through."""

    _USE_BASE_FACTOR = False

    def __init__(self, value_range=(0, 255), bins=256, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self.bins = bins

    def transform_images(self, images, transformation, training=True):
        if not training:
            return convert_to_tensor(images)
        return self._apply(self._cast(images), transformation)

    def _equalize_channel(self, channel):
        bins = self.bins
        lo, hi = float(self.value_range[0]), float(self.value_range[1])
        scale = 255.0 / (hi - lo)
        level = channel * scale + (0.0 - lo * scale)
        flat = (level.to(torch.float32) * (bins - 1) / 255.0).to(torch.int32).clamp(0, bins - 1).reshape(-1)
        hist = torch.bincount(flat.long(), minlength=bins)
        if int(torch.count_nonzero(hist)) <= 1:
            out = level
        else:
            cdf = torch.cumsum(hist, dim=0)
            cdf_min = cdf[torch.nonzero(cdf)[0][0]]
            denom = cdf[-1] - cdf_min
            denom = torch.where(denom == 0, torch.ones_like(denom), denom)
            table = torch.clip(torch.round(((cdf - cdf_min) * 255) / denom), 0, 255)
            index = torch.clip(level / 255.0 * (bins - 1), 0, bins - 1).to(torch.int32)
            out = table[index.long()].to(level.dtype)
        back = (hi - lo) / 255.0
        return out * back + (lo - 0.0 * back)

    def _apply(self, images, t):
        axis = -1 if self.data_format == "channels_last" else -3
        planes = [self._equalize_channel(images.select(axis, i)) for i in range(images.shape[axis])]
        return torch.stack(planes, dim=axis).to(images.dtype)

    def get_config(self):
        return {**super().get_config(), "bins": self.bins, "value_range": self.value_range}


@keras_export("keras.layers.ContrastLimitedAdaptiveHistogramEqualization")
class ContrastLimitedAdaptiveHistogramEqualization(_Base):
    """CLAHE with the arithmetic of keras/src/layers/preprocessing/image_preprocessing/clahe.py:116-312: symmetric padding to
    whole tiles, histograms of truncated levels, clipping at ``clip_limit * tile pixels / 256`` with the excess spread
    evenly, a look-up table per tile from its cumulative histogram, and bilinear blending of the four neighbouring tables
    around tile centres.  Applied in training and inference alike."""

    _USE_BASE_FACTOR = False
    _ALWAYS = True

    def __init__(self, value_range=(0, 255), clip_limit=4.0, tile_grid_size=(8, 8), data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self.clip_limit = clip_limit
        self.tile_grid_size = tuple(tile_grid_size)

    def transform_images(self, images, transformation, training=True):
        images = convert_to_tensor(images)
        return self._apply(images, transformation)

    @staticmethod
    def _mirror(n, pad, device):
        """Indices of ``n + pad`` positions that read ``n`` real ones, the tail mirrored about the edge (edge repeated)."""
        idx = torch.arange(n + pad, device=device)
        return torch.where(idx >= n, 2 * n - 1 - idx, idx).clamp(0, n - 1)

    def _apply(self, images, t):
        original = images.dtype
        batched = images.ndim == 4
        x = images if batched else images.unsqueeze(0)
        if self.data_format == "channels_first":
            x = x.permute(0, 2, 3, 1)
        x = self._transform_value_range(x.to(torch.float32), self.value_range, (0, 255))
        B, H, W, C = x.shape
        gh, gw = self.tile_grid_size
        th, tw = -(-H // gh), -(-W // gw)
        ph, pw = th * gh - H, tw * gw - W
        if ph or pw:
            x = x[:, self._mirror(H, ph, x.device)][:, :, self._mirror(W, pw, x.device)]
        Hp, Wp = H + ph, W + pw
        levels = x.to(torch.int32).clamp(0, 255)
        tiles = levels.reshape(B, gh, th, gw, tw, C).permute(0, 1, 3, 5, 2, 4).reshape(B, gh, gw, C, th * tw)
        hist = torch.zeros((B, gh, gw, C, 256), dtype=torch.float32, device=x.device)
        hist.scatter_add_(-1, tiles.long(), torch.ones_like(tiles, dtype=torch.float32))
        if self.clip_limit > 0:
            # the histograms the limit is compared with are integer counts and the limit takes their type: a limit below one
            # clips every bin to zero (keras/src/layers/preprocessing/image_preprocessing/clahe.py:176-190 over
            # keras/src/backend/torch/nn.py:872-886, whose one_hot stays int64)
            limit = float(int(self.clip_limit * (th * tw) / 256.0))
            clipped = hist.clamp(0, limit)
            hist = clipped + (hist - clipped).sum(dim=-1, keepdim=True) / 256.0
        cdf = hist.cumsum(dim=-1)
        lowest = cdf.amin(dim=-1, keepdim=True)
        span = float(th * tw) - lowest
        span = torch.where(span == 0, torch.ones_like(span), span)
        table = ((cdf - lowest) * 255.0 / span).clamp(0, 255)
        # one ring of repeated border tiles, then every pixel blends the tables of the four tile centres around it
        table = torch.cat([table[:, :1], table, table[:, -1:]], dim=1)
        table = torch.cat([table[:, :, :1], table, table[:, :, -1:]], dim=2)
        ys = (torch.arange(Hp, dtype=torch.float32, device=x.device) - th / 2.0) / th + 1.0
        xs = (torch.arange(Wp, dtype=torch.float32, device=x.device) - tw / 2.0) / tw + 1.0
        y0f, x0f = ys.floor(), xs.floor()
        wy, wx = (ys - y0f).reshape(1, Hp, 1, 1), (xs - x0f).reshape(1, 1, Wp, 1)
        y0, y1 = y0f.clamp(0, gh + 1).long(), (y0f + 1).clamp(0, gh + 1).long()
        x0, x1 = x0f.clamp(0, gw + 1).long(), (x0f + 1).clamp(0, gw + 1).long()
        step_c, step_x = 256, 256 * C
        step_y = step_x * (gw + 2)
        step_b = step_y * (gh + 2)
        flat = table.reshape(-1)
        base = (torch.arange(B, device=x.device).reshape(B, 1, 1, 1) * step_b + torch.arange(C, device=x.device).reshape(1, 1, 1, C) * step_c
                + levels.long())

        def look(yi, xi):
            return flat[base + yi.reshape(1, Hp, 1, 1) * step_y + xi.reshape(1, 1, Wp, 1) * step_x]

        upper = look(y0, x0) * (1.0 - wx) + look(y0, x1) * wx
        lower = look(y1, x0) * (1.0 - wx) + look(y1, x1) * wx
        out = (upper * (1.0 - wy) + lower * wy)[:, :H, :W]
        out = self._transform_value_range(out, (0, 255), self.value_range).to(original)
        if self.data_format == "channels_first":
            out = out.permute(0, 3, 1, 2)
        return out if batched else out[0]

    def get_config(self):
        return {**super().get_config(), "value_range": self.value_range, "clip_limit": self.clip_limit, "tile_grid_size": self.tile_grid_size}


# ------------------------------------------------------------------------------ batch mixing
@keras_export("keras.layers.MixUp")
class MixUp(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, alpha=0.2, data_format=None, seed=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.alpha = alpha
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        from keras_b200 import random

        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        perm = random.shuffle(torch.arange(n), seed=seed if seed is not None else self._get_seed_generator()).cpu()
        lam = random.beta((n,), self.alpha, self.alpha, seed=seed if seed is not None else self._get_seed_generator())
        return {"mix_weight": lam, "permutation_order": perm}

    def _apply(self, images, t):
        lam = self._per_sample(t["mix_weight"].to(images.device).to(images.dtype))
        return lam * images + (1 - lam) * images[t["permutation_order"].to(images.device)]

    def transform_labels(self, labels, transformation, training=True):
        if not training:
            return labels
        labels = labels.to(torch.float32) if not labels.dtype.is_floating_point else labels
        lam = self._per_sample(transformation["mix_weight"].to(labels.device).to(labels.dtype), labels.ndim)
        return lam * labels + (1 - lam) * labels[transformation["permutation_order"].to(labels.device)]

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        if not training:
            return bounding_boxes
        perm = transformation["permutation_order"]
        boxes, labels = bounding_boxes["boxes"], bounding_boxes["labels"]
        return {"boxes": torch.cat([boxes, boxes[perm.to(boxes.device)]], dim=1), "labels": torch.cat([labels, labels[perm.to(labels.device)]], dim=1)}

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        if not training:
            return segmentation_masks
        return self._apply(convert_to_tensor(segmentation_masks).to(torch.float32), transformation)

    def get_config(self):
        return {**super().get_config(), "alpha": self.alpha, "seed": self.seed}


@keras_export("keras.layers.CutMix")
class CutMix(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, factor=1.0, seed=None, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.factor = self._check_factor(factor, (0, 1))
        if self.factor[0] < 0:
            self.factor = (0.0, self.factor[1])
        self._seeded(seed)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        from keras_b200 import random

        images = self._images_of(data)
        if len(images.shape) == 3:
            return None
        n, h, w = self._batch_hw(images)
        gen = seed if seed is not None else self._get_seed_generator()
        # The draws, in the reference's order (keras/src/layers/preprocessing/image_preprocessing/cut_mix.py:60-183): a shared
        # Beta parameter, one Beta(alpha, alpha) weight per image, the window's left edge, its top edge, then the partner order.
        alpha = self._uniform((), self.factor[0], self.factor[1], seed=gen) + 1e-6
        mix = random.beta((n,), alpha, alpha, seed=gen).cpu()
        ratio = torch.sqrt(1.0 - mix)
        bw, bh = ratio * w, ratio * h
        x1 = self._uniform((n,), seed=gen).cpu() * (w - bw)
        y1 = self._uniform((n,), seed=gen).cpu() * (h - bh)
        x2, y2 = x1 + bw, y1 + bh
        perm = random.shuffle(torch.arange(n, dtype=torch.int32), seed=gen).cpu().long()
        area = ((y2 - y1) * (x2 - x1)) / float(h * w)
        return {"permutation_order": perm, "box": (y1, y2, x1, x2), "mix_weight": 1.0 - area, "input_shape": (h, w)}

    def _mask(self, t, dev):
        h, w = t["input_shape"]
        y1, y2, x1, x2 = [v.to(dev).reshape(-1, 1, 1) for v in t["box"]]
        ys = torch.arange(h, device=dev, dtype=torch.float32).reshape(1, h, 1)
        xs = torch.arange(w, device=dev, dtype=torch.float32).reshape(1, 1, w)
        return ((ys >= y1) & (ys < y2) & (xs >= x1) & (xs < x2)).unsqueeze(self._channel_axis())

    def _apply(self, images, t):
        return torch.where(self._mask(t, images.device), images[t["permutation_order"].to(images.device)], images)

    def transform_labels(self, labels, transformation, training=True):
        if not training:
            return labels
        labels = labels.to(torch.float32) if not labels.dtype.is_floating_point else labels
        lam = self._per_sample(transformation["mix_weight"].to(labels.device).to(labels.dtype), labels.ndim)
        return lam * labels + (1 - lam) * labels[transformation["permutation_order"].to(labels.device)]

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        if not training:
            return segmentation_masks
        return self._apply(convert_to_tensor(segmentation_masks), transformation)

    def get_config(self):
        return {**super().get_config(), "factor": self.factor, "seed": self.seed}


# ---------------------------------------------------------------------------- policy layers
@keras_export("keras.layers.RandomColorJitter")
class RandomColorJitter(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, value_range=(0, 255), brightness_factor=None, contrast_factor=None, saturation_factor=None, hue_factor=None, seed=None,
                 data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self.brightness_factor, self.contrast_factor = brightness_factor, contrast_factor
        self.saturation_factor, self.hue_factor = saturation_factor, hue_factor
        self._seeded(seed)
        self.random_brightness = RandomBrightness(brightness_factor, value_range=value_range, seed=seed) if brightness_factor is not None else None
        self.random_contrast = RandomContrast(contrast_factor, value_range=value_range, seed=seed) if contrast_factor is not None else None
        self.random_saturation = RandomSaturation(saturation_factor, value_range=value_range, seed=seed, data_format=data_format) if saturation_factor is not None else None
        self.random_hue = RandomHue(hue_factor, value_range=value_range, seed=seed, data_format=data_format) if hue_factor is not None else None

    def build(self, input_shape):
        for lyr in (self.random_brightness, self.random_contrast, self.random_saturation, self.random_hue):
            if lyr is not None:
                lyr.build(input_shape)

    def transform_images(self, images, transformation, training=True):
        images = self._cast(images)
        if training:
            for lyr in (self.random_brightness, self.random_contrast, self.random_saturation, self.random_hue):
                if lyr is not None:
                    # all four adjustments draw from this layer's generator, one after the other
                    t = lyr.get_random_transformation(images, training=True, seed=self._get_seed_generator())
                    images = lyr.transform_images(images, t, training=True)
        return images

    def get_config(self):
        return {**super().get_config(), "value_range": self.value_range, "brightness_factor": self.brightness_factor,
                "contrast_factor": self.contrast_factor, "saturation_factor": self.saturation_factor, "hue_factor": self.hue_factor, "seed": self.seed}


def _policy_layers(value_range, factor, interpolation, seed, data_format, geometric=True):
    """The candidate operations of RandAugment / AugMix, keyed by name."""
    ops = {
        "auto_contrast": AutoContrast(value_range=value_range, data_format=data_format),
        "equalization": Equalization(value_range=value_range, data_format=data_format),
        "random_brightness": RandomBrightness(factor, value_range=value_range, seed=seed, data_format=data_format),
        "random_color_degeneration": RandomColorDegeneration(factor, value_range=value_range, seed=seed, data_format=data_format),
        "random_contrast": RandomContrast(factor, value_range=value_range, seed=seed, data_format=data_format),
        "random_sharpness": RandomSharpness(factor, value_range=value_range, seed=seed, data_format=data_format),
        "random_posterization": RandomPosterization(max(1, int(round(8 - 4 * abs(factor if isinstance(factor, (int, float)) else factor[1])))),
                                                    value_range=value_range, seed=seed, data_format=data_format),
        "solarization": Solarization(addition_factor=factor, threshold_factor=factor, value_range=value_range, seed=seed, data_format=data_format),
    }
    if geometric:
        ops.update({
            "random_shear": RandomShear(x_factor=factor, y_factor=factor, interpolation=interpolation, seed=seed, data_format=data_format),
            "random_translation": RandomTranslation(factor, factor, interpolation=interpolation, seed=seed, data_format=data_format),
            "random_rotation": RandomRotation(factor, interpolation=interpolation, seed=seed, data_format=data_format),
        })
    return ops


@keras_export("keras.layers.RandAugment")
class RandAugment(_Base):
    _USE_BASE_FACTOR = False
    _AUGMENT_LAYERS = ["random_shear", "random_translation", "random_rotation", "random_brightness", "random_color_degeneration",
                       "random_contrast", "random_sharpness", "random_posterization", "solarization", "auto_contrast", "equalization"]

    def __init__(self, value_range=(0, 255), num_ops=2, factor=0.5, interpolation="bilinear", seed=None, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self.num_ops, self.interpolation = num_ops, interpolation
        self.factor = self._check_factor(factor, (0, 1))
        self._factor_arg = factor
        self._seeded(seed)
        self._ops = _policy_layers(value_range, self.factor[1], interpolation, seed, self.data_format)
        for k, v in self._ops.items():
            setattr(self, k, v)

    def build(self, input_shape):
        for lyr in self._ops.values():
            lyr.build(input_shape)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        from keras_b200 import random

        gen = seed if seed is not None else self._get_seed_generator()
        order = random.shuffle(torch.arange(len(self._AUGMENT_LAYERS)), seed=gen).cpu().tolist()[: self.num_ops]
        out = {}
        for i in order:
            name = self._AUGMENT_LAYERS[i]
            out[name] = self._ops[name].get_random_transformation(data, training=training, seed=self._get_seed_generator())
        return out

    def transform_images(self, images, transformation, training=True):
        images = self._cast(images)
        if training:
            for name, t in transformation.items():
                images = self._ops[name].transform_images(images, t, training=True)
        return images

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        if training:
            for name, t in transformation.items():
                lyr = self._ops[name]
                lyr.bounding_box_format = self.bounding_box_format
                bounding_boxes = lyr.transform_bounding_boxes(bounding_boxes, t, training=True)
        return bounding_boxes

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        if training:
            for name, t in transformation.items():
                segmentation_masks = self._ops[name].transform_segmentation_masks(segmentation_masks, t, training=True)
        return segmentation_masks

    def get_config(self):
        return {**super().get_config(), "value_range": self.value_range, "num_ops": self.num_ops, "factor": self._factor_arg,
                "interpolation": self.interpolation, "seed": self.seed}


@keras_export("keras.layers.AugMix")
class AugMix(_Base):
    _USE_BASE_FACTOR = False

    def __init__(self, value_range=(0, 255), num_chains=3, chain_depth=3, factor=0.3, alpha=1.0, all_ops=True, interpolation="bilinear",
                 seed=None, data_format=None, **kwargs):
        super().__init__(data_format=data_format, **kwargs)
        self.value_range = _check_value_range(value_range)
        self.num_chains, self.chain_depth, self.alpha, self.all_ops, self.interpolation = num_chains, chain_depth, alpha, all_ops, interpolation
        self.factor = self._check_factor(factor, (0, 1))
        self._factor_arg = factor
        self._seeded(seed)
        ops = _policy_layers(value_range, self.factor[1], interpolation, seed, self.data_format)
        names = ["auto_contrast", "equalization", "random_posterization", "solarization", "random_rotation", "random_shear", "random_translation"]
        if all_ops:
            names += ["random_brightness", "random_color_degeneration", "random_contrast", "random_sharpness"]
        self._names = names
        self._ops = {n: ops[n] for n in names}
        for k, v in self._ops.items():
            setattr(self, k, v)

    def build(self, input_shape):
        for lyr in self._ops.values():
            lyr.build(input_shape)

    def get_random_transformation(self, data, training=True, seed=None):
        if not training:
            return None
        from keras_b200 import random

        gen = seed if seed is not None else self._get_seed_generator()
        images = self._images_of(data)
        n = images.shape[0] if len(images.shape) == 4 else 1
        g = random.gamma((n, self.num_chains), self.alpha, seed=gen)
        chain_w = g / g.sum(dim=1, keepdim=True)
        mix = random.beta((n,), self.alpha, self.alpha, seed=gen)
        chains = []
        for _ in range(self.num_chains):
            idx = random.randint((self.chain_depth,), 0, len(self._names), seed=gen).cpu().tolist()
            chains.append([self._names[i] for i in idx])
        return {"chain_mixing_weights": chain_w, "weight_sample": mix, "chains": chains}

    def transform_images(self, images, transformation, training=True):
        images = self._cast(images)
        if not training:
            return images
        t = transformation
        cw = t["chain_mixing_weights"].to(images.device).to(images.dtype)
        acc = torch.zeros_like(images)
        for c, chain in enumerate(t["chains"]):
            aug = images
            for name in chain:
                lyr = self._ops[name]
                aug = lyr.transform_images(aug, lyr.get_random_transformation(aug, training=True), training=True)
            acc = acc + self._per_sample(cw[:, c]) * aug
        m = self._per_sample(t["weight_sample"].to(images.device).to(images.dtype))
        return self._clip(m * images + (1 - m) * acc)

    def get_config(self):
        return {**super().get_config(), "value_range": self.value_range, "num_chains": self.num_chains, "chain_depth": self.chain_depth,
                "factor": self._factor_arg, "alpha": self.alpha, "all_ops": self.all_ops, "interpolation": self.interpolation, "seed": self.seed}


@keras_export("keras.layers.MaxNumBoundingBoxes")
class MaxNumBoundingBoxes(_Base):
    _USE_BASE_FACTOR = False
    _ALWAYS = True

    def __init__(self, max_number, fill_value=-1, **kwargs):
        super().__init__(**kwargs)
        self.max_number, self.fill_value = int(max_number), int(fill_value)

    def transform_images(self, images, transformation=None, training=True):
        return convert_to_tensor(images)

    def call(self, data, training=True):
        if isinstance(data, dict) and "bounding_boxes" in data and not self.bounding_box_format:
            self.bounding_box_format = "xyxy"  # the format is irrelevant for padding / truncation
        return super().call(data, training=training)

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        return bbx.densify_bounding_boxes(bounding_boxes, is_batched=True, max_boxes=self.max_number, boxes_default_value=self.fill_value,
                                          labels_default_value=self.fill_value)

    def compute_output_shape(self, input_shape):
        if isinstance(input_shape, dict) and "bounding_boxes" in input_shape:
            out = dict(input_shape)
            bb = dict(input_shape["bounding_boxes"])
            bs, ls = list(bb["boxes"]), list(bb["labels"])
            bs[-2] = self.max_number
            ls[-1] = self.max_number
            bb["boxes"], bb["labels"] = tuple(bs), tuple(ls)
            out["bounding_boxes"] = bb
            return out
        return input_shape

    def get_config(self):
        return {**super().get_config(), "max_number": self.max_number, "fill_value": self.fill_value}
