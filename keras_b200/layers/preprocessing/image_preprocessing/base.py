"""Base class of the image preprocessing / augmentation layers
(keras/src/layers/preprocessing/image_preprocessing/base_image_preprocessing_layer.py).

Sub-classes draw one random ``transformation`` per call (per-sample parameters as batched tensors) and apply
it to images, labels, bounding boxes and segmentation masks.  All arithmetic runs as batched torch ops on the
device that holds the images.
"""

import math

import torch

from keras_b200.core import config
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.layers.preprocessing.data_layer import DataLayer
from keras_b200.layers.preprocessing.image_preprocessing.bounding_boxes import densify_bounding_boxes


class BaseImagePreprocessingLayer(DataLayer):
    _USE_BASE_FACTOR = True
    _FACTOR_BOUNDS = (-1, 1)

    def __init__(self, factor=None, bounding_box_format=None, data_format=None, **kwargs):
        super().__init__(**kwargs)
        self.bounding_box_format = bounding_box_format
        self.data_format = config.standardize_data_format(data_format)
        if self._USE_BASE_FACTOR:
            factor = factor or 0.0
            self._set_factor(factor)
        elif factor is not None:
            raise ValueError(f"Layer {self.__class__.__name__} does not take a `factor` argument. Received: factor={factor}")

    def _set_factor(self, factor):
        self.factor = self._check_factor(factor, self._FACTOR_BOUNDS)

    @staticmethod
    def _check_factor(factor, bounds, name="factor"):
        msg = f"The `{name}` argument should be a number (or a list of two numbers) in the range [{bounds[0]}, {bounds[1]}]. Received: {name}={factor}"
        if isinstance(factor, (tuple, list)):
            if len(factor) != 2 or factor[0] > bounds[1] or factor[1] < bounds[0]:
                raise ValueError(msg)
            lower, upper = sorted(factor)
        elif isinstance(factor, (int, float)):
            if factor < bounds[0] or factor > bounds[1]:
                raise ValueError(msg)
            factor = abs(factor)
            lower, upper = max(-factor, bounds[0]), factor
        else:
            raise ValueError(msg)
        return lower, upper

    # -- random helpers ------------------------------------------------------------------
    def _uniform(self, shape, lo=0.0, hi=1.0, like=None, seed=None):
        from keras_b200 import random

        t = random.uniform(shape, minval=lo, maxval=hi, seed=seed if seed is not None else self._get_seed_generator())
        if like is not None and isinstance(like, torch.Tensor) and t.device != like.device:
            t = t.to(like.device)
        return t

    def _images_of(self, data):
        return data["images"] if isinstance(data, dict) else data

    def _batch_hw(self, images):
        shape = tuple(images.shape)
        batched = len(shape) == 4
        if self.data_format == "channels_last":
            h, w = shape[-3], shape[-2]
        else:
            h, w = shape[-2], shape[-1]
        return (shape[0] if batched else 1), h, w

    # -- layout helpers: sub-classes compute on [B, C, H, W] float tensors -----------------
    def _to_bchw(self, images):
        x = images
        if self.data_format == "channels_last":
            x = x.permute(0, 3, 1, 2)
        return x

    def _from_bchw(self, x):
        if self.data_format == "channels_last":
            x = x.permute(0, 2, 3, 1)
        return x

    def _per_sample(self, v, ndim=4):
        return v.reshape((-1,) + (1,) * (ndim - 1))

    # -- API -----------------------------------------------------------------------------
    def get_random_transformation(self, data, training=True, seed=None):
        return None

    def _transform_images(self, images, transformation, interpolation):
        raise NotImplementedError()

    def transform_images(self, images, transformation, training=True):
        raise NotImplementedError()

    def transform_labels(self, labels, transformation, training=True):
        return labels

    def transform_bounding_boxes(self, bounding_boxes, transformation, training=True):
        return bounding_boxes

    def transform_segmentation_masks(self, segmentation_masks, transformation, training=True):
        return segmentation_masks

    def transform_single_image(self, image, transformation, training=True):
        return self.transform_images(image.unsqueeze(0), transformation=transformation, training=training).squeeze(0)

    def transform_single_label(self, label, transformation, training=True):
        return self.transform_labels(label.unsqueeze(0), transformation=transformation, training=training).squeeze(0)

    def transform_single_bounding_box(self, bounding_box, transformation, training=True):
        bb = {k: (convert_to_tensor(v).unsqueeze(0) if k in ("boxes", "labels") else v) for k, v in bounding_box.items()}
        out = self.transform_bounding_boxes(bb, transformation=transformation, training=training)
        return {k: (v.squeeze(0) if k in ("boxes", "labels") else v) for k, v in out.items()}

    def transform_single_segmentation_mask(self, segmentation_mask, transformation, training=True):
        m = convert_to_tensor(segmentation_mask).unsqueeze(0)
        return self.transform_segmentation_masks(m, transformation=transformation, training=training).squeeze(0)

    def _is_batched(self, maybe_image_batch):
        n = len(maybe_image_batch.shape)
        if n == 3:
            return False
        if n == 4:
            return True
        raise ValueError(f"Expected image tensor to have rank 3 (single image) or 4 (batch of images). Received: data.shape={tuple(maybe_image_batch.shape)}")

    def call(self, data, training=True):
        transformation = self.get_random_transformation(data, training=training)
        if isinstance(data, dict):
            data = dict(data)
            images = convert_to_tensor(data["images"])
            batched = self._is_batched(images)
            data["images"] = (self.transform_images if batched else self.transform_single_image)(images, transformation=transformation, training=training)
            if "bounding_boxes" in data:
                if not self.bounding_box_format:
                    raise ValueError("You passed an input with a 'bounding_boxes' key, but you didn't specify a bounding box format. Pass a "
                                     f"`bounding_box_format` argument to your {self.__class__.__name__} layer, e.g. `bounding_box_format='xyxy'`.")
                bb = densify_bounding_boxes(data["bounding_boxes"], is_batched=batched)
                fn = self.transform_bounding_boxes if batched else self.transform_single_bounding_box
                data["bounding_boxes"] = fn(bb, transformation=transformation, training=training)
            if "labels" in data:
                fn = self.transform_labels if batched else self.transform_single_label
                data["labels"] = fn(convert_to_tensor(data["labels"]), transformation=transformation, training=training)
            if "segmentation_masks" in data:
                fn = self.transform_segmentation_masks if batched else self.transform_single_segmentation_mask
                data["segmentation_masks"] = fn(convert_to_tensor(data["segmentation_masks"]), transformation=transformation, training=training)
            return data
        images = convert_to_tensor(data)
        if self._is_batched(images):
            return self.transform_images(images, transformation=transformation, training=training)
        return self.transform_single_image(images, transformation=transformation, training=training)

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"data_format": self.data_format})
        if self.bounding_box_format is not None:
            cfg.update({"bounding_box_format": self.bounding_box_format})
        return cfg

    # -- value ranges --------------------------------------------------------------------
    def _transform_value_range(self, images, original_range, target_range, dtype="float32"):
        if original_range[0] == target_range[0] and original_range[1] == target_range[1]:
            return images
        images = images.to(getattr(torch, dtype))
        images = (images - original_range[0]) / (original_range[1] - original_range[0])
        return images * (target_range[1] - target_range[0]) + target_range[0]

    # -- affine helpers ------------------------------------------------------------------
    @staticmethod
    def forward_affine(angle, translate_x, translate_y, scale, shear_x, shear_y, height, width, center_x=0.5, center_y=0.5):
        """Per-sample forward map p' = M p of pixel coordinates (angle/shear in degrees, translation in pixels).
        Returns ``(a0, a1, a2, b0, b1, b2)``."""
        ang = torch.deg2rad(angle)
        shx, shy = torch.tan(torch.deg2rad(shear_x)), torch.tan(torch.deg2rad(shear_y))
        cos, sin = torch.cos(ang), torch.sin(ang)
        cx, cy = center_x * (width - 1), center_y * (height - 1)
        a0, a1 = scale * (cos - shx * sin), scale * (sin + shx * cos)
        b0, b1 = scale * (shy * cos - sin), scale * (shy * sin + cos)
        a2 = cx + translate_x - a0 * cx - a1 * cy
        b2 = cy + translate_y - b0 * cx - b1 * cy
        return a0, a1, a2, b0, b1, b2

    @staticmethod
    def inverse_affine_params(a0, a1, a2, b0, b1, b2):
        """The 8-parameter output→input projective transform expected by ``ops.image.affine_transform``."""
        det = a0 * b1 - a1 * b0
        i0, i1 = b1 / det, -a1 / det
        j0, j1 = -b0 / det, a0 / det
        i2 = -(i0 * a2 + i1 * b2)
        j2 = -(j0 * a2 + j1 * b2)
        z = torch.zeros_like(a0)
        return torch.stack([i0, i1, i2, j0, j1, j2, z, z], dim=-1)

    def _apply_affine(self, images, forward, interpolation, fill_mode, fill_value):
        from keras_b200.ops import image as image_ops

        params = self.inverse_affine_params(*forward).to(torch.float32)
        return image_ops.affine_transform(images, params.to(images.device), interpolation=interpolation, fill_mode=fill_mode,
                                          fill_value=fill_value, data_format=self.data_format)

    @staticmethod
    def _box_hull(boxes, forward):
        """Apply the forward affine map to the corners of ``xyxy`` boxes ``[B, N, 4]`` and return their hulls."""
        a0, a1, a2, b0, b1, b2 = [t.reshape(-1, 1, 1).to(boxes.dtype).to(boxes.device) for t in forward]
        x1, y1, x2, y2 = boxes[..., 0:1], boxes[..., 1:2], boxes[..., 2:3], boxes[..., 3:4]
        xs = torch.cat([x1, x2, x1, x2], dim=-1)
        ys = torch.cat([y1, y1, y2, y2], dim=-1)
        nx = a0 * xs + a1 * ys + a2
        ny = b0 * xs + b1 * ys + b2
        return torch.stack([nx.amin(-1), ny.amin(-1), nx.amax(-1), ny.amax(-1)], dim=-1)

    def _boxes_io(self, bounding_boxes, height, width, fn, out_height=None, out_width=None):
        """Convert to absolute ``xyxy``, apply ``fn(boxes) -> boxes``, clip to the output image and convert back."""
        from keras_b200.layers.preprocessing.image_preprocessing import bounding_boxes as bbx

        out_height = height if out_height is None else out_height
        out_width = width if out_width is None else out_width
        bb = bbx.convert_format(bounding_boxes, self.bounding_box_format, "xyxy", height, width)
        bb = dict(bb)
        bb["boxes"] = fn(bb["boxes"])
        bb = bbx.clip_to_image_size(bb, out_height, out_width, "xyxy")
        return bbx.convert_format(bb, "xyxy", self.bounding_box_format, out_height, out_width)
