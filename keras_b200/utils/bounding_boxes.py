"""``keras.utils.bounding_boxes``: format conversion, clipping, IoU, affine helpers and anchor delta coding."""

import math

import torch

from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.layers.preprocessing.image_preprocessing.bounding_boxes import (  # noqa: F401
    affine_transform, clip_to_image_size, compute_ciou, compute_iou, convert_format, crop, pad,
)


def _variance(variance, like):
    if variance is None:
        return None
    v = convert_to_tensor(variance).to(like.dtype).to(like.device)
    if v.numel() != 4:
        raise ValueError(f"`variance` must be a list/tuple/array of 4 numbers. Received: variance={variance}")
    return v.reshape((1,) * (like.ndim - 1) + (4,))


@keras_export("keras.utils.bounding_boxes.encode_box_to_deltas")
def encode_box_to_deltas(anchors, boxes, anchor_format, box_format, encoding_format="center_yxhw", variance=None, image_shape=None):
    """Regression targets of ``boxes`` relative to ``anchors`` (keras/src/layers/preprocessing/image_preprocessing/
    bounding_boxes/converters.py:256-345): centre offsets scaled by the anchor size and log size ratios."""
    if encoding_format not in ("center_xywh", "center_yxhw"):
        raise ValueError(f"`encoding_format` should be one of 'center_xywh' or 'center_yxhw', got {encoding_format}")
    h, w = (image_shape[0], image_shape[1]) if image_shape is not None else (None, None)
    a = convert_format(anchors, anchor_format, encoding_format, h, w)
    b = convert_format(boxes, box_format, encoding_format, h, w)
    deltas = torch.cat([(b[..., :2] - a[..., :2]) / a[..., 2:], torch.log(b[..., 2:] / a[..., 2:])], dim=-1)
    v = _variance(variance, deltas)
    return deltas / v if v is not None else deltas


@keras_export("keras.utils.bounding_boxes.decode_deltas_to_boxes")
def decode_deltas_to_boxes(anchors, boxes_delta, anchor_format, box_format, encoded_format="center_yxhw", variance=None, image_shape=None):
    """Inverse of ``encode_box_to_deltas``; ``anchors`` may be a dict of per-level anchors matched by key."""
    if encoded_format not in ("center_xywh", "center_yxhw"):
        raise ValueError(f"`encoded_format` should be one of 'center_xywh' or 'center_yxhw', got {encoded_format}")
    h, w = (image_shape[0], image_shape[1]) if image_shape is not None else (None, None)

    def one(anchor, delta):
        a = convert_format(anchor, anchor_format, encoded_format, h, w)
        d = convert_to_tensor(delta).to(a.dtype)
        v = _variance(variance, d)
        if v is not None:
            d = d * v
        decoded = torch.cat([d[..., :2] * a[..., 2:] + a[..., :2], torch.exp(d[..., 2:]) * a[..., 2:]], dim=-1)
        return convert_format(decoded, encoded_format, box_format, h, w)

    if isinstance(anchors, dict):
        return {k: one(anchors[k], boxes_delta[k]) for k in anchors}
    return one(anchors, boxes_delta)
