"""Bounding-box helpers: format conversion, clipping, IoU, affine transforms, validation
(keras/src/layers/preprocessing/image_preprocessing/bounding_boxes/{converters,iou,validation,bounding_box}.py).

Boxes travel as ``{"boxes": [..., N, 4], "labels": [..., N]}``; padding boxes have label ``-1``.
"""

import torch

from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor

SUPPORTED_FORMATS = ("xyxy", "yxyx", "xywh", "center_xywh", "center_yxhw", "rel_xyxy", "rel_yxyx", "rel_xywh", "rel_center_xywh")


def _split(b):
    return b[..., 0:1], b[..., 1:2], b[..., 2:3], b[..., 3:4]


def _to_xyxy(boxes, fmt, height, width):
    a, b, c, d = _split(boxes)
    rel = fmt.startswith("rel_")
    f = fmt[4:] if rel else fmt
    if f == "xyxy":
        x1, y1, x2, y2 = a, b, c, d
    elif f == "yxyx":
        y1, x1, y2, x2 = a, b, c, d
    elif f == "xywh":
        x1, y1, x2, y2 = a, b, a + c, b + d
    elif f == "center_xywh":
        x1, y1, x2, y2 = a - c / 2, b - d / 2, a + c / 2, b + d / 2
    elif f == "center_yxhw":
        y1, x1, y2, x2 = a - c / 2, b - d / 2, a + c / 2, b + d / 2
    else:
        raise ValueError(f"Unsupported bounding box format: {fmt}")
    if rel:
        _need_size(height, width, fmt)
        x1, x2, y1, y2 = x1 * width, x2 * width, y1 * height, y2 * height
    return x1, y1, x2, y2


def _from_xyxy(x1, y1, x2, y2, fmt, height, width):
    rel = fmt.startswith("rel_")
    f = fmt[4:] if rel else fmt
    if rel:
        _need_size(height, width, fmt)
        x1, x2, y1, y2 = x1 / width, x2 / width, y1 / height, y2 / height
    if f == "xyxy":
        parts = (x1, y1, x2, y2)
    elif f == "yxyx":
        parts = (y1, x1, y2, x2)
    elif f == "xywh":
        parts = (x1, y1, x2 - x1, y2 - y1)
    elif f == "center_xywh":
        parts = ((x1 + x2) / 2, (y1 + y2) / 2, x2 - x1, y2 - y1)
    elif f == "center_yxhw":
        parts = ((y1 + y2) / 2, (x1 + x2) / 2, y2 - y1, x2 - x1)
    else:
        raise ValueError(f"Unsupported bounding box format: {fmt}")
    return torch.cat(parts, dim=-1)


def _need_size(height, width, fmt):
    if height is None or width is None:
        raise ValueError(f"Relative bounding box formats need `height` and `width`. Received: format={fmt}, height={height}, width={width}")


@keras_export("keras.utils.bounding_boxes.convert_format")
def convert_format(boxes, source, target, height=None, width=None, dtype="float32"):
    """Convert ``boxes`` (tensor or ``{"boxes", "labels"}`` dict) between bounding-box formats."""
    if isinstance(boxes, dict):
        out = dict(boxes)
        out["boxes"] = convert_format(boxes["boxes"], source, target, height, width, dtype)
        return out
    source, target = source.lower(), target.lower()
    for f in (source, target):
        if f not in SUPPORTED_FORMATS:
            raise ValueError(f"Invalid bounding box format {f!r}. Supported formats: {SUPPORTED_FORMATS}")
    b = convert_to_tensor(boxes).to(getattr(torch, dtype))
    if b.shape[-1] != 4:
        raise ValueError(f"Expected `boxes` to have a last dimension of 4. Received: boxes.shape={tuple(b.shape)}")
    if source == target:
        return b
    if isinstance(height, torch.Tensor) and height.ndim == 1:
        height, width = height.reshape(-1, 1, 1).to(b.dtype), width.reshape(-1, 1, 1).to(b.dtype)
    return _from_xyxy(*_to_xyxy(b, source, height, width), target, height, width)


@keras_export("keras.utils.bounding_boxes.clip_to_image_size")
def clip_to_image_size(bounding_boxes, height=None, width=None, bounding_box_format="xyxy"):
    if bounding_box_format not in ("xyxy", "rel_xyxy"):
        raise NotImplementedError(f"clip_to_image_size supports 'xyxy' and 'rel_xyxy'. Received: {bounding_box_format}")
    boxes = convert_to_tensor(bounding_boxes["boxes"]).to(torch.float32)
    labels = convert_to_tensor(bounding_boxes["labels"])
    if bounding_box_format == "xyxy":
        _need_size(height, width, bounding_box_format)
        hi_x, hi_y = float(width), float(height)
    else:
        hi_x = hi_y = 1.0
    x1, y1, x2, y2 = _split(boxes)
    x1, x2 = x1.clamp(0, hi_x), x2.clamp(0, hi_x)
    y1, y2 = y1.clamp(0, hi_y), y2.clamp(0, hi_y)
    area = ((x2 - x1) * (y2 - y1)).squeeze(-1)
    out = dict(bounding_boxes)
    out["boxes"] = torch.cat([x1, y1, x2, y2], dim=-1)
    out["labels"] = torch.where(area > 0, labels, torch.full_like(labels, -1))
    return out


@keras_export("keras.utils.bounding_boxes.affine_transform")
def affine_transform(boxes, angle, translate_x, translate_y, scale, shear_x, shear_y, height, width, center_x=None, center_y=None,
                     bounding_box_format="xyxy"):
    """Apply a per-sample affine map (angle in degrees, translation as a fraction of the image) to ``xyxy`` boxes
    ``[B, N, 4]`` and return the axis-aligned hulls."""
    if bounding_box_format != "xyxy":
        raise NotImplementedError("affine_transform expects 'xyxy' boxes.")
    b = convert_to_tensor(boxes).to(torch.float32)
    B = b.shape[0]
    dev = b.device

    def vec(v, default):
        if v is None:
            v = default
        t = convert_to_tensor(v).to(torch.float32).to(dev).reshape(-1)
        return t.expand(B) if t.numel() == 1 else t

    cx = vec(center_x, 0.5) * width
    cy = vec(center_y, 0.5) * height
    ang = torch.deg2rad(vec(angle, 0.0))
    tx, ty = vec(translate_x, 0.0) * width, vec(translate_y, 0.0) * height
    sc = vec(scale, 1.0)
    shx, shy = torch.tan(torch.deg2rad(vec(shear_x, 0.0))), torch.tan(torch.deg2rad(vec(shear_y, 0.0)))
    cos, sin = torch.cos(ang), torch.sin(ang)
    # forward map p' = c + t + scale * [[1, shx], [shy, 1]] @ [[cos, sin], [-sin, cos]] @ (p - c): rotation is
    # counter-clockwise on screen (y grows downwards)
    a0, a1 = sc * (cos - shx * sin), sc * (sin + shx * cos)
    b0, b1 = sc * (shy * cos - sin), sc * (shy * sin + cos)
    x1, y1, x2, y2 = _split(b)
    xs = torch.cat([x1, x2, x1, x2], dim=-1) - cx.reshape(B, 1, 1)
    ys = torch.cat([y1, y1, y2, y2], dim=-1) - cy.reshape(B, 1, 1)
    nx = a0.reshape(B, 1, 1) * xs + a1.reshape(B, 1, 1) * ys + (cx + tx).reshape(B, 1, 1)
    ny = b0.reshape(B, 1, 1) * xs + b1.reshape(B, 1, 1) * ys + (cy + ty).reshape(B, 1, 1)
    return torch.stack([nx.amin(-1), ny.amin(-1), nx.amax(-1), ny.amax(-1)], dim=-1)


@keras_export("keras.utils.bounding_boxes.crop")
def crop(boxes, top, left, height, width, bounding_box_format="xyxy"):
    if bounding_box_format != "xyxy":
        raise NotImplementedError("crop expects 'xyxy' boxes.")
    b = convert_to_tensor(boxes).to(torch.float32)
    x1, y1, x2, y2 = _split(b)
    x1, x2 = (x1 - left).clamp(0, width), (x2 - left).clamp(0, width)
    y1, y2 = (y1 - top).clamp(0, height), (y2 - top).clamp(0, height)
    return torch.cat([x1, y1, x2, y2], dim=-1)


@keras_export("keras.utils.bounding_boxes.pad")
def pad(boxes, top, left, height=None, width=None, bounding_box_format="xyxy"):
    if bounding_box_format != "xyxy":
        raise NotImplementedError("pad expects 'xyxy' boxes.")
    b = convert_to_tensor(boxes).to(torch.float32)
    x1, y1, x2, y2 = _split(b)
    return torch.cat([x1 + left, y1 + top, x2 + left, y2 + top], dim=-1)


@keras_export("keras.utils.bounding_boxes.compute_iou")
def compute_iou(boxes1, boxes2, bounding_box_format, use_masking=False, mask_val=-1, image_shape=None):
    b1 = convert_to_tensor(boxes1).to(torch.float32)
    b2 = convert_to_tensor(boxes2).to(torch.float32)
    if b1.ndim not in (2, 3) or b2.ndim not in (2, 3):
        raise ValueError(f"compute_iou() expects boxes of rank 2 or 3. Received: boxes1.shape={tuple(b1.shape)}, boxes2.shape={tuple(b2.shape)}")
    h = w = None
    if bounding_box_format.startswith("rel_"):
        if image_shape is None:
            raise ValueError("When using relative bounding box formats (e.g. `rel_yxyx`) the `image_shape` argument must be provided")
        h, w = image_shape[0], image_shape[1]
    b1 = convert_format(b1, bounding_box_format, "yxyx", h, w)
    b2 = convert_format(b2, bounding_box_format, "yxyx", h, w)

    def area(b):
        return (b[..., 2] - b[..., 0]) * (b[..., 3] - b[..., 1])

    a1, a2 = area(b1), area(b2)
    lu = torch.maximum(b1[..., :, None, :2], b2[..., None, :, :2])
    rd = torch.minimum(b1[..., :, None, 2:], b2[..., None, :, 2:])
    inter = (rd - lu).clamp(min=0)
    inter = inter[..., 0] * inter[..., 1]
    union = a1[..., :, None] + a2[..., None, :] - inter
    iou = inter / (union + 1e-7)
    if use_masking:
        m1 = (b1[..., 0] <= -1)[..., :, None]
        m2 = (b2[..., 0] <= -1)[..., None, :]
        iou = torch.where(m1 | m2, torch.full_like(iou, float(mask_val)), iou)
    return iou


@keras_export("keras.utils.bounding_boxes.compute_ciou")
def compute_ciou(boxes1, boxes2, bounding_box_format, image_shape=None):
    import math

    b1 = convert_to_tensor(boxes1).to(torch.float32)
    b2 = convert_to_tensor(boxes2).to(torch.float32)
    h = w = None
    if bounding_box_format.startswith("rel_"):
        h, w = image_shape[0], image_shape[1]
    b1 = convert_format(b1, bounding_box_format, "xyxy", h, w)
    b2 = convert_format(b2, bounding_box_format, "xyxy", h, w)
    x1, y1, x2, y2 = b1.unbind(-1)
    X1, Y1, X2, Y2 = b2.unbind(-1)
    w1, h1, w2, h2 = x2 - x1, y2 - y1 + 1e-7, X2 - X1, Y2 - Y1 + 1e-7
    inter = (torch.minimum(x2, X2) - torch.maximum(x1, X1)).clamp(min=0) * (torch.minimum(y2, Y2) - torch.maximum(y1, Y1)).clamp(min=0)
    union = w1 * h1 + w2 * h2 - inter + 1e-7
    iou = inter / union
    cw = torch.maximum(x2, X2) - torch.minimum(x1, X1)
    ch = torch.maximum(y2, Y2) - torch.minimum(y1, Y1)
    c2 = cw ** 2 + ch ** 2 + 1e-7
    rho2 = ((X1 + X2 - x1 - x2) ** 2 + (Y1 + Y2 - y1 - y2) ** 2) / 4
    v = (4 / math.pi ** 2) * (torch.atan(w2 / h2) - torch.atan(w1 / h1)) ** 2
    alpha = v / (v - iou + (1 + 1e-7))
    return iou - (rho2 / c2 + v * alpha)


def validate_bounding_boxes(bounding_boxes):
    if not isinstance(bounding_boxes, dict) or "labels" not in bounding_boxes or "boxes" not in bounding_boxes:
        raise ValueError(f"Expected `bounding_boxes` argument to be a dict with keys 'boxes' and 'labels'. Received: bounding_boxes={bounding_boxes}")
    boxes, labels = bounding_boxes["boxes"], bounding_boxes["labels"]
    if isinstance(boxes, list):
        if not isinstance(labels, list):
            raise ValueError(f"If `bounding_boxes['boxes']` is a list, then `bounding_boxes['labels']` must also be a list.Received: bounding_boxes['labels']={labels}")
        if len(boxes) != len(labels):
            raise ValueError(f"If `bounding_boxes['boxes']` and `bounding_boxes['labels']` are both lists, they must have the same length. Received: len(bounding_boxes['boxes'])={len(boxes)} and len(bounding_boxes['labels'])={len(labels)} and ")
    elif hasattr(boxes, "shape") and hasattr(labels, "shape"):
        if len(boxes.shape) == 3:
            if len(labels.shape) not in (2, 3):
                raise ValueError(f"Expected `bounding_boxes['labels']` to have rank 2 or 3. Received: labels.shape={tuple(labels.shape)}")
        elif len(boxes.shape) == 2:
            if len(labels.shape) not in (1, 2):
                raise ValueError(f"Expected `bounding_boxes['labels']` to have rank 1 or 2. Received: labels.shape={tuple(labels.shape)}")
        else:
            raise ValueError(f"Expected `bounding_boxes['boxes']` to have rank 2 or 3. Received: boxes.shape={tuple(boxes.shape)}")
        if boxes.shape[-1] != 4:
            raise ValueError(f"Expected `bounding_boxes['boxes']` to have a last dimension of 4. Received: boxes.shape={tuple(boxes.shape)}")


def densify_bounding_boxes(bounding_boxes, is_batched=False, max_boxes=None, boxes_default_value=0, labels_default_value=-1, backend=None):
    validate_bounding_boxes(bounding_boxes)
    boxes, labels = bounding_boxes["boxes"], bounding_boxes["labels"]
    if isinstance(boxes, list) and is_batched:
        n = max_boxes if max_boxes is not None else max((len(b) for b in boxes), default=0)
        bt = torch.full((len(boxes), n, 4), float(boxes_default_value))
        lt = torch.full((len(boxes), n), labels_default_value, dtype=torch.int64)
        for i, (b, l) in enumerate(zip(boxes, labels)):
            b = convert_to_tensor(b).reshape(-1, 4)[:n]
            l = convert_to_tensor(l).reshape(-1)[:n]
            bt[i, : b.shape[0]] = b.to(bt.dtype).cpu()
            lt[i, : l.shape[0]] = l.to(lt.dtype).cpu()
        return {"boxes": bt, "labels": lt}
    boxes = convert_to_tensor(boxes).to(torch.float32)
    labels = convert_to_tensor(labels)
    if max_boxes is not None:
        axis = 1 if is_batched else 0
        cur = boxes.shape[axis]
        if cur > max_boxes:
            boxes = boxes.narrow(axis, 0, max_boxes)
            labels = labels.narrow(axis, 0, max_boxes)
        elif cur < max_boxes:
            pad_n = max_boxes - cur
            bshape = list(boxes.shape)
            bshape[axis] = pad_n
            lshape = list(labels.shape)
            lshape[axis] = pad_n
            boxes = torch.cat([boxes, torch.full(bshape, float(boxes_default_value), dtype=boxes.dtype, device=boxes.device)], dim=axis)
            labels = torch.cat([labels, torch.full(lshape, labels_default_value, dtype=labels.dtype, device=labels.device)], dim=axis)
    return {"boxes": boxes, "labels": labels}
