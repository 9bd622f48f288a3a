"""Drawing helpers on image batches: ``draw_bounding_boxes``, ``draw_segmentation_masks``
(keras/src/visualization/{draw_bounding_boxes,draw_segmentation_masks}.py).  The reference rasterises with OpenCV;
here boxes and labels are drawn with PIL and masks are blended with NumPy."""

import numpy as np

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_numpy, is_tensor
from keras_b200.layers.preprocessing.image_preprocessing import bounding_boxes as bbx


def _np(x):
    return convert_to_numpy(x) if is_tensor(x) else np.asarray(x)


@keras_export("keras.visualization.draw_bounding_boxes")
def draw_bounding_boxes(images, bounding_boxes, bounding_box_format, class_mapping=None, color=(128, 128, 128), line_thickness=2, text_thickness=1,
                        font_scale=1.0, data_format=None):
    """Return a ``uint8`` copy of ``images`` with the boxes (and class names, if ``class_mapping`` is given) drawn."""
    try:
        from PIL import Image, ImageDraw
    except ImportError:
        raise ImportError("The `draw_bounding_boxes` function requires the `PIL` package. Please install it with `pip install pillow`.")
    class_mapping = class_mapping or {}
    text_thickness = text_thickness or line_thickness
    data_format = data_format or config.image_data_format()
    images = _np(images)
    if images.ndim != 4:
        raise ValueError(f"`images` must be batched 4D tensor. Received: images.shape={images.shape}")
    if not isinstance(bounding_boxes, dict):
        raise TypeError(f"`bounding_boxes` should be a dict. Received: bounding_boxes={bounding_boxes} of type {type(bounding_boxes)}")
    if "boxes" not in bounding_boxes or "labels" not in bounding_boxes:
        raise ValueError(f"`bounding_boxes` should be a dict containing 'boxes' and 'labels' keys. Received: bounding_boxes={bounding_boxes}")
    if data_format == "channels_first":
        images = images.transpose(0, 2, 3, 1)
    h, w = images.shape[1], images.shape[2]
    boxes = _np(bbx.convert_format(bounding_boxes["boxes"], bounding_box_format, "xyxy", h, w))
    labels = _np(bounding_boxes["labels"])
    confidences = _np(bounding_boxes["confidences"]) if "confidences" in bounding_boxes else None
    out = []
    for i in range(images.shape[0]):
        img = Image.fromarray(np.clip(images[i], 0, 255).astype("uint8")).convert("RGB")
        draw = ImageDraw.Draw(img)
        for b in range(boxes.shape[1]):
            cid = int(labels[i, b])
            if cid == -1:
                continue
            x1, y1, x2, y2 = [float(v) for v in boxes[i, b]]
            draw.rectangle([x1, y1, x2, y2], outline=tuple(color), width=int(line_thickness))
            if cid in class_mapping:
                text = str(class_mapping[cid])
                if confidences is not None:
                    text = f"{text} | {float(confidences[i, b]):.2f}"
                draw.text((x1 + 2, max(y1 - 12 * font_scale, 0)), text, fill=tuple(color))
        out.append(np.asarray(img))
    out = np.stack(out).astype("uint8")
    if data_format == "channels_first":
        out = out.transpose(0, 3, 1, 2)
    return out


def _generate_color_palette(num_classes):
    palette = np.array([2 ** 25 - 1, 2 ** 15 - 1, 2 ** 21 - 1])
    return [((i * palette) % 255).tolist() for i in range(num_classes)]


@keras_export("keras.visualization.draw_segmentation_masks")
def draw_segmentation_masks(images, segmentation_masks, num_classes=None, color_mapping=None, alpha=0.8, blend=True, ignore_index=-1, data_format=None):
    data_format = data_format or config.image_data_format()
    images = _np(images).astype("uint8")
    masks = _np(segmentation_masks)
    if not np.issubdtype(masks.dtype, np.integer):
        dtype = masks.dtype
        raise TypeError(f"`segmentation_masks` must be in integer dtype. Received: segmentation_masks.dtype={dtype}")
    if images.ndim != 4:
        raise ValueError(f"`images` must be batched 4D tensor. Received: images.shape={images.shape}")
    if data_format == "channels_first":
        images = images.transpose(0, 2, 3, 1)
        masks = masks.transpose(0, 2, 3, 1)
    if masks.ndim == 4 and masks.shape[-1] == 1:
        masks = masks[..., 0]
    if num_classes is None:
        num_classes = int(masks.max()) + 1
    if color_mapping is None:
        colors = _generate_color_palette(num_classes)
    else:
        colors = [color_mapping[i] for i in range(num_classes)]
    colors = np.array(colors + [[0, 0, 0]], dtype="uint8")
    valid = masks != ignore_index
    idx = np.where(valid, masks, num_classes)
    colored = colors[idx]
    if blend:
        a = np.where(valid[..., None], alpha, 0.0)
        out = (images.astype("float32") * (1 - a) + colored.astype("float32") * a).clip(0, 255).astype("uint8")
    else:
        out = np.where(valid[..., None], colored, images).astype("uint8")
    if data_format == "channels_first":
        out = out.transpose(0, 3, 1, 2)
    return out
