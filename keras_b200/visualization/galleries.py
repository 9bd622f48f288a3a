"""Image-grid plots: ``plot_image_gallery``, ``plot_bounding_box_gallery``, ``plot_segmentation_mask_gallery``
(keras/src/visualization/plot_*.py).  With matplotlib installed the grid is a matplotlib figure (shown or saved to
``path``); without it the grid is composed with PIL and returned as an image (and saved to ``path`` when given)."""

import math

import numpy as np

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_numpy, is_tensor
from keras_b200.visualization.drawing import draw_bounding_boxes, draw_segmentation_masks

try:
    import matplotlib.pyplot as plt
except ImportError:
    plt = None


def _np(x):
    return convert_to_numpy(x) if is_tensor(x) else np.asarray(x)


def _extract_image_batch(images, num_images, batch_size):
    num_samples = min(num_images, batch_size)
    return images[:num_samples]


def _to_uint8(images, value_range):
    lo, hi = value_range
    images = (np.asarray(images, dtype="float32") - lo) / float(hi - lo) * 255.0
    return images.clip(0, 255).astype("uint8")


@keras_export("keras.visualization.plot_image_gallery")
def plot_image_gallery(images, y_true=None, y_pred=None, label_map=None, rows=None, cols=None, value_range=(0, 255), scale=2, path=None, show=None,
                       transparent=True, dpi=60, legend_handles=None, data_format=None):
    if path is not None and show:
        raise ValueError("plot_gallery() expects either `path` to be set, or `show` to be true.")
    if (y_true is not None or y_pred is not None) and label_map is None:
        raise ValueError("If `y_true` or `y_pred` are provided, `label_map` must also be provided.")
    show = show if show is not None else (path is None)
    data_format = data_format or config.image_data_format()
    images = _np(images)
    if data_format == "channels_first":
        images = images.transpose(0, 2, 3, 1)
    batch_size = images.shape[0] if images.ndim == 4 else 1
    rows = rows or int(math.ceil(math.sqrt(batch_size)))
    cols = cols or int(math.ceil(batch_size // rows))
    num_images = rows * cols
    images = _to_uint8(_extract_image_batch(images, num_images, batch_size), value_range)
    if images.shape[-1] == 1:
        images = np.repeat(images, 3, axis=-1)
    titles = []
    for i in range(images.shape[0]):
        t = ""
        if y_true is not None and i < len(y_true):
            t += f"Label: {label_map[int(np.asarray(y_true[i]))]}"
        if y_pred is not None and i < len(y_pred):
            t += ("\n" if t else "") + f"Prediction: {label_map[int(np.asarray(y_pred[i]))]}"
        titles.append(t)
    if plt is not None:
        fig, axes = plt.subplots(nrows=rows, ncols=cols, figsize=(cols * scale, rows * scale), frameon=False, layout="tight", squeeze=True,
                                 sharex="row", sharey="col")
        fig.subplots_adjust(wspace=0, hspace=0)
        if isinstance(axes, np.ndarray) and len(axes.shape) == 1:
            axes = np.expand_dims(axes, 0) if rows == 1 else np.expand_dims(axes, -1)
        if legend_handles is not None:
            fig.legend(handles=legend_handles, loc="lower center")
        for r in range(rows):
            for c in range(cols):
                i = r * cols + c
                ax = axes[r, c] if isinstance(axes, np.ndarray) else axes
                ax.axis("off")
                if i < images.shape[0]:
                    ax.imshow(images[i], aspect="auto")
                    if titles[i]:
                        ax.set_title(titles[i], fontsize=12)
        if path is not None:
            plt.savefig(fname=path, pad_inches=0, bbox_inches="tight", transparent=transparent, dpi=dpi)
            plt.close()
        elif show:
            plt.show()
            plt.close()
        return None
    from PIL import Image, ImageDraw

    h, w = images.shape[1], images.shape[2]
    title_h = 24 if any(titles) else 0
    grid = Image.new("RGB", (cols * w, rows * (h + title_h)), (255, 255, 255))
    draw = ImageDraw.Draw(grid)
    for i in range(images.shape[0]):
        r, c = divmod(i, cols)
        grid.paste(Image.fromarray(images[i][..., :3]), (c * w, r * (h + title_h) + title_h))
        if titles[i]:
            draw.text((c * w + 2, r * (h + title_h) + 2), titles[i].replace("\n", " | "), fill=(0, 0, 0))
    if path is not None:
        grid.save(path)
    return grid


@keras_export("keras.visualization.plot_bounding_box_gallery")
def plot_bounding_box_gallery(images, bounding_box_format, y_true=None, y_pred=None, value_range=(0, 255), true_color=(0, 188, 212),
                              pred_color=(255, 235, 59), line_thickness=2, font_scale=1.0, text_thickness=None, class_mapping=None,
                              ground_truth_mapping=None, prediction_mapping=None, legend=False, legend_handles=None, rows=None, cols=None,
                              data_format=None, **kwargs):
    prediction_mapping = prediction_mapping or class_mapping
    ground_truth_mapping = ground_truth_mapping or class_mapping
    data_format = data_format or config.image_data_format()
    plotted = _to_uint8(_np(images), value_range)
    draw_fn = lambda imgs, boxes, color, mapping: draw_bounding_boxes(imgs, boxes, bounding_box_format, class_mapping=mapping, color=color,
                                                                      line_thickness=line_thickness, text_thickness=text_thickness,
                                                                      font_scale=font_scale, data_format=data_format)
    if y_true is not None:
        plotted = draw_fn(plotted, y_true, true_color, ground_truth_mapping)
    if y_pred is not None:
        plotted = draw_fn(plotted, y_pred, pred_color, prediction_mapping)
    if legend:
        if legend_handles:
            raise ValueError("Only pass `legend` OR `legend_handles` to `keras.visualization.plot_bounding_box_gallery()`.")
        if plt is not None:
            from matplotlib import patches

            legend_handles = [patches.Patch(color=np.array(true_color) / 255.0, label="Ground Truth"),
                              patches.Patch(color=np.array(pred_color) / 255.0, label="Prediction")]
    return plot_image_gallery(plotted, value_range=(0, 255), legend_handles=legend_handles, rows=rows, cols=cols, data_format=data_format, **kwargs)


@keras_export("keras.visualization.plot_segmentation_mask_gallery")
def plot_segmentation_mask_gallery(images, num_classes, value_range=(0, 255), y_true=None, y_pred=None, color_mapping=None, blend=True, alpha=0.8,
                                   ignore_index=-1, data_format=None, **kwargs):
    data_format = data_format or config.image_data_format()
    images = _to_uint8(_np(images), value_range)
    axis = 2 if data_format == "channels_last" else 3
    plotted = images
    for y in (y_true, y_pred):
        if y is not None:
            drawn = draw_segmentation_masks(images, _np(y), num_classes=num_classes, color_mapping=color_mapping, alpha=alpha, blend=blend,
                                            ignore_index=ignore_index, data_format=data_format)
            plotted = np.concatenate([plotted, drawn], axis=axis)  # side by side: image | truth | prediction
    return plot_image_gallery(plotted, value_range=(0, 255), data_format=data_format, **kwargs)
