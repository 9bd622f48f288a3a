from keras_b200.visualization.drawing import draw_bounding_boxes, draw_segmentation_masks  # noqa: F401
from keras_b200.visualization.galleries import plot_bounding_box_gallery, plot_image_gallery, plot_segmentation_mask_gallery  # noqa: F401
