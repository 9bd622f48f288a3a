"""``keras.preprocessing.image`` (keras/api/preprocessing/image/__init__.py)."""

from keras_b200.utils.image_utils import array_to_img, img_to_array, load_img, save_img, smart_resize  # noqa: F401
