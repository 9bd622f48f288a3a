"""``keras.preprocessing``: the dataset builders and the legacy ``image`` / ``sequence`` helper namespaces
(keras/api/preprocessing/__init__.py)."""

from keras_b200.preprocessing import image, sequence  # noqa: F401
from keras_b200.utils.dataset_utils import image_dataset_from_directory, text_dataset_from_directory, timeseries_dataset_from_array  # noqa: F401
