"""Boston housing regression data (keras/src/datasets/boston_housing.py)."""

import numpy as np

from keras_b200.core.export_registry import keras_export
from keras_b200.datasets._common import ORIGIN, shuffled_split
from keras_b200.utils.file_utils import get_file


@keras_export("keras.datasets.boston_housing.load_data")
def load_data(path="boston_housing.npz", test_split=0.2, seed=113):
    if not (0 <= test_split < 1):
        raise ValueError(f"Invalid `test_split` argument: {test_split}. It must be between 0 and 1 (exclusive of 1).")
    path = get_file(path, origin=ORIGIN + "boston_housing.npz", file_hash="f553886a1f8d56431e820c5b82552d9d95cfcb96d1e678153f8839538947dff5")
    with np.load(path, allow_pickle=False) as f:
        x, y = f["x"], f["y"]
    return shuffled_split(x, y, test_split, seed)
