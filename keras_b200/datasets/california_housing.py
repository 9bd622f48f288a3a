"""California housing regression data (keras/src/datasets/california_housing.py)."""

import numpy as np

from keras_b200.core.export_registry import keras_export
from keras_b200.datasets._common import ORIGIN, shuffled_split
from keras_b200.utils.file_utils import get_file


@keras_export("keras.datasets.california_housing.load_data")
def load_data(version="large", path="california_housing.npz", test_split=0.2, seed=113):
    if not (0 <= test_split < 1):
        raise ValueError(f"Invalid `test_split` argument: {test_split}. It must be between 0 and 1 (exclusive of 1).")
    path = get_file(path, origin=ORIGIN + "california_housing.npz", file_hash="1a2e3a52e0398de6463aebe6f4a8da34fb21fbb6b934cf88c3425e766f2a1a6f")
    with np.load(path, allow_pickle=False) as f:
        x, y = f["x"], f["y"]
    if version == "small":
        x, y = x[:600], y[:600]
    elif version != "large":
        raise ValueError(f"Argument `version` must be one of 'small', 'large'. Received: version={version}")
    return shuffled_split(x, y, test_split, seed)
