"""MNIST digits (keras/src/datasets/mnist.py)."""

import numpy as np

from keras_b200.core.export_registry import keras_export
from keras_b200.datasets._common import ORIGIN
from keras_b200.utils.file_utils import get_file


@keras_export("keras.datasets.mnist.load_data")
def load_data(path="mnist.npz"):
    path = get_file(fname=path, origin=ORIGIN + "mnist.npz", file_hash="731c5ac602752760c8e48fbffcf8c3b850d9dc2a2aedcf2cc48468fc17b673d1")
    with np.load(path, allow_pickle=False) as f:
        return (f["x_train"], f["y_train"]), (f["x_test"], f["y_test"])
