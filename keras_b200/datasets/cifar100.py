"""CIFAR-100 (keras/src/datasets/cifar100.py)."""

import os

import numpy as np

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.datasets.cifar10 import load_batch
from keras_b200.utils.file_utils import get_file


@keras_export("keras.datasets.cifar100.load_data")
def load_data(label_mode="fine"):
    if label_mode not in ["fine", "coarse"]:
        raise ValueError(f'`label_mode` must be one of `"fine"`, `"coarse"`. Received: label_mode={label_mode}.')
    path = get_file(fname="cifar-100-python-target", origin="https://www.cs.toronto.edu/~kriz/cifar-100-python.tar.gz", extract=True,
                    file_hash="85cd44d02ba6437773c5bbd22e183051d648de2e7d6b014e1ef29b855ba677a7")
    path = os.path.join(path, "cifar-100-python")
    x_train, y_train = load_batch(os.path.join(path, "train"), label_key=f"{label_mode}_labels")
    x_test, y_test = load_batch(os.path.join(path, "test"), label_key=f"{label_mode}_labels")
    y_train, y_test = np.reshape(y_train, (len(y_train), 1)), np.reshape(y_test, (len(y_test), 1))
    if config.image_data_format() == "channels_last":
        x_train, x_test = x_train.transpose(0, 2, 3, 1), x_test.transpose(0, 2, 3, 1)
    return (x_train, y_train), (x_test, y_test)
