"""CIFAR-10 (keras/src/datasets/cifar10.py)."""

import os

import numpy as np

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.datasets._common import RestrictedUnpickler
from keras_b200.utils.file_utils import get_file


def load_batch(fpath, label_key="labels"):
    with open(fpath, "rb") as f:
        d = RestrictedUnpickler(f, encoding="bytes").load()
    d = {k.decode("utf8"): v for k, v in d.items()}
    data = d["data"]
    return data.reshape(data.shape[0], 3, 32, 32), d[label_key]


@keras_export("keras.datasets.cifar10.load_data")
def load_data():
    path = get_file(fname="cifar-10-batches-py-target", origin="https://www.cs.toronto.edu/~kriz/cifar-10-python.tar.gz", extract=True,
                    file_hash="6d958be074577803d12ecdefd02955f39262c83c16fe9348329d7fe0b5c001ce")
    path = os.path.join(path, "cifar-10-batches-py")
    xs, ys = [], []
    for i in range(1, 6):
        x, y = load_batch(os.path.join(path, f"data_batch_{i}"))
        xs.append(x)
        ys.append(np.asarray(y, dtype="uint8"))
    x_train, y_train = np.concatenate(xs).astype("uint8"), np.concatenate(ys).reshape(-1, 1)
    x_test, y_test = load_batch(os.path.join(path, "test_batch"))
    y_test = np.asarray(y_test, dtype=y_train.dtype).reshape(-1, 1)
    x_test = x_test.astype(x_train.dtype)
    if config.image_data_format() == "channels_last":
        x_train, x_test = x_train.transpose(0, 2, 3, 1), x_test.transpose(0, 2, 3, 1)
    return (x_train, y_train), (x_test, y_test)
