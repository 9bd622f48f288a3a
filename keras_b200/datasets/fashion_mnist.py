"""Fashion-MNIST (keras/src/datasets/fashion_mnist.py): four gzip'd IDX files."""

import gzip
import os

import numpy as np

from keras_b200.core.export_registry import keras_export
from keras_b200.datasets._common import ORIGIN
from keras_b200.utils.file_utils import get_file


def _idx(path, offset, shape=None):
    with gzip.open(path, "rb") as f:
        a = np.frombuffer(f.read(), np.uint8, offset=offset)
    return a if shape is None else a.reshape(shape)


@keras_export("keras.datasets.fashion_mnist.load_data")
def load_data():
    sub = os.path.join("datasets", "fashion-mnist")
    names = ["train-labels-idx1-ubyte.gz", "train-images-idx3-ubyte.gz", "t10k-labels-idx1-ubyte.gz", "t10k-images-idx3-ubyte.gz"]
    p = [get_file(n, origin=ORIGIN + n, cache_subdir=sub) for n in names]
    y_train = _idx(p[0], 8)
    x_train = _idx(p[1], 16, (len(y_train), 28, 28))
    y_test = _idx(p[2], 8)
    x_test = _idx(p[3], 16, (len(y_test), 28, 28))
    return (x_train, y_train), (x_test, y_test)
