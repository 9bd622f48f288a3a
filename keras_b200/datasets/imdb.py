"""IMDB sentiment (keras/src/datasets/imdb.py)."""

import json

import numpy as np

from keras_b200.core.export_registry import keras_export
from keras_b200.datasets import _common as c
from keras_b200.utils.file_utils import get_file


@keras_export("keras.datasets.imdb.load_data")
def load_data(path="imdb.npz", num_words=None, skip_top=0, maxlen=None, seed=113, start_char=1, oov_char=2, index_from=3, **kwargs):
    path = get_file(fname=path, origin=c.ORIGIN + "imdb.npz", file_hash="69664113be75683a8fe16e3ed0ab59fda8886cb3cd7ada244f7d9544e4676b9f")
    f = c.load_npz(path)
    x_train, labels_train, x_test, labels_test = f["x_train"], f["y_train"], f["x_test"], f["y_test"]
    rng = np.random.RandomState(seed)
    order = np.arange(len(x_train))
    rng.shuffle(order)
    x_train, labels_train = x_train[order], labels_train[order]
    order = np.arange(len(x_test))
    rng.shuffle(order)
    x_test, labels_test = x_test[order], labels_test[order]
    x_train = c.shift_tokens(x_train, start_char, index_from)
    x_test = c.shift_tokens(x_test, start_char, index_from)
    if maxlen:
        x_train, labels_train = c.remove_long_seq(maxlen, x_train, labels_train)
        x_test, labels_test = c.remove_long_seq(maxlen, x_test, labels_test)
        if not x_train or not x_test:
            raise ValueError(f"After filtering for sequences shorter than maxlen={str(maxlen)}, no sequence was kept. Increase maxlen.")
    xs = c.restrict_vocabulary(x_train + x_test, num_words, skip_top, oov_char)
    labels = np.concatenate([labels_train, labels_test])
    n = len(x_train)
    return (np.array(xs[:n], dtype="object"), labels[:n]), (np.array(xs[n:], dtype="object"), labels[n:])


@keras_export("keras.datasets.imdb.get_word_index")
def get_word_index(path="imdb_word_index.json"):
    path = get_file(fname=path, origin=c.ORIGIN + "imdb_word_index.json", file_hash="bfafd718b763782e994055a2d397834f")
    with open(path) as f:
        return json.load(f)
