"""Reuters newswire topics (keras/src/datasets/reuters.py)."""

import json

import numpy as np

from keras_b200.core.export_registry import keras_export
from keras_b200.datasets import _common as c
from keras_b200.utils.file_utils import get_file

_LABELS = ("cocoa grain veg-oil earn acq wheat copper housing money-supply coffee sugar trade reserves ship cotton carcass crude nat-gas cpi money-fx "
           "interest gnp meal-feed alum oilseed gold tin strategic-metal livestock retail ipi iron-steel rubber heat jobs lei bop zinc orange pet-chem "
           "dlr gas silver wpi hog lead")


@keras_export("keras.datasets.reuters.load_data")
def load_data(path="reuters.npz", num_words=None, skip_top=0, maxlen=None, test_split=0.2, seed=113, start_char=1, oov_char=2, index_from=3):
    path = get_file(fname=path, origin=c.ORIGIN + "reuters.npz", file_hash="d6586e694ee56d7a4e65172e12b3e987c03096cb01eab99753921ef915959916")
    f = c.load_npz(path)
    xs, labels = f["x"], f["y"]
    order = np.arange(len(xs))
    np.random.RandomState(seed).shuffle(order)
    xs, labels = xs[order], labels[order]
    xs = c.shift_tokens(xs, start_char, index_from) if (start_char is not None or index_from) else xs
    if maxlen:
        xs, labels = c.remove_long_seq(maxlen, xs, labels)
    xs = c.restrict_vocabulary(xs, num_words, skip_top, oov_char)
    cut = int(len(xs) * (1 - test_split))
    return (np.array(xs[:cut], dtype="object"), np.array(labels[:cut])), (np.array(xs[cut:], dtype="object"), np.array(labels[cut:]))


@keras_export("keras.datasets.reuters.get_word_index")
def get_word_index(path="reuters_word_index.json"):
    path = get_file(path, origin=c.ORIGIN + "reuters_word_index.json", file_hash="4d44cc38712099c9e383dc6e5f11a921")
    with open(path) as f:
        return json.load(f)


@keras_export("keras.datasets.reuters.get_label_names")
def get_label_names():
    return tuple(_LABELS.split())
