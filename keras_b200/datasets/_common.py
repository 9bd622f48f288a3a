"""Shared pieces of the dataset loaders: download origin, guarded unpickling, split and token post-processing."""

import io
import pickle
import zipfile

import numpy as np

ORIGIN = "https://storage.googleapis.com/tensorflow/tf-keras-datasets/"

_SAFE_GLOBALS = frozenset({("numpy", "ndarray"), ("numpy", "dtype"), ("numpy.core.multiarray", "_reconstruct"), ("numpy._core.multiarray", "_reconstruct")})


class RestrictedUnpickler(pickle.Unpickler):
    """Unpickler that only reconstructs NumPy arrays (object arrays of token lists, CIFAR batches)."""

    def find_class(self, module, name):
        if (module, name) in _SAFE_GLOBALS:
            return super().find_class(module, name)
        raise pickle.UnpicklingError(f"Refusing to deserialize `{module}.{name}` while loading a Keras dataset. The file may be corrupted or malicious.")


def load_npz(path):
    """Arrays of an ``.npz`` archive; object arrays go through ``RestrictedUnpickler``."""
    out = {}
    with zipfile.ZipFile(path) as archive:
        for member in archive.namelist():
            if not member.endswith(".npy"):
                continue
            buf = io.BytesIO(archive.read(member))
            try:
                arr = np.lib.format.read_array(buf, allow_pickle=False)
            except ValueError:
                buf.seek(0)
                version = np.lib.format.read_magic(buf)
                if version[0] == 1:
                    np.lib.format.read_array_header_1_0(buf)
                elif version[0] in (2, 3):
                    np.lib.format.read_array_header_2_0(buf)
                else:
                    raise ValueError(f"Unsupported `.npy` file version: {version}.")
                arr = RestrictedUnpickler(buf).load()
            out[member[:-4]] = arr
    return out


def shuffled_split(x, y, test_split, seed):
    if not (0 <= test_split < 1):
        raise ValueError(f"Invalid `test_split` argument: {test_split}. It must be between 0 and 1 (exclusive of 1).")
    order = np.arange(len(x))
    np.random.RandomState(seed).shuffle(order)
    x, y = x[order], y[order]
    cut = int(len(x) * (1 - test_split))
    return (np.array(x[:cut]), np.array(y[:cut])), (np.array(x[cut:]), np.array(y[cut:]))


def remove_long_seq(maxlen, seq, label):
    new_seq, new_label = [], []
    for x, y in zip(seq, label):
        if len(x) < maxlen:
            new_seq.append(x)
            new_label.append(y)
    return new_seq, new_label


def shift_tokens(xs, start_char, index_from):
    if start_char is not None:
        return [[start_char] + [w + index_from for w in x] for x in xs]
    if index_from:
        return [[w + index_from for w in x] for x in xs]
    return [list(x) for x in xs]


def restrict_vocabulary(xs, num_words, skip_top, oov_char):
    if not num_words:
        num_words = max(max(x) for x in xs)
    if oov_char is not None:
        return [[w if skip_top <= w < num_words else oov_char for w in x] for x in xs]
    return [[w for w in x if skip_top <= w < num_words] for x in xs]
