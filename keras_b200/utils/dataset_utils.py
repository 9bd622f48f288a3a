"""Dataset helpers: ``split_dataset``, ``image/text/audio_dataset_from_directory``, ``timeseries_dataset_from_array``
(keras/src/utils/{dataset_utils,image_dataset_utils,text_dataset_utils,audio_dataset_utils,timeseries_dataset_utils}.py).

The reference builds ``tf.data`` (or grain) pipelines.  Here the result is a ``Dataset``: a re-iterable, lazily
evaluated pipeline of NumPy batches with ``map / batch / unbatch / shuffle / take / skip / prefetch / repeat``,
decoded by a thread pool and accepted directly by ``Model.fit``.
"""

import itertools
import os
import random as _pyrandom
import warnings
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from keras_b200 import tree
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.utils import io_utils


class Dataset:
    """Re-iterable pipeline of (structures of) NumPy arrays."""

    def __init__(self, make_iter, length=None):
        self._make_iter = make_iter
        self._length = length

    def __iter__(self):
        return iter(self._make_iter())

    def __len__(self):
        if self._length is None:
            raise TypeError("The length of this dataset is unknown.")
        return self._length

    def cardinality(self):
        return -2 if self._length is None else self._length

    @classmethod
    def from_tensor_slices(cls, data):
        flat = tree.flatten(data)
        n = len(flat[0])

        def gen():
            for i in range(n):
                yield tree.map_structure(lambda a: np.asarray(a)[i] if not isinstance(a, (list, tuple)) else a[i], data) if False else tree.pack_sequence_as(data, [f[i] for f in flat])

        return cls(gen, n)

    @classmethod
    def from_generator(cls, generator_fn, length=None):
        return cls(generator_fn, length)

    def map(self, fn, num_parallel_calls=None):
        src = self

        def gen():
            if num_parallel_calls and num_parallel_calls > 1:
                with ThreadPoolExecutor(num_parallel_calls) as pool:
                    it = iter(src)
                    while True:
                        chunk = list(itertools.islice(it, num_parallel_calls * 4))
                        if not chunk:
                            return
                        for out in pool.map(lambda e: fn(*e) if isinstance(e, tuple) else fn(e), chunk):
                            yield out
            else:
                for e in src:
                    yield fn(*e) if isinstance(e, tuple) else fn(e)

        return Dataset(gen, self._length)

    def batch(self, batch_size, drop_remainder=False):
        src = self

        def gen():
            buf = []
            for e in src:
                buf.append(e)
                if len(buf) == batch_size:
                    yield _stack(buf)
                    buf = []
            if buf and not drop_remainder:
                yield _stack(buf)

        length = None
        if self._length is not None:
            length = self._length // batch_size if drop_remainder else -(-self._length // batch_size)
        return Dataset(gen, length)

    def unbatch(self):
        src = self

        def gen():
            for b in src:
                flat = tree.flatten(b)
                for i in range(len(flat[0])):
                    yield tree.pack_sequence_as(b, [f[i] for f in flat])

        return Dataset(gen, None)

    def shuffle(self, buffer_size, seed=None, reshuffle_each_iteration=True):
        src = self
        state = {"epoch": 0}

        def gen():
            rng = _pyrandom.Random(None if seed is None else seed + (state["epoch"] if reshuffle_each_iteration else 0))
            state["epoch"] += 1
            buf = []
            for e in src:
                buf.append(e)
                if len(buf) >= buffer_size:
                    i = rng.randrange(len(buf))
                    buf[i], buf[-1] = buf[-1], buf[i]
                    yield buf.pop()
            rng.shuffle(buf)
            yield from buf

        return Dataset(gen, self._length)

    def take(self, n):
        src = self
        return Dataset(lambda: itertools.islice(iter(src), n), None if self._length is None else min(n, self._length))

    def skip(self, n):
        src = self
        return Dataset(lambda: itertools.islice(iter(src), n, None), None if self._length is None else max(self._length - n, 0))

    def repeat(self, count=None):
        src = self

        def gen():
            i = 0
            while count is None or i < count:
                yield from src
                i += 1

        return Dataset(gen, None if count is None or self._length is None else self._length * count)

    def prefetch(self, buffer_size=2):
        src = self

        def gen():
            import queue
            import threading

            q = queue.Queue(maxsize=max(int(buffer_size) if buffer_size and buffer_size > 0 else 2, 1))
            stop = object()

            def work():
                try:
                    for e in src:
                        q.put(e)
                    q.put(stop)
                except BaseException as exc:  # surfaced in the consumer
                    q.put(exc)

            threading.Thread(target=work, daemon=True).start()
            while True:
                e = q.get()
                if e is stop:
                    return
                if isinstance(e, BaseException):
                    raise e
                yield e

        return Dataset(gen, self._length)

    def cache(self):
        store = []
        src = self

        def gen():
            if store:
                yield from store
                return
            tmp = []
            for e in src:
                tmp.append(e)
                yield e
            store.extend(tmp)

        return Dataset(gen, self._length)

    def as_numpy_iterator(self):
        return iter(self)


def _stack(elements):
    first = elements[0]
    flats = [tree.flatten(e) for e in elements]
    cols = []
    for j in range(len(flats[0])):
        vals = [f[j] for f in flats]
        if isinstance(vals[0], (str, bytes)):
            cols.append(np.array(vals, dtype=object))
        else:
            cols.append(np.stack([np.asarray(v) for v in vals]))
    return tree.pack_sequence_as(first, cols)


# ------------------------------------------------------------------------------- split_dataset
@keras_export("keras.utils.split_dataset")
def split_dataset(dataset, left_size=None, right_size=None, shuffle=False, seed=None, preferred_backend=None):
    """Split arrays / tuples of arrays / ``Dataset`` / torch datasets into two ``Dataset`` objects of samples."""
    samples = _convert_dataset_to_list(dataset)
    if shuffle:
        if seed is None:
            seed = _pyrandom.randint(0, int(1e6))
        _pyrandom.Random(seed).shuffle(samples)
    total = len(samples)
    left_size, right_size = _rescale_dataset_split_sizes(left_size, right_size, total)
    left, right = samples[:left_size], samples[-right_size:]
    return Dataset.from_tensor_slices(_restore(left)), Dataset.from_tensor_slices(_restore(right))


def _restore(samples):
    if not samples:
        return np.zeros((0,))
    if isinstance(samples[0], tuple):
        return tuple(np.stack([np.asarray(s[i]) for s in samples]) for i in range(len(samples[0])))
    if isinstance(samples[0], dict):
        return {k: np.stack([np.asarray(s[k]) for s in samples]) for k in samples[0]}
    return np.stack([np.asarray(s) for s in samples])


def _convert_dataset_to_list(dataset):
    import torch

    if isinstance(dataset, (tuple, list)) and dataset and all(isinstance(a, (np.ndarray, torch.Tensor)) for a in dataset):
        arrays = [np.asarray(a.cpu()) if isinstance(a, torch.Tensor) else a for a in dataset]
        n = {len(a) for a in arrays}
        if len(n) != 1:
            raise ValueError(f"Received a tuple of NumPy arrays with different lengths. Mismatch found at index 1, Expected shape={arrays[0].shape} Received shape={arrays[1].shape}.")
        return [tuple(a[i] for a in arrays) for i in range(len(arrays[0]))]
    if isinstance(dataset, np.ndarray):
        return list(dataset)
    if isinstance(dataset, torch.Tensor):
        return list(dataset.cpu().numpy())
    if isinstance(dataset, Dataset):
        out = []
        for e in dataset:
            out.append(e)
        if out:
            first = tree.flatten(out[0])[0]
            if hasattr(first, "ndim") and first.ndim >= 1 and dataset._length is not None and False:
                pass
        return out
    if isinstance(dataset, torch.utils.data.Dataset):
        return [tuple(np.asarray(v) for v in dataset[i]) if isinstance(dataset[i], (tuple, list)) else np.asarray(dataset[i]) for i in range(len(dataset))]
    if hasattr(dataset, "__iter__"):
        return list(dataset)
    raise TypeError(f"The `dataset` argument must be either a `Dataset`, a `torch.utils.data.Dataset` object, or a list/tuple of arrays. Received: dataset={dataset} of type {type(dataset)}")


def _rescale_dataset_split_sizes(left_size, right_size, total_length):
    left_size_type, right_size_type = type(left_size), type(right_size)
    if left_size is None and right_size is None:
        raise ValueError("At least one of the `left_size` or `right_size` must be specified. Received: left_size=None and right_size=None")
    if (left_size is not None and left_size_type not in [int, float]) and (right_size is not None and right_size_type not in [int, float]):
        raise TypeError(f"Invalid `left_size` and `right_size` Types. Expected: integer or float or None, Received: type(left_size)={left_size_type} and type(right_size)={right_size_type}")
    if left_size is not None and left_size_type not in [int, float]:
        raise TypeError(f"Invalid `left_size` Type. Expected: int or float or None, Received: type(left_size)={left_size_type}.  ")
    if right_size is not None and right_size_type not in [int, float]:
        raise TypeError(f"Invalid `right_size` Type. Expected: int or float or None,Received: type(right_size)={right_size_type}.")
    if left_size == 0 and right_size == 0:
        raise ValueError("Both `left_size` and `right_size` are zero. At least one of the split sizes must be non-zero.")
    if left_size_type is int and (left_size <= 0 or left_size >= total_length) or left_size_type is float and (left_size <= 0 or left_size >= 1):
        raise ValueError(f"`left_size` should be either a positive integer smaller than {total_length}, or a float within the range `[0, 1]`. Received: left_size={left_size}")
    if right_size_type is int and (right_size <= 0 or right_size >= total_length) or right_size_type is float and (right_size <= 0 or right_size >= 1):
        raise ValueError(f"`right_size` should be either a positive integer and smaller than {total_length} or a float within the range `[0, 1]`. Received: right_size={right_size}")
    if right_size_type is left_size_type is float and right_size + left_size > 1:
        raise ValueError("The sum of `left_size` and `right_size` is greater than 1. It must be less than or equal to 1.")
    if left_size_type is float:
        left_size = round(left_size * total_length)
    elif left_size_type is int:
        left_size = float(left_size)
    if right_size_type is float:
        right_size = round(right_size * total_length)
    elif right_size_type is int:
        right_size = float(right_size)
    if left_size is None:
        left_size = total_length - right_size
    elif right_size is None:
        right_size = total_length - left_size
    if left_size + right_size > total_length:
        raise ValueError(f"The sum of `left_size` and `right_size` should be smaller than the {total_length}. Received: left_size + right_size = {left_size + right_size}and total_length = {total_length}")
    for split, side in [(left_size, "left"), (right_size, "right")]:
        if split == 0:
            raise ValueError(f"With `dataset` of length={total_length}, `left_size`={left_size} and `right_size`={right_size}.Resulting {side} side dataset split will be empty. Adjust any of the aforementioned parameters")
    return int(left_size), int(right_size)


# ------------------------------------------------------------------------ directory indexing
def index_directory(directory, labels, formats, class_names=None, shuffle=True, seed=None, follow_links=False, verbose=True):
    """List files below ``directory``; returns ``(file_paths, labels, class_names)``."""
    if labels == "inferred":
        subdirs = sorted(d for d in os.listdir(directory) if os.path.isdir(os.path.join(directory, d)) and not d.startswith("."))
        if class_names is not None:
            if not set(class_names).issubset(set(subdirs)):
                raise ValueError(f"The `class_names` passed did not match the names of the subdirectories of the target directory. Expected: {subdirs} (or a subset of it), but received: class_names={class_names}")
            subdirs = list(class_names)
    else:
        subdirs = [""]
        if class_names is not None:
            if labels is None:
                raise ValueError("When `labels=None` (no labels), argument `class_names` cannot be specified.")
            raise ValueError(f"When argument `labels` is specified, argument `class_names` cannot be specified (the `class_names` will be the sorted list of labels).")
    class_names = subdirs
    class_indices = dict(zip(class_names, range(len(class_names))))
    filenames, file_labels = [], []
    for sub in subdirs:
        root = os.path.join(directory, sub)
        found = []
        for dirpath, _, files in sorted(os.walk(root, followlinks=follow_links)):
            for f in sorted(files):
                if f.lower().endswith(tuple(formats)):
                    found.append(os.path.join(dirpath, f))
        filenames += found
        file_labels += [class_indices.get(sub, 0)] * len(found)
    if labels not in ("inferred", None):
        if len(labels) != len(filenames):
            raise ValueError(f"Expected the lengths of `labels` to match the number of files in the target directory. len(labels) is {len(labels)} while we found {len(filenames)} files in directory {directory}.")
        class_names = [str(label) for label in sorted(set(labels))]
        file_labels = list(labels)
    if verbose:
        if labels is None:
            io_utils.print_msg(f"Found {len(filenames)} files.")
        else:
            io_utils.print_msg(f"Found {len(filenames)} files belonging to {len(class_names)} classes.")
    if shuffle:
        if seed is None:
            seed = np.random.randint(1e6)
        rng = np.random.RandomState(seed)
        rng.shuffle(filenames)
        rng = np.random.RandomState(seed)
        rng.shuffle(file_labels)
    return filenames, (None if labels is None else file_labels), class_names


def get_training_or_validation_split(samples, labels, validation_split, subset):
    if not validation_split:
        return samples, labels
    num_val = int(validation_split * len(samples))
    if subset == "training":
        io_utils.print_msg(f"Using {len(samples) - num_val} files for training.")
        samples = samples[:-num_val]
        labels = labels[:-num_val] if labels is not None else None
    elif subset == "validation":
        io_utils.print_msg(f"Using {num_val} files for validation.")
        samples = samples[-num_val:]
        labels = labels[-num_val:] if labels is not None else None
    else:
        raise ValueError(f'`subset` must be either "training" or "validation", received: {subset}')
    return samples, labels


def _encode_label(label, label_mode, num_classes):
    if label_mode == "int":
        return np.int32(label)
    if label_mode == "binary":
        return np.array([label], dtype="float32")
    if label_mode == "categorical":
        out = np.zeros((num_classes,), dtype="float32")
        out[int(label)] = 1.0
        return out
    raise ValueError(f'`label_mode` argument must be one of "int", "categorical", "binary", or None. Received: label_mode={label_mode}')


def check_validation_split_arg(validation_split, subset, shuffle, seed):
    if validation_split and not 0 < validation_split < 1:
        raise ValueError(f"`validation_split` must be between 0 and 1, received: {validation_split}")
    if (validation_split or subset) and not (validation_split and subset):
        raise ValueError("If `subset` is set, `validation_split` must be set, and inversely.")
    if subset not in ("training", "validation", "both", None):
        raise ValueError(f'`subset` must be either "training", "validation" or "both", received: {subset}')
    if validation_split and shuffle and seed is None:
        raise ValueError("If using `validation_split` and shuffling the data, you must provide a `seed` argument, to make sure that there is no overlap between the training and validation subset.")


def _files_dataset(paths, labels, label_mode, num_classes, load_fn, batch_size, shuffle, seed, workers=8):
    n = len(paths)

    def make():
        order = list(range(n))
        if shuffle:
            _pyrandom.Random(seed).shuffle(order)
        with ThreadPoolExecutor(workers) as pool:
            step = batch_size or 1
            for s in range(0, n, step):
                idx = order[s:s + step]
                items = list(pool.map(lambda i: load_fn(paths[i]), idx))
                if batch_size is None:
                    x = items[0]
                    yield (x, _encode_label(labels[idx[0]], label_mode, num_classes)) if label_mode else x
                else:
                    x = _stack(items) if not isinstance(items[0], (str, bytes)) else np.array(items, dtype=object)
                    if label_mode:
                        yield x, np.stack([_encode_label(labels[i], label_mode, num_classes) for i in idx])
                    else:
                        yield x

    length = n if batch_size is None else -(-n // batch_size)
    return Dataset(make, length)


def _directory_dataset(directory, labels, label_mode, class_names, formats, load_fn, batch_size, shuffle, seed, validation_split, subset, follow_links, verbose):
    if labels not in ("inferred", None):
        if not isinstance(labels, (list, tuple)):
            raise ValueError(f'`labels` argument should be a list/tuple of integer labels, of the same size as the number of files in the target directory. If you wish to infer the labels from the subdirectory names in the target directory, pass `labels="inferred"`. If you wish to get a dataset that only contains data (no labels), pass `labels=None`. Received: labels={labels}')
        if class_names:
            raise ValueError(f"You can only pass `class_names` if `labels='inferred'`. Received: labels={labels}, and class_names={class_names}")
    if label_mode not in {"int", "categorical", "binary", None}:
        raise ValueError(f'`label_mode` argument must be one of "int", "categorical", "binary", or None. Received: label_mode={label_mode}')
    if labels is None or label_mode is None:
        labels = None
        label_mode = None
    check_validation_split_arg(validation_split, subset, shuffle, seed)
    if seed is None:
        seed = np.random.randint(1e6)
    paths, file_labels, class_names = index_directory(directory, labels, formats=formats, class_names=class_names, shuffle=shuffle, seed=seed,
                                                      follow_links=follow_links, verbose=verbose)
    if label_mode == "binary" and len(class_names) != 2:
        raise ValueError(f'When passing `label_mode="binary"`, there must be exactly 2 class_names. Received: class_names={class_names}')
    num_classes = len(class_names) if class_names else 0

    def build(sub):
        p, l = get_training_or_validation_split(paths, file_labels, validation_split, sub)
        if not p:
            raise ValueError(f"No files found in directory {directory}. Allowed formats: {formats}")
        ds = _files_dataset(p, l, label_mode, num_classes, load_fn, batch_size, shuffle, seed)
        ds.class_names = class_names
        ds.file_paths = p
        return ds

    if subset == "both":
        return [build("training"), build("validation")]
    return build(subset)


IMAGE_FORMATS = (".bmp", ".gif", ".jpeg", ".jpg", ".png")


@keras_export(["keras.utils.image_dataset_from_directory", "keras.preprocessing.image_dataset_from_directory"])
def image_dataset_from_directory(directory, labels="inferred", label_mode="int", class_names=None, color_mode="rgb", batch_size=32,
                                 image_size=(256, 256), shuffle=True, seed=None, validation_split=None, subset=None, interpolation="bilinear",
                                 follow_links=False, crop_to_aspect_ratio=False, pad_to_aspect_ratio=False, data_format=None, format="tf",
                                 verbose=True):
    from keras_b200.utils import image_utils

    if color_mode not in ("rgb", "rgba", "grayscale"):
        raise ValueError(f'`color_mode` must be one of {{"rgb", "rgba", "grayscale"}}. Received: color_mode={color_mode}')
    if crop_to_aspect_ratio and pad_to_aspect_ratio:
        raise ValueError("Only one of `pad_to_aspect_ratio`, `crop_to_aspect_ratio` can be set to `True`.")
    data_format = config.standardize_data_format(data_format)

    def load(path):
        img = image_utils.load_img(path, color_mode=color_mode, target_size=None if pad_to_aspect_ratio else image_size,
                                   interpolation=interpolation, keep_aspect_ratio=crop_to_aspect_ratio)
        arr = image_utils.img_to_array(img, data_format="channels_last", dtype="float32")
        if pad_to_aspect_ratio:
            from keras_b200 import ops
            from keras_b200.core.tensor import convert_to_numpy

            arr = convert_to_numpy(ops.image.resize(arr, image_size, interpolation=interpolation, pad_to_aspect_ratio=True, data_format="channels_last"))
        if data_format == "channels_first":
            arr = arr.transpose(2, 0, 1)
        return arr

    return _directory_dataset(directory, labels, label_mode, class_names, IMAGE_FORMATS, load, batch_size, shuffle, seed, validation_split,
                              subset, follow_links, verbose)


@keras_export(["keras.utils.text_dataset_from_directory", "keras.preprocessing.text_dataset_from_directory"])
def text_dataset_from_directory(directory, labels="inferred", label_mode="int", class_names=None, batch_size=32, max_length=None, shuffle=True,
                                seed=None, validation_split=None, subset=None, follow_links=False, format="tf", verbose=True):
    def load(path):
        with open(path, "r", encoding="utf-8", errors="ignore") as f:
            s = f.read()
        return s[:max_length] if max_length is not None else s

    return _directory_dataset(directory, labels, label_mode, class_names, (".txt",), load, batch_size, shuffle, seed, validation_split, subset,
                              follow_links, verbose)


@keras_export("keras.utils.audio_dataset_from_directory")
def audio_dataset_from_directory(directory, labels="inferred", label_mode="int", class_names=None, batch_size=32, sampling_rate=None,
                                 output_sequence_length=None, ragged=False, shuffle=True, seed=None, validation_split=None, subset=None,
                                 follow_links=False, verbose=True):
    if sampling_rate is not None:
        if not isinstance(sampling_rate, int):
            raise ValueError(f"`sampling_rate` should have an integer value. Received: sampling_rate={sampling_rate}")
        if sampling_rate <= 0:
            raise ValueError(f"`sampling_rate` should be higher than 0. Received: sampling_rate={sampling_rate}")
    if ragged and output_sequence_length is not None:
        raise ValueError("Cannot set both `ragged` and `output_sequence_length`")

    def load(path):
        from scipy.io import wavfile

        rate, data = wavfile.read(path)
        if data.dtype.kind == "i":
            data = data.astype("float32") / float(np.iinfo(data.dtype).max + 1)
        elif data.dtype.kind == "u":
            data = (data.astype("float32") - 128.0) / 128.0
        data = data.astype("float32")
        if data.ndim == 1:
            data = data[:, None]
        if sampling_rate is not None and rate != sampling_rate:
            from scipy import signal

            data = signal.resample_poly(data, sampling_rate, rate, axis=0).astype("float32")
        if output_sequence_length is not None:
            if data.shape[0] >= output_sequence_length:
                data = data[:output_sequence_length]
            else:
                data = np.pad(data, ((0, output_sequence_length - data.shape[0]), (0, 0)))
        return data

    if output_sequence_length is None and not ragged and batch_size is not None:
        inner = load

        def load_padded(path):
            return inner(path)

        ds = _directory_dataset(directory, labels, label_mode, class_names, (".wav",), load_padded, None, shuffle, seed, validation_split, subset,
                                follow_links, verbose)

        def pad_batch(d):
            def make():
                buf = []
                for e in d:
                    buf.append(e)
                    if len(buf) == batch_size:
                        yield _pad_audio(buf)
                        buf = []
                if buf:
                    yield _pad_audio(buf)

            out = Dataset(make, -(-len(d) // batch_size))
            out.class_names, out.file_paths = d.class_names, d.file_paths
            return out

        return [pad_batch(d) for d in ds] if isinstance(ds, list) else pad_batch(ds)
    return _directory_dataset(directory, labels, label_mode, class_names, (".wav",), load, batch_size, shuffle, seed, validation_split, subset,
                              follow_links, verbose)


def _pad_audio(elements):
    has_label = isinstance(elements[0], tuple)
    xs = [e[0] if has_label else e for e in elements]
    n = max(x.shape[0] for x in xs)
    x = np.stack([np.pad(a, ((0, n - a.shape[0]), (0, 0))) for a in xs])
    if has_label:
        return x, np.stack([e[1] for e in elements])
    return x


@keras_export(["keras.utils.timeseries_dataset_from_array", "keras.preprocessing.timeseries_dataset_from_array"])
def timeseries_dataset_from_array(data, targets, sequence_length, sequence_stride=1, sampling_rate=1, batch_size=128, shuffle=False, seed=None,
                                  start_index=None, end_index=None):
    if start_index:
        if start_index < 0:
            raise ValueError(f"`start_index` must be 0 or greater. Received: start_index={start_index}")
        if start_index >= len(data):
            raise ValueError(f"`start_index` must be lower than the length of the data. Received: start_index={start_index}, for data of length {len(data)}")
    if end_index:
        if start_index and end_index <= start_index:
            raise ValueError(f"`end_index` must be higher than `start_index`. Received: start_index={start_index}, and end_index={end_index} ")
        if end_index >= len(data):
            raise ValueError(f"`end_index` must be lower than the length of the data. Received: end_index={end_index}, for data of length {len(data)}")
        if end_index <= 0:
            raise ValueError(f"`end_index` must be higher than 0. Received: end_index={end_index}")
    if sampling_rate <= 0:
        raise ValueError(f"`sampling_rate` must be higher than 0. Received: sampling_rate={sampling_rate}")
    if sampling_rate >= len(data):
        raise ValueError(f"`sampling_rate` must be lower than the length of the data. Received: sampling_rate={sampling_rate}, for data of length {len(data)}")
    if sequence_stride <= 0:
        raise ValueError(f"`sequence_stride` must be higher than 0. Received: sequence_stride={sequence_stride}")
    if sequence_stride >= len(data):
        raise ValueError(f"`sequence_stride` must be lower than the length of the data. Received: sequence_stride={sequence_stride}, for data of length {len(data)}")
    if start_index is None:
        start_index = 0
    if end_index is None:
        end_index = len(data)
    data = np.asarray(data)
    num_seqs = end_index - start_index - (sequence_length - 1) * sampling_rate
    if targets is not None:
        targets = np.asarray(targets)
        num_seqs = min(num_seqs, len(targets))
    if num_seqs <= 0:
        starts = np.zeros((0,), dtype="int64")
    else:
        starts = np.arange(0, num_seqs, sequence_stride, dtype="int64")
    offsets = np.arange(0, sequence_length * sampling_rate, sampling_rate)
    n = len(starts)

    def make():
        order = starts.copy()
        if shuffle:
            np.random.RandomState(seed if seed is not None else np.random.randint(1e6)).shuffle(order)
        step = batch_size or 1
        for s in range(0, n, step):
            idx = order[s:s + step] + start_index
            x = data[idx[:, None] + offsets[None, :]]
            if batch_size is None:
                x = x[0]
            if targets is not None:
                y = targets[idx - start_index + start_index] if False else targets[idx]
                yield (x, y if batch_size is not None else y[0])
            else:
                yield x

    return Dataset(make, n if batch_size is None else -(-n // batch_size))
