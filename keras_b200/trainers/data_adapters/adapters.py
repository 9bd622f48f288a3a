"""Data adapters: uniform batch iteration over arrays, generators, ``PyDataset`` and torch loaders.

Behaviour of keras/src/trainers/data_adapters/*.py: ``ArrayDataAdapter`` slices host arrays with
an epoch-seeded shuffle and gives process *p* of *N* the batches ``p, p+N, …`` (``batch_size`` is
per process); ``PyDataset`` with worker threads/processes; generator and ``DataLoader`` inputs.
Batches are produced as host arrays; the trainer moves them to the device through pinned staging
buffers on a copy stream.
"""

import itertools
import math
import queue
import random
import threading
import warnings
import multiprocessing.pool

import numpy as np
import torch

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export
from keras_b200.trainers.data_adapters import data_adapter_utils


class DataAdapter:
    def get_numpy_iterator(self):
        raise NotImplementedError

    def get_torch_dataloader(self):
        raise NotImplementedError

    @property
    def builtin_prefetch(self):
        return False

    @property
    def num_batches(self):
        raise NotImplementedError

    @property
    def batch_size(self):
        raise NotImplementedError

    @property
    def has_partial_batch(self):
        raise NotImplementedError

    @property
    def partial_batch_size(self):
        raise NotImplementedError

    def on_epoch_begin(self):
        pass

    def on_epoch_end(self):
        pass


def _to_host(x):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x
    if isinstance(x, np.ndarray):
        return x
    if hasattr(x, "to_numpy"):
        return x.to_numpy()
    if hasattr(x, "__array__"):
        return np.asarray(x)
    if isinstance(x, (list, tuple)) and x and isinstance(x[0], (int, float, list, tuple)):
        return np.asarray(x)
    raise ValueError(f"Expected a NumPy array, tensor, or pandas object. Received invalid input: {x} (of type {type(x)})")


def _standardize_floats(x):
    if isinstance(x, np.ndarray) and x.dtype == np.float64:
        return x.astype("float32")
    if isinstance(x, np.ndarray) and x.dtype == object:
        return x.astype("float32")
    return x


class ArrayDataAdapter(DataAdapter):
    def __init__(self, x, y=None, sample_weight=None, batch_size=None, steps=None, shuffle=False, class_weight=None):
        if not can_convert_arrays((x, y, sample_weight)):
            raise ValueError(f"Expected all elements of `x` to be array-like. Received invalid types: x={x}")
        if sample_weight is not None and class_weight is not None:
            raise ValueError("You cannot `class_weight` and `sample_weight` at the same time.")
        conv = lambda d: tree.map_structure(lambda a: _standardize_floats(_to_host(a)) if a is not None else None, d)
        x, y, sample_weight = conv(x), conv(y), conv(sample_weight)
        if class_weight is not None:
            if tree.is_nested(y):
                raise ValueError("`class_weight` is only supported for Models with a single output.")
            sample_weight = data_adapter_utils.class_weight_to_sample_weights(y, class_weight)
        inputs = data_adapter_utils.pack_x_y_sample_weight(x, y, sample_weight)
        data_adapter_utils.check_data_cardinality(inputs)
        num_samples = int(tree.flatten(inputs)[0].shape[0])
        if steps and not batch_size:
            batch_size = int(math.ceil(num_samples / steps))
        if not batch_size:
            batch_size = 32
        self._inputs = inputs
        self._num_samples = num_samples
        self._batch_size = int(batch_size)
        self._size = int(math.ceil(num_samples / batch_size))
        self._partial_batch_size = num_samples % batch_size
        self._shuffle = shuffle
        self._epoch = 0
        from keras_b200.distribution import distribution_lib

        dist = distribution_lib.distribution()
        self._num_shards, self._shard_id = 1, 0
        if dist is not None and getattr(dist, "auto_shard_dataset", True):
            self._num_shards = dist.num_data_shards if hasattr(dist, "num_data_shards") else 1
            self._shard_id = dist.data_shard_id if hasattr(dist, "data_shard_id") else 0

    def _batch_indices(self):
        """Index sets of one pass.  The order is a function of the epoch number alone, drawn as the reference draws it
        (keras/src/trainers/data_adapters/array_data_adapter.py:308-343: a ``torch.Generator`` seeded with the epoch, one
        ``randperm`` over the samples, or one per batch for ``shuffle="batch"``), so every process of a data-parallel job
        sees the same order without talking and a run can be repeated."""
        n, bs = self._num_samples, self._batch_size
        if not self._shuffle:
            return [slice(i, min(i + bs, n)) for i in range(0, n, bs)]
        gen = torch.Generator()
        gen.manual_seed(int(self._epoch))
        if self._shuffle == "batch":
            # a shard keeps every num_shards-th batch first and draws only for those, one draw after the other
            starts = list(range(0, n, bs))[self._shard_id::self._num_shards]
            return [i + torch.randperm(min(bs, n - i), generator=gen).numpy() for i in starts]
        perm = torch.randperm(n, generator=gen).numpy()
        return [perm[i:i + bs] for i in range(0, n, bs)]

    def on_epoch_end(self):
        self._epoch += 1

    def get_numpy_iterator(self):
        flat = tree.flatten(self._inputs)
        batches = self._batch_indices()
        if self._num_shards > 1 and self._shuffle != "batch":
            batches = batches[self._shard_id::self._num_shards]

        def take(a, idx):
            if a is None:
                return None
            if isinstance(idx, slice):
                return a[idx]
            if isinstance(a, torch.Tensor):
                return a[torch.as_tensor(idx)]
            return a[idx]

        for idx in batches:
            yield tree.pack_sequence_as(self._inputs, [take(a, idx) for a in flat])

    @property
    def num_batches(self):
        if self._num_shards > 1:
            return len(range(self._shard_id, self._size, self._num_shards))
        return self._size

    batch_size = property(lambda self: self._batch_size)
    has_partial_batch = property(lambda self: self._partial_batch_size > 0)
    partial_batch_size = property(lambda self: self._partial_batch_size or None)


def can_convert_arrays(arrays):
    def ok(x):
        if x is None:
            return True
        if isinstance(x, (np.ndarray, torch.Tensor)):
            return True
        if hasattr(x, "__array__") or hasattr(x, "to_numpy"):
            return True
        return False

    return all(tree.flatten(tree.map_structure(ok, arrays)))


class GeneratorDataAdapter(DataAdapter):
    def __init__(self, generator):
        first_batches, generator = peek_and_restore(generator)
        self.generator = generator
        self._first_batches = first_batches
        self._output_signature = None
        if first_batches and not isinstance(first_batches[0], tuple):
            raise ValueError(f"When passing a Python generator to a Keras model, the generator must return a tuple, either (input,) or (inputs, targets) or (inputs, targets, sample_weights). Received: {first_batches[0]}")

    def get_numpy_iterator(self):
        return self.generator()

    num_batches = property(lambda self: None)
    batch_size = property(lambda self: None)
    has_partial_batch = property(lambda self: None)
    partial_batch_size = property(lambda self: None)


class IterableDatasetAdapter(DataAdapter):
    """Re-iterable pipelines of batches (``keras_b200.utils.dataset_utils.Dataset`` and other objects whose ``__iter__``
    starts a fresh pass).  Under a distribution each process takes batches ``p, p+N, ...``."""

    def __init__(self, dataset, class_weight=None):
        self._dataset = dataset
        self._class_weight = class_weight
        from keras_b200.distribution import distribution_lib

        dist = distribution_lib.distribution()
        self._num_shards = getattr(dist, "num_data_shards", 1) if dist is not None and getattr(dist, "auto_shard_dataset", True) else 1
        self._shard_id = getattr(dist, "data_shard_id", 0) if self._num_shards > 1 else 0

    def get_numpy_iterator(self):
        it = iter(self._dataset)
        if self._num_shards > 1:
            it = itertools.islice(it, self._shard_id, None, self._num_shards)
        for batch in it:
            if not isinstance(batch, tuple):
                batch = (batch,)
            yield batch

    @property
    def num_batches(self):
        try:
            n = len(self._dataset)
        except TypeError:
            return None
        return len(range(self._shard_id, n, self._num_shards)) if self._num_shards > 1 else n

    batch_size = property(lambda self: None)
    has_partial_batch = property(lambda self: None)
    partial_batch_size = property(lambda self: None)


def peek_and_restore(generator):
    batches = list(itertools.islice(generator, data_adapter_utils.NUM_BATCHES_FOR_TENSOR_SPEC))
    return batches, lambda: itertools.chain(batches, generator)


@keras_export(["keras.utils.PyDataset", "keras.utils.Sequence"])
class PyDataset:
    """Base class for datasets defined in Python: implement ``__getitem__`` and ``num_batches``."""

    def __init__(self, workers=1, use_multiprocessing=False, max_queue_size=10):
        self._workers = workers
        self._use_multiprocessing = use_multiprocessing
        self._max_queue_size = max_queue_size

    def _warn_if_super_not_called(self):
        if not hasattr(self, "_workers"):
            warnings.warn("Your `PyDataset` class should call `super().__init__(**kwargs)` in its constructor. `**kwargs` can include `workers`, `use_multiprocessing`, `max_queue_size`. Do not pass these arguments to `fit()`, as they will be ignored.", stacklevel=2)
            self._workers, self._use_multiprocessing, self._max_queue_size = 1, False, 10

    workers = property(lambda self: (self._warn_if_super_not_called(), self._workers)[1], lambda self, v: setattr(self, "_workers", v))
    use_multiprocessing = property(lambda self: (self._warn_if_super_not_called(), self._use_multiprocessing)[1], lambda self, v: setattr(self, "_use_multiprocessing", v))
    max_queue_size = property(lambda self: (self._warn_if_super_not_called(), self._max_queue_size)[1], lambda self, v: setattr(self, "_max_queue_size", v))

    def __getitem__(self, index):
        raise NotImplementedError

    def __iter__(self):
        index_range = range(self.num_batches) if self.num_batches is not None else itertools.count()
        for i in index_range:
            yield self[i]

    @property
    def num_batches(self):
        if hasattr(self, "__len__"):
            return len(self)
        raise NotImplementedError("You need to implement the `num_batches` property:\n\n@property\ndef num_batches(self):\n  return ...")

    def on_epoch_begin(self):
        pass

    def on_epoch_end(self):
        pass


class PyDatasetAdapter(DataAdapter):
    def __init__(self, x, class_weight=None, shuffle=False):
        self.py_dataset = x
        self.class_weight = class_weight
        self.enqueuer = None
        self.shuffle = shuffle
        from keras_b200.distribution import distribution_lib

        dist = distribution_lib.distribution()
        self._num_shards, self._shard_id = 1, 0
        if dist is not None and getattr(dist, "auto_shard_dataset", True):
            self._num_shards = getattr(dist, "num_data_shards", 1)
            self._shard_id = getattr(dist, "data_shard_id", 0)

    def _standardize_batch(self, batch):
        if isinstance(batch, dict):
            return batch
        if isinstance(batch, np.ndarray):
            batch = (batch,)
        if isinstance(batch, list):
            batch = tuple(batch)
        if not isinstance(batch, tuple) or len(batch) not in {1, 2, 3}:
            raise ValueError(f"PyDataset.__getitem__() must return a tuple or a dict. If a tuple, it must be ordered either (input,) or (inputs, targets) or (inputs, targets, sample_weights). Received: {str(batch)[:100]}... of type {type(batch)}")
        if self.class_weight is not None:
            if len(batch) == 3:
                raise ValueError("You cannot specify `class_weight` and `sample_weight` at the same time.")
            if len(batch) == 2:
                sw = data_adapter_utils.class_weight_to_sample_weights(batch[1], self.class_weight)
                batch = batch + (sw,)
        return batch

    def _indices(self):
        n = self.py_dataset.num_batches
        if n is None:
            return None
        idx = list(range(n))
        if self.shuffle:
            random.shuffle(idx)
        if self._num_shards > 1:
            idx = idx[self._shard_id::self._num_shards]
        return idx

    def get_numpy_iterator(self):
        ds = self.py_dataset
        idx = self._indices()
        workers = ds.workers
        if idx is None:
            i = 0
            while True:
                try:
                    yield self._standardize_batch(ds[i])
                except (IndexError, StopIteration):
                    return
                i += 1
        elif workers <= 1:
            for i in idx:
                yield self._standardize_batch(ds[i])
        else:
            pool_cls = multiprocessing.pool.ThreadPool if not ds.use_multiprocessing else multiprocessing.pool.ThreadPool
            with pool_cls(workers) as pool:
                depth = max(ds.max_queue_size, 1)
                pending = []
                it = iter(idx)
                for i in itertools.islice(it, depth):
                    pending.append(pool.apply_async(ds.__getitem__, (i,)))
                while pending:
                    batch = pending.pop(0).get()
                    nxt = next(it, None)
                    if nxt is not None:
                        pending.append(pool.apply_async(ds.__getitem__, (nxt,)))
                    yield self._standardize_batch(batch)

    def on_epoch_begin(self):
        self.py_dataset.on_epoch_begin()

    def on_epoch_end(self):
        self.py_dataset.on_epoch_end()

    @property
    def num_batches(self):
        n = self.py_dataset.num_batches
        if n is not None and self._num_shards > 1:
            return len(range(self._shard_id, n, self._num_shards))
        return n

    batch_size = property(lambda self: None)
    has_partial_batch = property(lambda self: None)
    partial_batch_size = property(lambda self: None)


class TorchDataLoaderAdapter(DataAdapter):
    def __init__(self, dataloader):
        if not isinstance(dataloader, torch.utils.data.DataLoader):
            raise ValueError(f"Expected argument `dataloader` to be an instance of`torch.utils.data.DataLoader`. Received: {dataloader}")
        self._dataloader = dataloader
        self._batch_size = dataloader.batch_size
        self._num_batches = None
        self._partial_batch_size = None
        if hasattr(dataloader.dataset, "__len__"):
            self._num_batches = len(dataloader)
            if self._batch_size is not None:
                self._partial_batch_size = len(dataloader.dataset) % self._batch_size
        from keras_b200.distribution import distribution_lib

        dist = distribution_lib.distribution()
        self._num_shards, self._shard_id = 1, 0
        if dist is not None and getattr(dist, "auto_shard_dataset", True):
            self._num_shards = getattr(dist, "num_data_shards", 1)
            self._shard_id = getattr(dist, "data_shard_id", 0)

    def get_numpy_iterator(self):
        for i, batch in enumerate(self._dataloader):
            if self._num_shards > 1 and i % self._num_shards != self._shard_id:
                continue
            yield tuple(batch) if isinstance(batch, list) else batch

    @property
    def num_batches(self):
        if self._num_batches is not None and self._num_shards > 1:
            return len(range(self._shard_id, self._num_batches, self._num_shards))
        return self._num_batches

    batch_size = property(lambda self: self._batch_size)
    has_partial_batch = property(lambda self: None if self._partial_batch_size is None else self._partial_batch_size > 0)
    partial_batch_size = property(lambda self: self._partial_batch_size)

    @property
    def builtin_prefetch(self):
        prefetch_factor = self._dataloader.prefetch_factor
        return prefetch_factor is not None and prefetch_factor > 0


def get_data_adapter(x, y=None, sample_weight=None, batch_size=None, steps_per_epoch=None, shuffle=False, class_weight=None):
    if isinstance(x, DataAdapter):
        return x
    if can_convert_arrays((x, y, sample_weight)) and not isinstance(x, (PyDataset, torch.utils.data.DataLoader)) and not _is_generator(x):
        return ArrayDataAdapter(x, y, sample_weight=sample_weight, class_weight=class_weight, shuffle=shuffle, batch_size=batch_size, steps=steps_per_epoch)
    if isinstance(x, PyDataset):
        if y is not None:
            raise ValueError("When providing `x` as a PyDataset, `y` should not be passed. Instead, the targets should be included as part of the PyDataset.")
        if sample_weight is not None:
            raise ValueError("When providing `x` as a PyDataset, `sample_weight` should not be passed. Instead, the sample weights should be included as part of the PyDataset.")
        return PyDatasetAdapter(x, class_weight=class_weight, shuffle=shuffle)
    if isinstance(x, torch.utils.data.DataLoader):
        if y is not None:
            raise ValueError("When providing `x` as a torch DataLoader, `y` should not be passed. Instead, the targets should be included as part of the torch DataLoader.")
        if sample_weight is not None:
            raise ValueError("When providing `x` as a torch DataLoader, `sample_weights` should not be passed. Instead, the sample weights should be included as part of the torch DataLoader.")
        if class_weight is not None:
            raise ValueError("Argument `class_weight` is not supported for torch DataLoader inputs. You can modify your `__getitem__ ` method to return input tensor, label and class_weight. ")
        return TorchDataLoaderAdapter(x)
    if hasattr(x, "__iter__") and not hasattr(x, "__next__") and not _is_generator(x) and not isinstance(x, (list, tuple, dict, str, bytes)):
        if y is not None or sample_weight is not None:
            raise ValueError("When providing `x` as a dataset, `y` and `sample_weight` should not be passed. Instead, they should be included as part of the dataset.")
        return IterableDatasetAdapter(x, class_weight=class_weight)
    if _is_generator(x) or hasattr(x, "__next__"):
        if y is not None:
            raise ValueError("When providing `x` as a generator, `y` should not be passed. Instead, the targets should be included as part of the generator.")
        if sample_weight is not None:
            raise ValueError("When providing `x` as a generator, `sample_weight` should not be passed. Instead, the sample weights should be included as part of the generator.")
        if class_weight is not None:
            raise ValueError("Argument `class_weight` is not supported for Python generator inputs. Received: class_weight={class_weight}")
        return GeneratorDataAdapter(x)
    raise ValueError(f"Unrecognized data type: x={x} (of type {type(x)})")


def _is_generator(x):
    import inspect

    return inspect.isgenerator(x)
