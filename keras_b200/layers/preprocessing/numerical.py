"""Numeric / categorical preprocessing layers: ``Normalization``, ``Rescaling``, ``CategoryEncoding``,
``Discretization``, ``Hashing``, ``HashedCrossing``, ``Pipeline``, ``MelSpectrogram``, ``STFTSpectrogram``
(keras/src/layers/preprocessing/{normalization,rescaling,category_encoding,discretization,hashing,
hashed_crossing,pipeline,mel_spectrogram,stft_spectrogram}.py)."""

import hashlib
import itertools
import math

import numpy as np
import torch

from keras_b200 import ops, tree
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.core.tensor import convert_to_numpy, convert_to_tensor, is_tensor
from keras_b200.layers.layer import Layer
from keras_b200.layers.preprocessing.data_layer import DataLayer
from keras_b200.saving import serialization_lib


def _extract_batch(batch):
    if isinstance(batch, (tuple, list)):
        return batch[0]
    return batch


def _iter_batches(data):
    """Yield array batches from arrays, tensors, DataLoaders, PyDatasets or generic iterables."""
    from keras_b200.trainers.data_adapters import adapters

    py_dataset = getattr(adapters, "PyDataset", None)
    if isinstance(data, np.ndarray) or is_tensor(data):
        yield data
    elif py_dataset is not None and isinstance(data, py_dataset):
        for i in range(len(data)):
            yield _extract_batch(data[i])
    elif hasattr(data, "__iter__"):
        for b in data:
            yield _extract_batch(b)
    else:
        raise TypeError(f"Unsupported data type: {type(data)}. `adapt` supports `np.ndarray`, backend tensors, `keras.utils.PyDataset`, and iterables of batches (e.g. list, generator).")


@keras_export("keras.layers.Normalization")
class Normalization(DataLayer):
    def __init__(self, axis=-1, mean=None, variance=None, invert=False, **kwargs):
        super().__init__(**kwargs)
        if axis is None:
            axis = ()
        elif isinstance(axis, int):
            axis = (axis,)
        else:
            axis = tuple(axis)
        self.axis = axis
        self.input_mean, self.input_variance, self.invert = mean, variance, invert
        self.supports_masking = True
        self._build_input_shape = None
        self.mean = None
        if (mean is not None) != (variance is not None):
            raise ValueError(f"When setting values directly, both `mean` and `variance` must be set. Received: mean={mean} and variance={variance}")
        if mean is not None:
            if np.shape(mean) != np.shape(variance):
                raise ValueError(f"When setting values directly, `mean` and `variance` must have the same shape. Received: mean shape {np.shape(mean)} and variance shape {np.shape(variance)}")
            if len(np.shape(mean)) > len(self.axis):
                raise ValueError(f"The rank of `mean` must be less than or equal to the number of axes ({len(self.axis)}). Received: mean shape {np.shape(mean)} for axis {self.axis}")

    def build(self, input_shape):
        if input_shape is None:
            return
        ndim = len(input_shape)
        self._build_input_shape = input_shape
        if any(a < -ndim or a >= ndim for a in self.axis):
            raise ValueError(f"All `axis` values must be in the range [-ndim, ndim). Received inputs with ndim={ndim}, while axis={self.axis}")
        self._keep_axis = tuple(sorted(d if d >= 0 else d + ndim for d in self.axis))
        for d in self._keep_axis:
            if input_shape[d] is None:
                raise ValueError(f"All `axis` values to be kept must have a known shape. Received axis={self.axis}, inputs.shape={input_shape}, with unknown axis at index {d}")
        self._reduce_axis = tuple(d for d in range(ndim) if d not in self._keep_axis)
        self._broadcast_shape = [input_shape[d] if d in self._keep_axis else 1 for d in range(ndim)]
        self._mean_and_var_shape = tuple(input_shape[d] for d in self._keep_axis)
        if self.input_mean is None:
            self.adapt_mean = self.add_weight(name="mean", shape=self._mean_and_var_shape, initializer="zeros", trainable=False)
            self.adapt_variance = self.add_weight(name="variance", shape=self._mean_and_var_shape, initializer="ones", trainable=False)
            self.count = self.add_weight(name="count", shape=(), dtype="int", initializer="zeros", trainable=False)
            self.built = True
            self.finalize_state()
        else:
            mean = convert_to_tensor(self.input_mean)
            variance = convert_to_tensor(self.input_variance)
            if mean.ndim == 0:
                mean = ops.broadcast_to(mean, self._broadcast_shape)
                variance = ops.broadcast_to(variance, self._broadcast_shape)
            else:
                expanded = [1] * ndim
                for i in range(1, mean.ndim + 1):
                    expanded[self._keep_axis[-i]] = mean.shape[-i]
                mean = ops.broadcast_to(ops.reshape(mean, expanded), self._broadcast_shape)
                variance = ops.broadcast_to(ops.reshape(variance, expanded), self._broadcast_shape)
            self.mean = ops.cast(mean, dtype=self.compute_dtype)
            self.variance = ops.cast(variance, dtype=self.compute_dtype)
            self.built = True

    def adapt(self, data):
        """Compute mean and variance over ``data`` (array, tensor or iterable of batches) with Chan's parallel update."""
        batches = _iter_batches(data)
        first = next(batches, None)
        if first is None:
            raise ValueError("adapt() received an empty iterable (no batches). Expected at least one batch.")
        input_shape = tuple(first.shape)
        if not self.built:
            self.build(input_shape)
        else:
            for d in self._keep_axis:
                if input_shape[d] != self._build_input_shape[d]:
                    raise ValueError(f"The layer was built with input_shape={self._build_input_shape}, but adapt() is being called with data with an incompatible shape, data.shape={input_shape}")
        total_mean = total_var = None
        total_count = 0
        for batch in itertools.chain([first], batches):
            b = convert_to_tensor(batch).to(torch.float64)
            n = 1
            for d in self._reduce_axis:
                n *= b.shape[d]
            bm = b.mean(dim=self._reduce_axis) if self._reduce_axis else b
            bv = b.var(dim=self._reduce_axis, unbiased=False) if self._reduce_axis else torch.zeros_like(b)
            if total_mean is None:
                total_mean, total_var, total_count = bm, bv, n
            else:
                new_count = total_count + n
                wb, wt = n / new_count, total_count / new_count
                new_mean = total_mean * wt + bm * wb
                total_var = (total_var + (total_mean - new_mean) ** 2) * wt + (bv + (bm - new_mean) ** 2) * wb
                total_mean, total_count = new_mean, new_count
        self.adapt_mean.assign(total_mean.to(torch.float32).reshape(self._mean_and_var_shape))
        self.adapt_variance.assign(total_var.to(torch.float32).reshape(self._mean_and_var_shape))
        self.finalize_state()

    def finalize_state(self):
        if self.input_mean is not None or not self.built:
            return
        self.mean = ops.cast(ops.reshape(self.adapt_mean, self._broadcast_shape), self.compute_dtype)
        self.variance = ops.cast(ops.reshape(self.adapt_variance, self._broadcast_shape), self.compute_dtype)

    def call(self, inputs):
        if self.mean is None:
            raise ValueError("You must call `.build(input_shape)` on the layer before using it.")
        inputs = ops.cast(convert_to_tensor(inputs), self.compute_dtype)
        mean, variance = self.mean, self.variance
        if isinstance(mean, torch.Tensor) and isinstance(inputs, torch.Tensor) and mean.device != inputs.device:
            mean, variance = mean.to(inputs.device), variance.to(inputs.device)
        eps = ops.cast(1e-7, self.compute_dtype) if False else 1e-7
        if self.invert:
            return ops.add(mean, ops.multiply(inputs, ops.maximum(ops.sqrt(variance), eps)))
        return ops.divide(ops.subtract(inputs, mean), ops.maximum(ops.sqrt(variance), eps))

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"axis": self.axis, "invert": self.invert,
                    "mean": np.array(self.input_mean).tolist() if self.input_mean is not None else None,
                    "variance": np.array(self.input_variance).tolist() if self.input_variance is not None else None})
        return cfg

    def load_own_variables(self, store):
        super().load_own_variables(store)
        self.finalize_state()

    def get_build_config(self):
        if self._build_input_shape:
            return {"input_shape": self._build_input_shape}

    def build_from_config(self, config):
        if config:
            self.build(config["input_shape"])


@keras_export("keras.layers.Rescaling")
class Rescaling(DataLayer):
    def __init__(self, scale, offset=0.0, **kwargs):
        super().__init__(**kwargs)
        self.scale, self.offset = scale, offset
        self.supports_masking = True

    def call(self, inputs):
        dtype = self.compute_dtype
        scale = ops.cast(self.scale, dtype)
        offset = ops.cast(self.offset, dtype)
        x = ops.cast(convert_to_tensor(inputs), dtype)
        if isinstance(scale, torch.Tensor) and scale.ndim > 0 and isinstance(x, torch.Tensor) and x.ndim == 4 and scale.numel() == x.shape[1] and scale.numel() != x.shape[-1]:
            scale = scale.reshape(1, -1, 1, 1)  # per-channel scale on channels_first images
            offset = offset.reshape(1, -1, 1, 1) if isinstance(offset, torch.Tensor) and offset.ndim > 0 else offset
        return ops.add(ops.multiply(x, scale), offset)

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        def ser(v):
            if isinstance(v, (np.ndarray, torch.Tensor)):
                return convert_to_numpy(v).tolist()
            return v

        return {**super().get_config(), "scale": ser(self.scale), "offset": ser(self.offset)}


def encode_categorical_inputs(inputs, output_mode, depth, dtype, sparse=False, count_weights=None):
    """int / one_hot / multi_hot / count encoding of integer inputs (keras/src/utils/numerical_utils.py:106-196)."""
    if output_mode == "int":
        return ops.cast(inputs, dtype)
    x = convert_to_tensor(inputs).to(torch.int64)
    rank_1 = x.ndim == 0
    if rank_1:
        x = x.reshape(1)
    if output_mode == "one_hot":
        if x.ndim > 0 and x.shape[-1] == 1 and x.ndim > 1:
            x = x.squeeze(-1)
        valid = (x >= 0) & (x < depth)
        out = torch.nn.functional.one_hot(x.clamp(0, depth - 1), depth).to(dtype) * valid.unsqueeze(-1).to(dtype)
        return out
    if x.ndim > 2:
        raise ValueError(f"When output_mode is anything other than `'int'`, maximum supported output rank is 2. Received output_mode {output_mode} and input shape {tuple(x.shape)}, which would result in output rank {x.ndim}.")
    binary = output_mode == "multi_hot"
    flat = x.reshape(-1, x.shape[-1]) if x.ndim == 2 else x.reshape(1, -1)
    valid = (flat >= 0) & (flat < depth)
    w = torch.ones_like(flat, dtype=torch.float32) if count_weights is None else convert_to_tensor(count_weights).to(torch.float32).reshape(flat.shape)
    out = torch.zeros((flat.shape[0], depth), dtype=torch.float32, device=flat.device)
    out.scatter_add_(1, flat.clamp(0, depth - 1), w * valid.to(torch.float32))
    if binary:
        out = (out > 0).to(torch.float32)
    if x.ndim == 1:
        out = out[0]
    return out.to(dtype)


@keras_export("keras.layers.CategoryEncoding")
class CategoryEncoding(DataLayer):
    def __init__(self, num_tokens=None, output_mode="multi_hot", sparse=False, **kwargs):
        super().__init__(**kwargs)
        if output_mode not in ("count", "one_hot", "multi_hot"):
            raise ValueError(f"Unknown arg for output_mode: {output_mode}")
        if num_tokens is None:
            raise ValueError("num_tokens must be set to use this layer. If the number of tokens is not known beforehand, use the IntegerLookup layer instead.")
        if num_tokens < 1:
            raise ValueError(f"`num_tokens` must be >= 1. Received: num_tokens={num_tokens}.")
        self.num_tokens, self.output_mode, self.sparse = num_tokens, output_mode, sparse
        self._allow_non_tensor_positional_args = True
        self._convert_input_args = False

    def compute_output_shape(self, input_shape):
        if (input_shape is not None) and not len(input_shape):
            return (self.num_tokens,)
        if self.output_mode == "one_hot":
            if input_shape[-1] != 1:
                return tuple(input_shape) + (self.num_tokens,)
            if len(input_shape) == 1:
                return tuple(input_shape) + (self.num_tokens,)
            return tuple(input_shape[:-1]) + (self.num_tokens,)
        return tuple(input_shape[:-1]) + (self.num_tokens,)

    def compute_output_spec(self, inputs, count_weights=None):
        return KerasTensor(self.compute_output_shape(inputs.shape), dtype=self.compute_dtype)

    def call(self, inputs, count_weights=None):
        if count_weights is not None and self.output_mode != "count":
            raise ValueError(f"`count_weights` is not used when `output_mode` is not `'count'`. Received `count_weights={count_weights}`.")
        return encode_categorical_inputs(inputs, self.output_mode, self.num_tokens, getattr(torch, self.compute_dtype), self.sparse, count_weights)

    def get_config(self):
        return {**super().get_config(), "num_tokens": self.num_tokens, "output_mode": self.output_mode}


@keras_export("keras.layers.Discretization")
class Discretization(DataLayer):
    def __init__(self, bin_boundaries=None, num_bins=None, epsilon=0.01, output_mode="int", sparse=False, dtype=None, name=None):
        if dtype is None:
            dtype = "int64" if output_mode == "int" else None
        super().__init__(name=name, dtype=dtype)
        if output_mode not in ("int", "one_hot", "multi_hot", "count"):
            raise ValueError(f"Invalid value for argument `output_mode`. Received: output_mode={output_mode}")
        if num_bins is not None and num_bins < 0:
            raise ValueError(f"`num_bins` must be greater than or equal to 0. Received: `num_bins={num_bins}`")
        if num_bins is not None and bin_boundaries is not None and len(bin_boundaries) != num_bins - 1:
            raise ValueError(f"Both `num_bins` and `bin_boundaries` should not be set. Received: `num_bins={num_bins}` and `bin_boundaries={bin_boundaries}`")
        if num_bins is None and bin_boundaries is None:
            raise ValueError("You need to set either `num_bins` or `bin_boundaries`.")
        self.input_bin_boundaries = bin_boundaries
        self.bin_boundaries = bin_boundaries if bin_boundaries is not None else None
        self.num_bins, self.epsilon, self.output_mode, self.sparse = num_bins, epsilon, output_mode, sparse
        self.summary = None if self.bin_boundaries else np.array([[], []], dtype="float32")

    def build(self, input_shape=None):
        self.built = True

    @property
    def input_dtype(self):
        return "float32"

    def adapt(self, data, steps=None):
        if self.input_bin_boundaries is not None:
            raise ValueError("Cannot adapt a Discretization layer that has been initialized with `bin_boundaries`, use `num_bins` instead.")
        self.reset_state()
        for i, batch in enumerate(_iter_batches(data)):
            if steps is not None and i >= steps:
                break
            self.update_state(batch)
        self.finalize_state()

    def update_state(self, data):
        values = np.sort(np.reshape(convert_to_numpy(convert_to_tensor(data)).astype("float32"), [-1]))
        summary = _summarize(values, self.epsilon)
        self.summary = _merge_summaries(summary, self.summary, self.epsilon)

    def finalize_state(self):
        if self.input_bin_boundaries is not None:
            return
        self.bin_boundaries = _bin_boundaries(self.summary, self.num_bins).tolist()

    def reset_state(self):
        if self.input_bin_boundaries is not None:
            return
        self.summary = np.array([[], []], dtype="float32")

    def compute_output_spec(self, inputs):
        return KerasTensor(shape=inputs.shape, dtype=self.output_dtype)

    @property
    def output_dtype(self):
        return self.compute_dtype

    def load_own_variables(self, store):
        if len(store) == 1:
            self.summary = store["0"]
        return

    def call(self, inputs):
        if self.bin_boundaries is None:
            raise ValueError("You need to either pass the `bin_boundaries` argument at construction time or call `adapt(dataset)` before you can start using the `Discretization` layer.")
        x = convert_to_tensor(inputs)
        idx = torch.bucketize(x.to(torch.float32), torch.tensor(self.bin_boundaries, dtype=torch.float32, device=x.device), right=True)
        depth = len(self.bin_boundaries) + 1
        return encode_categorical_inputs(idx, self.output_mode, depth, getattr(torch, self.compute_dtype), self.sparse)

    def get_config(self):
        return {"bin_boundaries": self.bin_boundaries, "num_bins": self.num_bins, "epsilon": self.epsilon, "output_mode": self.output_mode,
                "sparse": self.sparse, "name": self.name, "dtype": self.dtype}


def _summarize(values, epsilon):
    """Reduce sorted values to at most 1/epsilon (value, weight) buckets."""
    values = np.reshape(values, [-1])
    num_buckets = 1.0 / epsilon
    n = np.size(values)
    increment = max(int(n / num_buckets), 1)
    start = increment
    boundaries = values[start::increment]
    weights = np.ones_like(boundaries) * increment
    return np.stack([boundaries, weights])


def _merge_summaries(prev, nxt, epsilon):
    merged = np.concatenate((prev, nxt), axis=1)
    merged = np.take(merged, np.argsort(merged[0]), axis=1)
    return _compress(merged, epsilon)


def _compress(summary, epsilon):
    if summary.shape[1] * epsilon < 1:
        return summary
    percents = epsilon + np.arange(0.0, 1.0, epsilon)
    cum = summary[1].cumsum()
    cum_percents = cum / cum[-1]
    new_bins = np.interp(percents, cum_percents, summary[0])
    cum_w = np.interp(percents, cum_percents, cum)
    new_w = cum_w - np.concatenate((np.array([0]), cum_w[:-1]))
    return np.stack((new_bins, new_w)).astype("float32")


def _bin_boundaries(summary, num_bins):
    return _compress(summary, 1.0 / num_bins)[0, :-1]


def _stable_hash(value, num_bins, salt=None):
    """Deterministic 64-bit hash of a value's string form (SipHash is not available; BLAKE2b keyed by ``salt``)."""
    if isinstance(value, bytes):
        data = value
    else:
        data = str(value).encode("utf-8")
    key = b""
    if salt is not None:
        key = b"".join(int(s & 0xFFFFFFFFFFFFFFFF).to_bytes(8, "little") for s in salt)
    h = hashlib.blake2b(data, digest_size=8, key=key).digest()
    return int.from_bytes(h, "little") % num_bins


@keras_export("keras.layers.Hashing")
class Hashing(Layer):
    """Hash and bin categorical features.  Values are hashed on the host from their string form; the reference uses
    TF's FarmHash/SipHash, so bucket assignments are deterministic here but not identical to the reference's."""

    def __init__(self, num_bins, mask_value=None, salt=None, output_mode="int", sparse=False, **kwargs):
        if "dtype" not in kwargs or kwargs["dtype"] is None:
            kwargs["dtype"] = "int64" if output_mode == "int" else "float32"
        super().__init__(**kwargs)
        if num_bins is None or num_bins <= 0:
            raise ValueError(f"The `num_bins` for `Hashing` cannot be `None` or non-positive values. Received: num_bins={num_bins}.")
        if output_mode not in ("int", "one_hot", "multi_hot", "count"):
            raise ValueError(f"Invalid value for argument `output_mode`. Expected one of ('int', 'one_hot', 'multi_hot', 'count'). Received: output_mode={output_mode}")
        self.num_bins, self.mask_value, self.output_mode, self.sparse = num_bins, mask_value, output_mode, sparse
        self.strong_hash = salt is not None
        self.salt = None
        if salt is not None:
            if isinstance(salt, (tuple, list)) and len(salt) == 2:
                self.salt = list(salt)
            elif isinstance(salt, int):
                self.salt = [salt, salt]
            else:
                raise ValueError(f"The `salt` argument for `Hashing` can only be a tuple of size 2 integers, or a single integer. Received: salt={salt}.")
        self._convert_input_args = False
        self._allow_non_tensor_positional_args = True
        self.supports_jit = False

    def call(self, inputs):
        arr = convert_to_numpy(inputs) if is_tensor(inputs) else np.asarray(inputs)
        flat = arr.reshape(-1)
        bins = self.num_bins - 1 if self.mask_value is not None else self.num_bins
        out = np.empty(flat.shape, dtype="int64")
        for i, v in enumerate(flat):
            if isinstance(v, bytes):
                v = v.decode("utf-8")
            if isinstance(v, np.generic):
                v = v.item()
            if self.mask_value is not None and v == self.mask_value:
                out[i] = 0
            else:
                h = _stable_hash(v, bins, self.salt)
                out[i] = h + 1 if self.mask_value is not None else h
        idx = torch.from_numpy(out.reshape(arr.shape))
        return encode_categorical_inputs(idx, self.output_mode, self.num_bins, getattr(torch, self.compute_dtype), self.sparse)

    def compute_output_spec(self, inputs):
        if self.output_mode == "int":
            return KerasTensor(shape=inputs.shape, dtype=self.compute_dtype)
        return KerasTensor(shape=tuple(inputs.shape[:-1]) + (self.num_bins,), dtype=self.compute_dtype)

    def get_config(self):
        return {**super().get_config(), "num_bins": self.num_bins, "salt": self.salt, "mask_value": self.mask_value,
                "output_mode": self.output_mode, "sparse": self.sparse}


@keras_export("keras.layers.HashedCrossing")
class HashedCrossing(Layer):
    def __init__(self, num_bins, output_mode="int", sparse=False, name=None, dtype=None, **kwargs):
        if output_mode == "int" and dtype is None:
            dtype = "int64"
        super().__init__(name=name, dtype=dtype)
        if output_mode not in ("int", "one_hot"):
            raise ValueError(f"Invalid value for argument `output_mode`. Expected one of ('int', 'one_hot'). Received: output_mode={output_mode}")
        self.num_bins, self.output_mode, self.sparse = num_bins, output_mode, sparse
        self._allow_non_tensor_positional_args = True
        self._convert_input_args = False
        self.supports_jit = False

    def compute_output_shape(self, input_shape):
        if not len(input_shape) == 2 or not isinstance(input_shape[0], tuple) or not isinstance(input_shape[1], tuple):
            raise ValueError(f"Expected as input a list/tuple of 2 tensors. Received input_shape={input_shape}")
        if input_shape[0][-1] != input_shape[1][-1]:
            raise ValueError(f"Expected the two input tensors to have identical shapes. Received input_shape={input_shape}")
        if not input_shape:
            return () if self.output_mode == "int" else (self.num_bins,)
        if self.output_mode == "int":
            return tuple(input_shape[0])
        if self.output_mode == "one_hot" and input_shape[0][-1] != 1:
            return tuple(input_shape[0]) + (self.num_bins,)
        return tuple(input_shape[0])[:-1] + (self.num_bins,)

    def call(self, inputs):
        if not isinstance(inputs, (tuple, list)) or len(inputs) != 2:
            raise ValueError(f"`HashedCrossing` should be called on a list or tuple of inputs. Received: inputs={inputs}" if not isinstance(inputs, (tuple, list)) else f"`HashedCrossing` should be called on exactly two inputs. Received: inputs={inputs}")
        arrs = [convert_to_numpy(i) if is_tensor(i) else np.asarray(i) for i in inputs]
        if arrs[0].shape != arrs[1].shape:
            raise ValueError(f"All `HashedCrossing` inputs should have equal shape. Received: inputs={inputs}")
        rank = arrs[0].ndim
        if rank > 2 or (rank == 2 and arrs[0].shape[-1] != 1):
            raise ValueError(f"All `HashedCrossing` inputs should have shape `()`, `(batch_size)` or `(batch_size, 1)`. Received: inputs={inputs}")
        flat = [a.reshape(-1) for a in arrs]

        def s(v):
            if isinstance(v, bytes):
                return v.decode("utf-8")
            return str(v.item() if isinstance(v, np.generic) else v)

        out = np.array([_stable_hash(s(a) + "_X_" + s(b), self.num_bins) for a, b in zip(*flat)], dtype="int64").reshape(arrs[0].shape)
        idx = torch.from_numpy(np.asarray(out))
        if self.output_mode == "one_hot" and rank == 0:
            return encode_categorical_inputs(idx.reshape(1), "one_hot", self.num_bins, getattr(torch, self.compute_dtype))[0]
        return encode_categorical_inputs(idx, self.output_mode, self.num_bins, getattr(torch, self.compute_dtype), self.sparse)

    def get_config(self):
        return {"num_bins": self.num_bins, "output_mode": self.output_mode, "sparse": self.sparse, "name": self.name, "dtype": self.dtype}


@keras_export("keras.layers.Pipeline")
class Pipeline(Layer):
    """Apply a series of layers to an input, in or out of a model."""

    def __init__(self, layers, name=None):
        super().__init__(name=name)
        self._pipeline_layers = layers
        self._convert_input_args = False
        self._allow_non_tensor_positional_args = True

    @property
    def layers(self):
        return self._pipeline_layers

    def call(self, inputs, training=True, mask=None):
        for layer in self._pipeline_layers:
            kw = {}
            if layer._call_has_mask_arg:
                kw["mask"] = mask
            if layer._call_has_training_arg and training is not None:
                kw["training"] = training
            outputs = layer(inputs, **kw)
            inputs = outputs

            def _get_mask_from_keras_tensor(kt):
                return getattr(kt, "_keras_mask", None)

            mask = tree.map_structure(_get_mask_from_keras_tensor, outputs)
        return outputs

    def compute_output_shape(self, input_shape):
        for layer in self._pipeline_layers:
            input_shape = layer.compute_output_shape(input_shape)
        return input_shape

    @classmethod
    def from_config(cls, config):
        config["layers"] = [serialization_lib.deserialize_keras_object(x) for x in config["layers"]]
        return cls(**config)

    def get_config(self):
        return {"layers": serialization_lib.serialize_keras_object(self._pipeline_layers), "name": self.name}


@keras_export("keras.layers.MelSpectrogram")
class MelSpectrogram(DataLayer):
    def __init__(self, fft_length=2048, sequence_stride=512, sequence_length=None, window="hann", sampling_rate=16000, num_mel_bins=128,
                 min_freq=20.0, max_freq=None, power_to_db=True, top_db=80.0, mag_exp=2.0, min_power=1e-10, ref_power=1.0, **kwargs):
        self.fft_length, self.sequence_stride = fft_length, sequence_stride
        self.sequence_length = sequence_length or fft_length
        self.window, self.sampling_rate, self.num_mel_bins = window, sampling_rate, num_mel_bins
        self.min_freq = min_freq
        self.max_freq = max_freq or int(sampling_rate / 2)
        self.power_to_db, self.top_db, self.mag_exp, self.min_power, self.ref_power = power_to_db, top_db, mag_exp, min_power, ref_power
        super().__init__(**kwargs)

    def call(self, inputs):
        dtype = "float32" if self.compute_dtype not in ["float32", "float64"] else self.compute_dtype
        outputs = self._spectrogram(inputs)
        outputs = self._melscale(outputs)
        if self.power_to_db:
            outputs = self._dbscale(outputs)
        outputs = ops.swapaxes(outputs, -1, -2)
        return ops.cast(outputs, dtype)

    def _spectrogram(self, inputs):
        real, imag = ops.stft(inputs, sequence_length=self.sequence_length, sequence_stride=self.sequence_stride, fft_length=self.fft_length,
                              window=self.window, center=True)
        spec = ops.sqrt(ops.add(ops.square(real), ops.square(imag)))
        return ops.power(spec, self.mag_exp)

    def _melscale(self, inputs):
        matrix = self.linear_to_mel_weight_matrix(num_mel_bins=self.num_mel_bins, num_spectrogram_bins=ops.shape(inputs)[-1],
                                                  sampling_rate=self.sampling_rate, lower_edge_hertz=self.min_freq, upper_edge_hertz=self.max_freq)
        return ops.tensordot(inputs, matrix, axes=1)

    def _dbscale(self, inputs):
        log_spec = 10.0 * ops.divide(ops.log(ops.maximum(inputs, self.min_power)), math.log(10.0))
        ref_value = abs(self.ref_power)
        log_spec = log_spec - 10.0 * math.log10(max(self.min_power, ref_value))
        log_spec = ops.maximum(log_spec, ops.max(log_spec) - self.top_db)
        return log_spec

    def _hertz_to_mel(self, f):
        return 2595.0 * ops.log10(1.0 + f / 700.0)

    def linear_to_mel_weight_matrix(self, num_mel_bins=20, num_spectrogram_bins=129, sampling_rate=8000, lower_edge_hertz=125.0,
                                    upper_edge_hertz=3800.0, dtype="float32"):
        sampling_rate = ops.cast(sampling_rate, dtype)
        lower = ops.cast(lower_edge_hertz, dtype)
        upper = ops.cast(upper_edge_hertz, dtype)
        bands_to_zero = 1
        nyquist = sampling_rate / 2.0
        linear = ops.linspace(0.0, nyquist, num_spectrogram_bins, dtype=dtype)[bands_to_zero:]
        spec_mel = ops.expand_dims(self._hertz_to_mel(linear), axis=1)
        edges = ops.linspace(self._hertz_to_mel(lower), self._hertz_to_mel(upper), num_mel_bins + 2, dtype=dtype)
        lower_e = ops.reshape(edges[:-2], (1, num_mel_bins))
        center = ops.reshape(edges[1:-1], (1, num_mel_bins))
        upper_e = ops.reshape(edges[2:], (1, num_mel_bins))
        lower_slopes = (spec_mel - lower_e) / (center - lower_e)
        upper_slopes = (upper_e - spec_mel) / (upper_e - center)
        mel = ops.maximum(0.0, ops.minimum(lower_slopes, upper_slopes))
        return ops.pad(mel, [[bands_to_zero, 0], [0, 0]])

    def compute_output_shape(self, input_shape):
        if len(input_shape) == 1:
            out = [self.num_mel_bins, (input_shape[0] + self.sequence_stride + 1) // self.sequence_stride if input_shape[0] is not None else None]
        else:
            out = [input_shape[0], self.num_mel_bins, (input_shape[1] + self.sequence_stride + 1) // self.sequence_stride if input_shape[1] is not None else None]
        return tuple(out)

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"fft_length": self.fft_length, "sequence_stride": self.sequence_stride, "sequence_length": self.sequence_length,
                    "window": self.window, "sampling_rate": self.sampling_rate, "num_mel_bins": self.num_mel_bins, "min_freq": self.min_freq,
                    "max_freq": self.max_freq, "power_to_db": self.power_to_db, "top_db": self.top_db, "mag_exp": self.mag_exp,
                    "min_power": self.min_power, "ref_power": self.ref_power})
        return cfg


@keras_export("keras.layers.STFTSpectrogram")
class STFTSpectrogram(Layer):
    """Spectrogram as a trainable 1-D convolution whose kernel is initialised to the STFT basis
    (keras/src/layers/preprocessing/stft_spectrogram.py)."""

    def __init__(self, mode="log", frame_length=256, frame_step=None, fft_length=None, window="hann", periodic=False, scaling="density",
                 padding="valid", expand_dims=False, data_format=None, **kwargs):
        from keras_b200.core import config as _config

        if frame_step is not None and (frame_step > frame_length or frame_step < 1):
            raise ValueError(f"`frame_step` should be a positive integer not greater than `frame_length`. Received frame_step={frame_step}, frame_length={frame_length}")
        if fft_length is not None and fft_length < frame_length:
            raise ValueError(f"`fft_length` should be not less than `frame_length`. Received fft_length={fft_length}, frame_length={frame_length}")
        if fft_length is not None and (fft_length & -fft_length) != fft_length:
            import warnings

            warnings.warn(f"`fft_length` is recommended to be a power of two. Received fft_length={fft_length}")
        all_modes = ["log", "magnitude", "psd", "real", "imag", "angle", "stft"]
        if mode not in all_modes:
            raise ValueError(f"Output mode is invalid, it must be one of {', '.join(all_modes)}. Received: mode={mode}")
        if scaling is not None and scaling not in ["density", "spectrum"]:
            raise ValueError(f"Scaling is invalid, it must be `None`, 'density' or 'spectrum'. Received scaling={scaling}")
        if padding not in ["valid", "same"]:
            raise ValueError(f"Padding is invalid, it should be 'valid', 'same'. Received: padding={padding}")
        if isinstance(window, str):
            from scipy import signal as _sig  # validates the window name

            _sig.get_window(window, 1)
        super().__init__(**kwargs)
        self.mode, self.frame_length = mode, frame_length
        self.frame_step = frame_step if frame_step is not None else self.frame_length // 2
        self._frame_step = frame_step
        self.fft_length = fft_length if fft_length is not None else frame_length
        self._fft_length = fft_length
        self.window, self.periodic, self.scaling, self.padding = window, periodic, scaling, padding
        self.expand_dims = expand_dims
        self.data_format = _config.standardize_data_format(data_format)
        self.input_spec = None

    def build(self, input_shape):
        from keras_b200 import initializers

        shape = (self.frame_length, 1, self.fft_length // 2 + 1)
        if self.mode != "imag":
            self.real_kernel = self.add_weight(name="real_kernel", shape=shape,
                                               initializer=initializers.STFT("real", self.window, self.scaling, self.periodic))
        if self.mode != "real":
            self.imag_kernel = self.add_weight(name="imag_kernel", shape=shape,
                                               initializer=initializers.STFT("imag", self.window, self.scaling, self.periodic))

    def _adjust_shapes(self, outputs):
        _, channels, freq_channels, time_seq = ops.shape(outputs)
        batch_size = -1
        if self.data_format == "channels_last":
            if self.expand_dims:
                outputs = ops.transpose(outputs, [0, 3, 2, 1])
            else:
                outputs = ops.reshape(outputs, [batch_size, channels * freq_channels, time_seq])
                outputs = ops.transpose(outputs, [0, 2, 1])
        else:
            if self.expand_dims:
                outputs = ops.transpose(outputs, [0, 1, 3, 2])
            else:
                outputs = ops.reshape(outputs, [batch_size, channels * freq_channels, time_seq])
        return outputs

    def _apply_conv(self, inputs, kernel):
        if self.data_format == "channels_last":
            _, time_seq, channels = ops.shape(inputs)
            inputs = ops.transpose(inputs, [0, 2, 1])
            inputs = ops.reshape(inputs, [-1, time_seq, 1])
        else:
            _, channels, time_seq = ops.shape(inputs)
            inputs = ops.reshape(inputs, [-1, 1, time_seq])
        outputs = ops.conv(inputs, ops.cast(kernel, inputs.dtype), padding=self.padding, strides=self.frame_step, data_format=self.data_format)
        batch_size = -1
        if self.data_format == "channels_last":
            _, time_seq, freq_channels = ops.shape(outputs)
            outputs = ops.transpose(outputs, [0, 2, 1])
            outputs = ops.reshape(outputs, [batch_size, channels, freq_channels, time_seq])
        else:
            _, freq_channels, time_seq = ops.shape(outputs)
            outputs = ops.reshape(outputs, [batch_size, channels, freq_channels, time_seq])
        return outputs

    def call(self, inputs):
        real = imag = power = None
        if self.mode != "imag":
            real = self._apply_conv(inputs, self.real_kernel)
        if self.mode != "real":
            imag = self._apply_conv(inputs, self.imag_kernel)
        if self.mode == "real":
            return self._adjust_shapes(real)
        if self.mode == "imag":
            return self._adjust_shapes(imag)
        if self.mode == "angle":
            return self._adjust_shapes(ops.arctan2(imag, real))
        if self.mode == "stft":
            return self._adjust_shapes(ops.concatenate([real, imag], axis=2))
        power = ops.square(real) + ops.square(imag)
        if self.mode == "psd":
            return self._adjust_shapes(power + ops.pad(power[:, :, 1:-1, :], [[0, 0], [0, 0], [1, 1], [0, 0]]))
        linear = ops.sqrt(ops.maximum(power, 1e-12))
        if self.mode == "magnitude":
            return self._adjust_shapes(linear)
        return self._adjust_shapes(ops.log(ops.maximum(linear, 1e-12)))

    def compute_output_shape(self, input_shape):
        if self.data_format == "channels_last":
            channels = input_shape[-1]
        else:
            channels = input_shape[1]
        freq = self.fft_length // 2 + 1
        if self.mode == "stft":
            freq *= 2
        from keras_b200.ops.operation_utils import compute_conv_output_shape

        shape = compute_conv_output_shape(input_shape, freq * channels, (self.frame_length,), strides=self.frame_step, padding=self.padding,
                                          data_format=self.data_format)
        if self.data_format == "channels_last":
            batch, time_seq, _ = shape
        else:
            batch, _, time_seq = shape
        if self.expand_dims:
            if self.data_format == "channels_last":
                return (batch, time_seq, freq, channels)
            return (batch, channels, time_seq, freq)
        return shape

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"mode": self.mode, "frame_length": self.frame_length, "frame_step": self._frame_step, "fft_length": self._fft_length,
                    "window": self.window, "periodic": self.periodic, "scaling": self.scaling, "padding": self.padding,
                    "data_format": self.data_format, "expand_dims": self.expand_dims})
        return cfg
