"""Vocabulary layers: ``IndexLookup``, ``IntegerLookup``, ``StringLookup``, ``TextVectorization``
(keras/src/layers/preprocessing/{index_lookup,integer_lookup,string_lookup,text_vectorization}.py).

The reference runs these through TensorFlow lookup tables even on the torch backend.  Here the vocabulary is a
host-side dict; string inputs are Python/NumPy strings (torch has no string tensors), integer outputs are
``int64`` tensors that move to the device with the rest of the batch.
"""

import collections
import os
import re
import string as _string

import numpy as np
import torch

from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.core.tensor import convert_to_numpy, is_tensor
from keras_b200.layers.layer import Layer
from keras_b200.layers.preprocessing.numerical import _iter_batches, _stable_hash, encode_categorical_inputs
from keras_b200.saving import serialization_lib


def _to_object_array(x):
    """Inputs → NumPy array (object dtype for strings, int64 for integers)."""
    if is_tensor(x):
        return convert_to_numpy(x)
    if isinstance(x, np.ndarray):
        arr = x
    elif isinstance(x, (str, bytes, int, np.integer)):
        arr = np.array(x)
    else:
        try:
            arr = np.array(x)
        except ValueError:
            arr = np.array(x, dtype=object)
    if arr.dtype.kind == "S":
        arr = np.char.decode(arr, "utf-8")
    if arr.dtype.kind == "O":
        flat = [v.decode("utf-8") if isinstance(v, bytes) else v for v in arr.reshape(-1)]
        arr = np.array(flat, dtype=object).reshape(arr.shape)
    return arr


class IndexLookup(Layer):
    def __init__(self, max_tokens, num_oov_indices, mask_token, oov_token, vocabulary_dtype, vocabulary=None, idf_weights=None, invert=False,
                 output_mode="int", sparse=False, pad_to_max_tokens=False, oov_method="floormod", name=None, salt=None, **kwargs):
        if max_tokens is not None and max_tokens <= 1:
            raise ValueError(f"If set, `max_tokens` must be greater than 1. Received: max_tokens={max_tokens}")
        if pad_to_max_tokens and max_tokens is None:
            raise ValueError(f"If pad_to_max_tokens is True, must set `max_tokens`. Received: max_tokens={max_tokens}")
        if num_oov_indices < 0:
            raise ValueError(f"`num_oov_indices` must be greater than or equal to 0. Received: num_oov_indices={num_oov_indices}")
        if output_mode == "binary":
            output_mode = "multi_hot"
        if output_mode == "tf-idf":
            output_mode = "tf_idf"
        if output_mode not in ("int", "one_hot", "multi_hot", "count", "tf_idf"):
            raise ValueError(f"Invalid value for argument `output_mode`. Received: output_mode={output_mode}")
        if invert and output_mode != "int":
            raise ValueError(f"`output_mode` must be `'int'` when `invert` is true. Received: output_mode={output_mode}")
        if sparse and output_mode == "int":
            raise ValueError(f"`sparse` may only be true if `output_mode` is `'one_hot'`, `'multi_hot'`, `'count'` or `'tf_idf'`. Received: sparse={sparse} and output_mode={output_mode}")
        if idf_weights is not None and output_mode != "tf_idf":
            raise ValueError(f"`idf_weights` should only be set if `output_mode` is `'tf_idf'`. Received: idf_weights={idf_weights} and output_mode={output_mode}")
        super().__init__(name=name)
        self._convert_input_args = False
        self._allow_non_tensor_positional_args = True
        self.supports_jit = False
        self.invert, self.max_tokens, self.num_oov_indices = invert, max_tokens, num_oov_indices
        self.mask_token, self.oov_token = mask_token, oov_token
        self.output_mode, self.sparse, self.pad_to_max_tokens = output_mode, sparse, pad_to_max_tokens
        self.vocabulary_dtype = vocabulary_dtype
        self.oov_method, self.salt = oov_method, salt
        self._frozen_vocab_size = kwargs.pop("vocabulary_size", None)
        self.input_vocabulary = vocabulary
        self.input_idf_weights = idf_weights
        self._has_input_vocabulary = vocabulary is not None
        self._tokens = []
        self._index = {}
        self.idf_weights_const = None
        self.reset_state()
        if vocabulary is not None:
            self.set_vocabulary(vocabulary, idf_weights)

    # -- vocabulary ----------------------------------------------------------------------
    def _oov_start_index(self):
        return 1 if self.mask_token is not None and self.output_mode == "int" else 0

    def _token_start_index(self):
        return self._oov_start_index() + self.num_oov_indices

    def get_vocabulary(self, include_special_tokens=True):
        if not self._tokens and not self._index:
            if not include_special_tokens:
                return []
        vocab = list(self._tokens)
        if self.mask_token is not None and self.output_mode == "int":
            lead = [self.mask_token]
        else:
            lead = []
        lead += [self.oov_token] * self.num_oov_indices
        if include_special_tokens:
            return lead + vocab
        return vocab

    def vocabulary_size(self):
        return self._token_start_index() + len(self._tokens)

    def _record_vocabulary_size(self):
        self._frozen_vocab_size = self.vocabulary_size()

    def set_vocabulary(self, vocabulary, idf_weights=None):
        if self.output_mode == "tf_idf":
            if idf_weights is None:
                raise ValueError("`idf_weights` must be set if output_mode is 'tf_idf'.")
        elif idf_weights is not None:
            raise ValueError(f"`idf_weights` should only be set if output_mode is `'tf_idf'`. Received: output_mode={self.output_mode} and idf_weights={idf_weights}")
        if isinstance(vocabulary, str):
            if serialization_lib.in_safe_mode():
                raise ValueError("Requested the loading of a vocabulary file outside of the model archive. This carries a potential risk of loading "
                                 "arbitrary and sensitive files and thus it is disallowed by default. If you trust the source of the artifact, you "
                                 "can override this error by passing `safe_mode=False` to the loading function, or calling "
                                 f"`keras.config.enable_unsafe_deserialization(). Vocabulary file: '{vocabulary}'")
            if not os.path.exists(vocabulary):
                raise ValueError(f"Vocabulary file {vocabulary} does not exist.")
            if self.output_mode == "tf_idf":
                raise ValueError("output_mode `'tf_idf'` does not support loading a vocabulary from file.")
            with open(vocabulary, "r", encoding="utf-8") as f:
                lines = f.read().splitlines()
            while lines and lines[-1] == "":
                lines.pop()
            vocabulary = [self._parse_token(t) for t in lines]
        if is_tensor(vocabulary):
            vocabulary = convert_to_numpy(vocabulary)
        vocabulary = list(_to_object_array(vocabulary).reshape(-1).tolist()) if not isinstance(vocabulary, list) else [
            v.decode("utf-8") if isinstance(v, bytes) else v for v in vocabulary]
        if is_tensor(idf_weights):
            idf_weights = convert_to_numpy(idf_weights)
        if len(vocabulary) == 0:
            raise ValueError(f"Cannot set an empty vocabulary. Received: vocabulary={vocabulary}")
        oov_start, token_start = self._oov_start_index(), self._token_start_index()
        special = [self.mask_token] * oov_start + [self.oov_token] * self.num_oov_indices
        found_special = list(vocabulary[:token_start]) == special
        tokens = vocabulary[token_start:] if found_special else vocabulary
        counts = collections.Counter(tokens)
        repeated = [t for t, c in counts.items() if c > 1]
        if repeated:
            raise ValueError(f"The passed vocabulary has at least one repeated term. Please uniquify your dataset. The repeated terms are: {repeated}")
        if self.mask_token is not None and self.mask_token in tokens:
            raise ValueError("Found reserved mask token at unexpected location in `vocabulary`. Note that passed `vocabulary` does not need to "
                             "include the OOV and mask tokens. Either remove all mask and OOV tokens, or include them only at the start of the "
                             f"vocabulary in precisely this order: {special}. Received: mask_token={self.mask_token} at vocabulary index {vocabulary.index(self.mask_token)}")
        if self.oov_token is not None and self.invert and self.oov_token in tokens:
            raise ValueError("Found reserved OOV token at unexpected location in `vocabulary`. Note that passed `vocabulary` does not need to "
                             "include the OOV and mask tokens. Either remove all mask and OOV tokens, or include them only at the start of the "
                             f"vocabulary in precisely this order: {special}. Received: oov_token={self.oov_token} at vocabulary index {vocabulary.index(self.oov_token)}")
        new_size = token_start + len(tokens)
        if self.max_tokens is not None and new_size > self.max_tokens:
            raise ValueError(f"Attempted to set a vocabulary larger than the maximum vocab size. Received vocabulary size is {new_size}; `max_tokens` is {self.max_tokens}.")
        self._set_tokens(tokens)
        self._record_vocabulary_size()
        if self.output_mode == "tf_idf" and idf_weights is not None:
            if len(vocabulary) != len(idf_weights):
                raise ValueError(f"`idf_weights` must be the same length as vocabulary. len(idf_weights) is {len(idf_weights)}; len(vocabulary) is {len(vocabulary)}")
            idf = np.asarray(idf_weights, dtype="float32")
            if idf.ndim != 1:
                raise ValueError(f"TF-IDF data must be a 1-index array. Received: type(idf_weights)={type(idf_weights)}")
            front, front_value = (0, 0) if found_special else (token_start, np.average(idf))
            back = self.max_tokens - front - len(idf) if self.pad_to_max_tokens and self.max_tokens is not None else 0
            self.idf_weights_const = np.pad(idf, (front, back), mode="constant", constant_values=(front_value, 0)).astype("float32")

    def _set_tokens(self, tokens):
        self._tokens = list(tokens)
        start = self._token_start_index()
        self._index = {t: i + start for i, t in enumerate(self._tokens)}

    def _parse_token(self, t):
        return t

    # -- adapt ---------------------------------------------------------------------------
    def adapt(self, data, steps=None):
        self.reset_state()
        if isinstance(data, (list, tuple)) and data and isinstance(data[0], (str, bytes, int, np.integer)):
            data = [np.array(data)]
        elif isinstance(data, (list, tuple)) and data and isinstance(data[0], (list, tuple)) and self.output_mode != "tf_idf" and False:
            data = [data]
        for i, batch in enumerate(_iter_batches_any(data)):
            if steps is not None and i >= steps:
                break
            self.update_state(batch)
        self.finalize_state()

    def update_state(self, data):
        if self._has_input_vocabulary:
            raise ValueError(f"Cannot adapt layer '{self.name}' after setting a static vocabulary via `vocabulary` argument or `set_vocabulary()` method.")
        docs = _as_documents(data)
        for doc in docs:
            self.token_counts.update(doc)
            if self.output_mode == "tf_idf":
                self.token_document_counts.update(set(doc))
        if self.output_mode == "tf_idf":
            self.num_documents += len(docs)

    def finalize_state(self):
        if self._has_input_vocabulary or not self.token_counts:
            self._record_vocabulary_size()
            return
        for special in (self.mask_token, self.oov_token):
            if special is not None:
                self.token_counts.pop(special, None)
        tokens = list(self.token_counts.keys())
        counts = np.array([self.token_counts[t] for t in tokens])
        keys = np.array(tokens, dtype=object) if tokens and isinstance(tokens[0], str) else np.array(tokens)
        order = np.lexsort((keys, counts))[::-1]
        token_start = self._token_start_index()
        if self.max_tokens:
            order = order[: self.max_tokens - token_start]
        tokens = [tokens[i] for i in order]
        self._set_tokens(tokens)
        if self.output_mode == "tf_idf":
            doc_counts = np.array([self.token_document_counts[t] for t in tokens], dtype="float64")
            idf = np.log(1 + self.num_documents / (1 + doc_counts)).astype("float32")
            idf = np.pad(idf, (token_start, 0), constant_values=float(idf.mean()) if len(idf) else 0.0)
            if self.pad_to_max_tokens and self.max_tokens is not None:
                idf = np.pad(idf, (0, self.max_tokens - idf.size), constant_values=0)
            self.idf_weights_const = idf.astype("float32")
        self.reset_state()
        self._record_vocabulary_size()

    def reset_state(self):
        if getattr(self, "_has_input_vocabulary", False):
            return
        self.token_counts = collections.Counter()
        self.token_document_counts = collections.Counter()
        self.num_documents = 0

    # -- call ----------------------------------------------------------------------------
    def _oov_index(self, token):
        if self.num_oov_indices == 0:
            return -1
        start = self._oov_start_index()
        if self.num_oov_indices == 1:
            return start
        if isinstance(token, (int, np.integer)) and self.oov_method == "floormod":
            return start + int(token) % self.num_oov_indices
        return start + _stable_hash(token, self.num_oov_indices, None if self.salt is None else ([self.salt, self.salt] if isinstance(self.salt, int) else self.salt))

    def _lookup(self, arr):
        flat = arr.reshape(-1)
        out = np.empty(flat.shape, dtype="int64")
        index, mask_token = self._index, self.mask_token
        mask_value = 0 if self.output_mode == "int" else -1
        for i, t in enumerate(flat):
            if isinstance(t, np.generic):
                t = t.item()
            if mask_token is not None and t == mask_token:
                out[i] = mask_value
                continue
            j = index.get(t)
            if j is None:
                j = self._oov_index(t)
                if j < 0:
                    raise ValueError(f"When `num_oov_indices=0` all inputs should be in vocabulary. Found OOV value: {t!r}")
            out[i] = j
        return out.reshape(arr.shape)

    def _inverse(self, arr):
        vocab = self.get_vocabulary()
        flat = arr.reshape(-1)
        oov = self.oov_token
        out = [vocab[i] if 0 <= i < len(vocab) else oov for i in flat.tolist()]
        res = np.array(out, dtype=object if self.vocabulary_dtype == "string" else "int64").reshape(arr.shape)
        return res

    def call(self, inputs):
        arr = _to_object_array(inputs)
        if self.invert:
            res = self._inverse(arr.astype("int64"))
            return res if self.vocabulary_dtype == "string" else torch.from_numpy(res)
        if arr.ndim == 0 and self.output_mode != "int":
            arr = arr.reshape(1)
        idx = self._lookup(arr)
        t = torch.from_numpy(np.ascontiguousarray(idx)) if idx.ndim else torch.tensor(int(idx))
        if self.output_mode == "int":
            return t.to(getattr(torch, self.dtype if self.dtype.startswith("int") else "int64"))
        depth = self.max_tokens if self.pad_to_max_tokens else self._frozen_vocab_size
        if depth is None:
            depth = self.vocabulary_size()
        dtype = torch.float32 if not self.dtype.startswith("float") else getattr(torch, self.dtype)
        mode = "count" if self.output_mode == "tf_idf" else self.output_mode
        out = encode_categorical_inputs(t, mode, depth, dtype, self.sparse)
        if self.output_mode == "tf_idf":
            if self.idf_weights_const is None:
                raise ValueError("When `output_mode` is `'tf_idf'`, `idf_weights` must be set (pass them or call `adapt()`).")
            out = out * torch.from_numpy(np.asarray(self.idf_weights_const)).to(out.dtype)
        return out

    def compute_output_shape(self, input_shape):
        if self.output_mode == "int":
            return input_shape
        depth = self.max_tokens if self.pad_to_max_tokens else self._frozen_vocab_size
        if self.output_mode == "one_hot":
            return tuple(input_shape) + (depth,) if not input_shape or input_shape[-1] != 1 else tuple(input_shape[:-1]) + (depth,)
        return tuple(input_shape[:-1]) + (depth,) if input_shape else (depth,)

    def compute_output_spec(self, inputs):
        dtype = "int64" if self.output_mode == "int" else "float32"
        return KerasTensor(self.compute_output_shape(inputs.shape), dtype=dtype)

    # -- persistence ---------------------------------------------------------------------
    def get_config(self):
        cfg = {"invert": self.invert, "max_tokens": self.max_tokens, "num_oov_indices": self.num_oov_indices, "oov_token": self.oov_token,
               "mask_token": self.mask_token, "output_mode": self.output_mode, "sparse": self.sparse, "pad_to_max_tokens": self.pad_to_max_tokens,
               "vocabulary_dtype": self.vocabulary_dtype, "idf_weights": _listify(self.input_idf_weights), "vocabulary": _listify(self.input_vocabulary),
               "vocabulary_size": self._frozen_vocab_size}
        base = super().get_config()
        return {**base, **cfg}

    def save_own_variables(self, store):
        if self.output_mode == "tf_idf":
            store["idf_weights"] = np.asarray(self.idf_weights_const)

    def load_own_variables(self, store):
        if self.output_mode == "tf_idf":
            self.idf_weights_const = np.asarray(store["idf_weights"])

    def save_assets(self, dir_path):
        if self.input_vocabulary is not None:
            return
        vocab = self.get_vocabulary(include_special_tokens=True)
        with open(os.path.join(dir_path, "vocabulary.txt"), "w", encoding="utf-8") as f:
            f.write("\n".join(str(w) for w in vocab))

    def load_assets(self, dir_path):
        if self.input_vocabulary is not None:
            return
        with open(os.path.join(dir_path, "vocabulary.txt"), "r", encoding="utf-8") as f:
            lines = f.read().splitlines()
        while lines and lines[-1] == "":
            lines.pop()
        values = [str(l) for l in lines] if self.vocabulary_dtype == "string" else [int(l) for l in lines]
        if self.output_mode == "tf_idf":
            self.set_vocabulary(values, idf_weights=np.asarray(self.idf_weights_const))
        else:
            self.set_vocabulary(values)

    def get_build_config(self):
        return {}

    def build_from_config(self, config):
        self.build(None)

    def build(self, input_shape=None):
        self.built = True


def _listify(x):
    if is_tensor(x):
        x = convert_to_numpy(x)
    if isinstance(x, np.ndarray):
        x = x.tolist()
    return x


def _iter_batches_any(data):
    if isinstance(data, (str, bytes)):
        yield np.array([data])
        return
    if isinstance(data, np.ndarray) or is_tensor(data):
        yield data
        return
    yield from _iter_batches(data)


def _as_documents(data):
    """A batch → list of documents (each a list of tokens)."""
    if isinstance(data, (list, tuple)) and data and isinstance(data[0], (list, tuple, np.ndarray)):
        return [list(_to_object_array(d).reshape(-1).tolist()) for d in data]
    arr = _to_object_array(data)
    if arr.ndim == 0:
        return [[arr.item()]]
    if arr.ndim == 1:
        return [[t] for t in arr.tolist()] if False else [arr.tolist()]
    return [row.reshape(-1).tolist() for row in arr]


@keras_export("keras.layers.IntegerLookup")
class IntegerLookup(IndexLookup):
    def __init__(self, max_tokens=None, num_oov_indices=1, mask_token=None, oov_token=-1, vocabulary=None, vocabulary_dtype="int64",
                 idf_weights=None, invert=False, output_mode="int", sparse=False, pad_to_max_tokens=False, oov_method="floormod", salt=None,
                 name=None, **kwargs):
        if max_tokens is not None and max_tokens <= 1:
            raise ValueError(f"If `max_tokens` is set for `IntegerLookup`, it must be greater than 1. Received: max_tokens={max_tokens}")
        if num_oov_indices < 0:
            raise ValueError(f"The value of `num_oov_indices` argument for `IntegerLookup` must >= 0. Received: num_oov_indices={num_oov_indices}")
        if vocabulary_dtype != "int64":
            raise ValueError(f"Only `vocabulary_dtype='int64'` is supported at this time. Received: vocabulary_dtype={vocabulary_dtype}")
        kwargs.pop("dtype", None)
        super().__init__(max_tokens=max_tokens, num_oov_indices=num_oov_indices, mask_token=mask_token, oov_token=oov_token,
                         vocabulary=vocabulary, vocabulary_dtype=vocabulary_dtype, idf_weights=idf_weights, invert=invert,
                         output_mode=output_mode, sparse=sparse, pad_to_max_tokens=pad_to_max_tokens, oov_method=oov_method, salt=salt,
                         name=name, **kwargs)

    def _parse_token(self, t):
        return int(t)

    def set_vocabulary(self, vocabulary, idf_weights=None):
        if not isinstance(vocabulary, str):
            vocabulary = [int(v) for v in _to_object_array(vocabulary).reshape(-1).tolist()]
        super().set_vocabulary(vocabulary, idf_weights)

    def get_config(self):
        cfg = super().get_config()
        cfg["oov_method"], cfg["salt"] = self.oov_method, self.salt
        return cfg


@keras_export("keras.layers.StringLookup")
class StringLookup(IndexLookup):
    def __init__(self, max_tokens=None, num_oov_indices=1, mask_token=None, oov_token="[UNK]", vocabulary=None, idf_weights=None, invert=False,
                 output_mode="int", pad_to_max_tokens=False, sparse=False, encoding="utf-8", name=None, salt=None, **kwargs):
        self.encoding = encoding
        kwargs.pop("dtype", None)
        kwargs.pop("vocabulary_dtype", None)
        super().__init__(max_tokens=max_tokens, num_oov_indices=num_oov_indices, mask_token=mask_token, oov_token=oov_token,
                         vocabulary=vocabulary, vocabulary_dtype="string", idf_weights=idf_weights, invert=invert, output_mode=output_mode,
                         pad_to_max_tokens=pad_to_max_tokens, sparse=sparse, name=name, salt=salt, oov_method="farmhash", **kwargs)

    def get_config(self):
        cfg = super().get_config()
        cfg.pop("vocabulary_dtype", None)
        cfg["encoding"], cfg["salt"] = self.encoding, self.salt
        return cfg


_STRIP_PUNCT = re.compile("[" + re.escape(r'!"#$%&()*+,-./:;<=>?@[\]^_`{|}~' + "'") + "]")


@keras_export("keras.layers.TextVectorization")
class TextVectorization(Layer):
    def __init__(self, max_tokens=None, standardize="lower_and_strip_punctuation", split="whitespace", ngrams=None, output_mode="int",
                 output_sequence_length=None, pad_to_max_tokens=False, vocabulary=None, idf_weights=None, sparse=False, ragged=False,
                 encoding="utf-8", name=None, **kwargs):
        super().__init__(name=name, **kwargs)
        if not (standardize is None or callable(standardize) or standardize in ("lower_and_strip_punctuation", "lower", "strip_punctuation")):
            raise ValueError(f"`standardize` arg must be a callable or one of None, 'lower_and_strip_punctuation', 'lower', 'strip_punctuation'. Received: standardize={standardize}")
        if not (split is None or callable(split) or split in ("whitespace", "character")):
            raise ValueError(f"`split` arg must be a callable or one of None, 'whitespace', 'character'. Received: split={split}")
        if output_mode == "binary":
            output_mode = "multi_hot"
        if output_mode == "tf-idf":
            output_mode = "tf_idf"
        if output_mode not in ("int", "multi_hot", "count", "tf_idf"):
            raise ValueError(f"Invalid value for argument `output_mode`. Received: output_mode={output_mode}")
        if not (ngrams is None or isinstance(ngrams, int) or (isinstance(ngrams, tuple) and all(isinstance(i, int) for i in ngrams))):
            raise ValueError(f"`ngrams` must be None, an integer, or a tuple of integers. Received: ngrams={ngrams}")
        if output_mode == "int" and not (isinstance(output_sequence_length, int) or output_sequence_length is None):
            raise ValueError(f"`output_sequence_length` must be either None or an integer when `output_mode` is 'int'. Received: output_sequence_length={output_sequence_length}")
        if output_mode != "int" and output_sequence_length is not None:
            raise ValueError(f"`output_sequence_length` must not be set if `output_mode` is not 'int'. Received output_sequence_length={output_sequence_length}.")
        if ragged and output_mode != "int":
            raise ValueError(f"`ragged` must not be true if `output_mode` is `'int'`. Received: ragged={ragged} and output_mode={output_mode}")
        self._max_tokens, self._standardize, self._split, self._ngrams_arg = max_tokens, standardize, split, ngrams
        self._ngrams = tuple(range(1, ngrams + 1)) if isinstance(ngrams, int) else ngrams
        self._ragged, self._output_mode, self._output_sequence_length, self._encoding = ragged, output_mode, output_sequence_length, encoding
        self._has_input_vocabulary = kwargs.pop("has_input_vocabulary", vocabulary is not None) if False else (vocabulary is not None)
        vocabulary_size = kwargs.pop("vocabulary_size", None) if False else None
        self._lookup_layer = StringLookup(max_tokens=max_tokens, vocabulary=vocabulary, idf_weights=idf_weights, pad_to_max_tokens=pad_to_max_tokens,
                                          mask_token="", output_mode=output_mode, sparse=sparse, encoding=encoding)
        self._convert_input_args = False
        self._allow_non_tensor_positional_args = True
        self.supports_jit = False

    @property
    def compute_dtype(self):
        return "string"

    @property
    def variable_dtype(self):
        return "string"

    def build(self, input_shape=None):
        self.built = True

    def compute_output_shape(self, input_shape):
        if self._output_mode == "int":
            return (input_shape[0], self._output_sequence_length)
        if self._split is None:
            if len(input_shape) <= 1:
                input_shape = tuple(input_shape) + (1,)
        else:
            input_shape = tuple(input_shape) + (None,)
        return self._lookup_layer.compute_output_shape(input_shape)

    def compute_output_spec(self, inputs):
        return KerasTensor(self.compute_output_shape(inputs.shape), dtype="int64" if self._output_mode == "int" else "float32")

    def adapt(self, data, batch_size=None, steps=None):
        self.reset_state()
        if isinstance(data, (list, tuple)) and data and isinstance(data[0], (str, bytes)):
            data = [np.array(data, dtype=object)]
        for i, batch in enumerate(_iter_batches_any(data)):
            if steps is not None and i >= steps:
                break
            self.update_state(batch)
        self.finalize_state()

    def update_state(self, data):
        self._lookup_layer.update_state(self._preprocess(data))

    def finalize_state(self):
        self._lookup_layer.finalize_state()

    def reset_state(self):
        self._lookup_layer.reset_state()

    def get_vocabulary(self, include_special_tokens=True):
        return self._lookup_layer.get_vocabulary(include_special_tokens)

    def vocabulary_size(self):
        return self._lookup_layer.vocabulary_size()

    def get_config(self):
        cfg = {"max_tokens": self._lookup_layer.max_tokens, "standardize": self._standardize, "split": self._split, "ngrams": self._ngrams_arg,
               "output_mode": self._output_mode, "output_sequence_length": self._output_sequence_length,
               "pad_to_max_tokens": self._lookup_layer.pad_to_max_tokens, "sparse": self._lookup_layer.sparse, "ragged": self._ragged,
               "vocabulary": _listify(self._lookup_layer.input_vocabulary), "idf_weights": _listify(self._lookup_layer.input_idf_weights),
               "encoding": self._encoding, "vocabulary_size": self.vocabulary_size()}
        base = super().get_config()
        return {**base, **cfg}

    @classmethod
    def from_config(cls, config):
        config = dict(config)
        config.pop("vocabulary_size", None)
        if not isinstance(config.get("standardize"), str) and config.get("standardize") is not None:
            config["standardize"] = serialization_lib.deserialize_keras_object(config["standardize"])
        if not isinstance(config.get("split"), str) and config.get("split") is not None:
            config["split"] = serialization_lib.deserialize_keras_object(config["split"])
        if isinstance(config.get("ngrams"), list):
            config["ngrams"] = tuple(config["ngrams"])
        return cls(**config)

    def set_vocabulary(self, vocabulary, idf_weights=None):
        self._lookup_layer.set_vocabulary(vocabulary, idf_weights=idf_weights)

    def _standardize_one(self, s):
        if isinstance(s, bytes):
            s = s.decode(self._encoding)
        if self._standardize in ("lower", "lower_and_strip_punctuation"):
            s = s.lower()
        if self._standardize in ("strip_punctuation", "lower_and_strip_punctuation"):
            s = _STRIP_PUNCT.sub("", s)
        return s

    def _preprocess(self, inputs):
        """Strings → list of token lists (one per example)."""
        arr = _to_object_array(inputs)
        if arr.ndim > 1:
            if arr.shape[-1] != 1:
                raise ValueError(f"When using `TextVectorization` to tokenize strings, the input rank must be 1 or the last shape dimension must be 1. Received: inputs.shape={arr.shape} with rank={arr.ndim}")
            arr = arr.reshape(arr.shape[:-1]) if self._split is not None else arr
        scalar = arr.ndim == 0
        flat = [arr.item()] if scalar else arr.reshape(-1).tolist()
        if callable(self._standardize):
            out = self._standardize(np.array(flat, dtype=object))
            flat = _to_object_array(out).reshape(-1).tolist()
        elif self._standardize is not None:
            flat = [self._standardize_one(s) for s in flat]
        else:
            flat = [s.decode(self._encoding) if isinstance(s, bytes) else s for s in flat]
        if self._split == "whitespace":
            docs = [s.split() for s in flat]
        elif self._split == "character":
            docs = [list(s) for s in flat]
        elif callable(self._split):
            docs = [list(_to_object_array(self._split(s)).reshape(-1).tolist()) for s in flat]
        else:
            docs = [[s] for s in flat]
        if self._ngrams is not None:
            docs = [[" ".join(d[i:i + n]) for n in self._ngrams for i in range(len(d) - n + 1)] for d in docs]
        self._last_scalar = scalar
        return docs

    def call(self, inputs):
        docs = self._preprocess(inputs)
        look = self._lookup_layer
        if self._output_mode == "int":
            rows = [look._lookup(np.array(d, dtype=object)) if d else np.zeros((0,), "int64") for d in docs]
            if self._ragged:
                return [torch.from_numpy(r) for r in rows]
            length = self._output_sequence_length if self._output_sequence_length is not None else max((len(r) for r in rows), default=0)
            out = np.zeros((len(rows), length), dtype="int64")
            for i, r in enumerate(rows):
                n = min(len(r), length)
                out[i, :n] = r[:n]
            if self._last_scalar:
                out = out[0]
            return torch.from_numpy(out)
        depth = look.max_tokens if look.pad_to_max_tokens else look.vocabulary_size()
        out = torch.zeros((len(docs), depth), dtype=torch.float32)
        for i, d in enumerate(docs):
            if d:
                idx = torch.from_numpy(look._lookup(np.array(d, dtype=object)))
                mode = "count" if self._output_mode == "tf_idf" else self._output_mode
                out[i] = encode_categorical_inputs(idx, mode, depth, torch.float32)
        if self._output_mode == "tf_idf":
            out = out * torch.from_numpy(np.asarray(look.idf_weights_const)).to(out.dtype)
        if self._last_scalar:
            out = out[0]
        return out

    def save_own_variables(self, store):
        self._lookup_layer.save_own_variables(store)

    def load_own_variables(self, store):
        self._lookup_layer.load_own_variables(store)

    def save_assets(self, dir_path):
        self._lookup_layer.save_assets(dir_path)

    def load_assets(self, dir_path):
        self._lookup_layer.load_assets(dir_path)
