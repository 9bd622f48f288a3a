"""``InputLayer`` / ``Input`` (keras/src/layers/core/input_layer.py)."""

import warnings

from keras_b200.core import config
from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.layer import Layer
from keras_b200.ops.node import Node


@keras_export("keras.layers.InputLayer")
class InputLayer(Layer):
    def __init__(self, shape=None, batch_size=None, dtype=None, sparse=None, ragged=None, batch_shape=None, input_tensor=None, optional=False, name=None, **kwargs):
        super().__init__(name=name)
        if "input_shape" in kwargs:
            warnings.warn("Argument `input_shape` is deprecated. Use `shape` instead.")
            shape = kwargs.pop("input_shape")
        if "batch_input_shape" in kwargs:
            batch_shape = kwargs.pop("batch_input_shape")
        if input_tensor is not None:
            if not isinstance(input_tensor, KerasTensor):
                raise ValueError(f"Argument `input_tensor` must be a KerasTensor. Received invalid type: input_tensor={input_tensor} (of type {type(input_tensor)})")
            if batch_size is not None and (len(input_tensor.shape) < 1 or input_tensor.shape[0] != batch_size):
                raise ValueError("When providing the `input_tensor` argument, you cannot provide an incompatible `batch_size` argument.")
            if shape is not None and tuple(shape) != tuple(input_tensor.shape[1:]):
                raise ValueError("When providing the `input_tensor` argument, you cannot provide an incompatible `shape` argument.")
            if batch_shape is not None and tuple(batch_shape) != tuple(input_tensor.shape):
                raise ValueError("When providing the `input_tensor` argument, you cannot provide an incompatible `batch_shape` argument.")
            shape = input_tensor.shape[1:]
            batch_shape = input_tensor.shape
            dtype = input_tensor.dtype
            sparse, ragged = input_tensor.sparse, input_tensor.ragged
        else:
            if shape is not None and batch_shape is not None:
                raise ValueError("You cannot pass both `shape` and `batch_shape` at the same time.")
            if batch_size is not None and batch_shape is not None and batch_shape[0] != batch_size:
                raise ValueError("When providing `batch_shape`, you cannot provide an incompatible `batch_size` argument.")
            if shape is None and batch_shape is None:
                raise ValueError("You must pass a `shape` argument.")
            if shape is not None:
                if isinstance(shape, int):
                    shape = (shape,)
                batch_shape = (batch_size,) + tuple(shape)
        self._batch_shape = tuple(None if d is None else int(d) for d in batch_shape)
        self._dtype = standardize_dtype(dtype or config.floatx())
        self.sparse = bool(sparse)
        self.ragged = bool(ragged)
        if input_tensor is None:
            input_tensor = KerasTensor(self._batch_shape, dtype=self._dtype, sparse=self.sparse, ragged=self.ragged, name=self.name)
        self._input_tensor = input_tensor
        Node(operation=self, call_args=(), call_kwargs={}, outputs=input_tensor)
        self.built = True
        self.optional = optional

    def call(self):
        return

    batch_shape = property(lambda self: self._batch_shape)
    dtype = property(lambda self: self._dtype)

    def get_config(self):
        return {"batch_shape": self.batch_shape, "dtype": self.dtype, "sparse": self.sparse, "ragged": self.ragged, "name": self.name, "optional": self.optional}


@keras_export(["keras.layers.Input", "keras.Input"])
def Input(shape=None, batch_size=None, dtype=None, sparse=None, ragged=None, batch_shape=None, name=None, tensor=None, optional=False):
    layer = InputLayer(shape=shape, batch_size=batch_size, dtype=dtype, sparse=sparse, ragged=ragged, batch_shape=batch_shape, name=name, input_tensor=tensor, optional=optional)
    return layer.output
