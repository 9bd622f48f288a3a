"""``DataLayer``: base of preprocessing layers that may run inside input pipelines
(keras/src/layers/preprocessing/data_layer.py:10).  The reference swaps compute backends when called from
tf.data/grain; here there is one tensor runtime, so ``self.backend`` is a fixed namespace exposing the same
attribute layout (``numpy``, ``nn``, ``image``, ``random``, ``core``, ``convert_to_tensor``, ``shape``, ``cast``)."""

from keras_b200.layers.layer import Layer


class _Namespace:
    name = "torch"
    _backend = "torch"

    def __getattr__(self, item):
        from keras_b200 import ops, random

        if item == "random":
            return random
        if item in ("numpy", "nn", "image", "core", "math", "linalg"):
            mod = getattr(ops, item, None)
            return mod if mod is not None else ops
        return getattr(ops, item)

    def set_backend(self, name):
        pass

    def reset(self):
        pass


class DataLayer(Layer):
    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.backend = _Namespace()
        self._allow_non_tensor_positional_args = True

    def _get_seed_generator(self, backend=None):
        if not hasattr(self, "seed") or not hasattr(self, "generator"):
            raise ValueError("The `seed` and `generator` variable must be set in the `__init__` method before calling `_get_seed_generator()`.")
        return self.generator

    def convert_weight(self, weight):
        return weight
