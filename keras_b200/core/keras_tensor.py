"""Symbolic tensor: a (shape, dtype) placeholder that records which op produced it.

Reference behaviour: keras/src/backend/common/keras_tensor.py:7-425.
"""

from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.naming import auto_name


def standardize_shape(shape):
    if shape is None:
        raise ValueError("Undefined shapes are not supported.")
    if not hasattr(shape, "__iter__"):
        raise ValueError(f"Cannot convert '{shape}' to a shape.")
    out = []
    for d in shape:
        if d is None:
            out.append(None)
            continue
        try:
            di = int(d)
        except (TypeError, ValueError):
            raise ValueError(f"Cannot convert '{shape}' to a shape. Found invalid entry '{d}'.")
        if di != d:
            raise ValueError(f"Cannot convert '{shape}' to a shape. Found invalid entry '{d}'.")
        if di < 0:
            raise ValueError(f"Cannot convert '{shape}' to a shape. Negative dimensions are not allowed.")
        out.append(di)
    return tuple(out)


@keras_export("keras.KerasTensor")
class KerasTensor:
    def __init__(self, shape, dtype="float32", sparse=False, ragged=False, record_history=True, name=None, **kwargs):
        self._shape = standardize_shape(shape)
        self._dtype = standardize_dtype(dtype)
        self._sparse = bool(sparse)
        self._ragged = bool(ragged)
        if self._sparse and self._ragged:
            raise ValueError("KerasTensor cannot have `sparse=True` and `ragged=True` at the same time.")
        self.name = name or auto_name(self.__class__.__name__)
        self.record_history = record_history

    shape = property(lambda self: self._shape)
    dtype = property(lambda self: self._dtype)
    sparse = property(lambda self: self._sparse)
    ragged = property(lambda self: self._ragged)

    @shape.setter
    def shape(self, value):
        raise AttributeError("The `shape` attribute of KerasTensor is immutable. One should create a new instance of KerasTensor for this.")

    @property
    def ndim(self):
        return len(self._shape)

    def reshape(self, newshape):
        from keras_b200 import ops

        return ops.reshape(self, newshape)

    def squeeze(self, axis=None):
        from keras_b200 import ops

        return ops.squeeze(self, axis)

    def __int__(self):
        raise ValueError("A KerasTensor is symbolic: it's a placeholder for a shape and a dtype. It doesn't have any actual numerical value. You cannot convert it to an int.")

    def __float__(self):
        raise ValueError("A KerasTensor is symbolic: it's a placeholder for a shape and a dtype. It doesn't have any actual numerical value. You cannot convert it to a float.")

    def __array__(self, *a, **k):
        raise ValueError("A KerasTensor is symbolic: it's a placeholder for a shape and a dtype. It doesn't have any actual numerical value. You cannot convert it to a NumPy array.")

    def __bool__(self):
        raise TypeError("A symbolic KerasTensor cannot be used as a boolean.")

    def __iter__(self):
        raise NotImplementedError("Iterating over a symbolic KerasTensor is not supported.")

    def __repr__(self):
        return f"<KerasTensor shape={self.shape}, dtype={self.dtype}, sparse={self.sparse}, ragged={self.ragged}, name={self.name}>"

    def __hash__(self):
        return id(self)

    def __getitem__(self, key):
        from keras_b200 import ops

        return ops.get_item(self, key)


def _bin(name, swap=False):
    def method(self, other):
        from keras_b200 import ops

        fn = getattr(ops, name)
        return fn(other, self) if swap else fn(self, other)

    return method


def _un(name):
    def method(self):
        from keras_b200 import ops

        return getattr(ops, name)(self)

    return method


for _dunder, _op in {
    "add": "add", "sub": "subtract", "mul": "multiply", "truediv": "divide",
    "floordiv": "floor_divide", "mod": "mod", "pow": "power", "matmul": "matmul",
    "and": "logical_and", "or": "logical_or", "xor": "logical_xor",
}.items():
    setattr(KerasTensor, f"__{_dunder}__", _bin(_op))
    setattr(KerasTensor, f"__r{_dunder}__", _bin(_op, swap=True))
for _dunder, _op in {
    "lt": "less", "le": "less_equal", "gt": "greater", "ge": "greater_equal", "ne": "not_equal",
}.items():
    setattr(KerasTensor, f"__{_dunder}__", _bin(_op))
KerasTensor.__eq__ = _bin("equal")
KerasTensor.__neg__ = _un("negative")
KerasTensor.__abs__ = _un("absolute")
KerasTensor.__invert__ = _un("logical_not")
KerasTensor.__div__ = _bin("divide")
KerasTensor.__rdiv__ = _bin("divide", swap=True)
KerasTensor.__round__ = lambda self, ndigits=None: __import__("keras_b200").ops.round(self, ndigits or 0)


def any_symbolic_tensors(args=None, kwargs=None):
    """True when any leaf of (args, kwargs) is a KerasTensor."""
    for x in args or ():
        if isinstance(x, KerasTensor):
            return True
        if isinstance(x, (list, tuple, dict)) and _has_symbolic(x):
            return True
    if kwargs:
        for x in kwargs.values():
            if isinstance(x, KerasTensor):
                return True
            if isinstance(x, (list, tuple, dict)) and _has_symbolic(x):
                return True
    return False


def _has_symbolic(x):
    if isinstance(x, KerasTensor):
        return True
    if isinstance(x, dict):
        return any(_has_symbolic(v) for v in x.values())
    if isinstance(x, (list, tuple)):
        return any(_has_symbolic(v) for v in x)
    return False


@keras_export(["keras.utils.is_keras_tensor", "keras.backend.is_keras_tensor"])
def is_keras_tensor(x):
    return isinstance(x, KerasTensor)
