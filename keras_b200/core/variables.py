"""``Variable``: a named, trainable tensor backed by a ``torch.nn.Parameter``.

Behaviour follows keras/src/backend/common/variables.py:15-553 and
keras/src/backend/torch/core.py:110-195.  Additions of this framework: a variable may be a
*shard* of a larger logical tensor (``layout`` / ``global_shape`` / ``shard_spec``), which is
how ``ModelParallel`` places weights; the reference's torch backend never applies layouts.
"""

import numpy as np
import torch

from keras_b200.core import config, global_state
from keras_b200.core.dtypes import standardize_dtype, to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import standardize_shape
from keras_b200.core.naming import auto_name
from keras_b200.core.scopes import current_path, get_stateless_scope, in_stateless_scope
from keras_b200.core.tensor import convert_to_tensor, get_device

_FLOAT_TORCH = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


@keras_export("keras.Variable")
class Variable:
    def __init__(
        self,
        initializer,
        shape=None,
        dtype=None,
        trainable=True,
        autocast=True,
        aggregation="none",
        synchronization="auto",
        name=None,
        layout=None,
        **kwargs,
    ):
        name = name or auto_name(self.__class__.__name__)
        if not isinstance(name, str) or "/" in name:
            raise ValueError(
                "Argument `name` must be a string and cannot contain character `/`. "
                f"Received: name={name}"
            )
        if aggregation not in (None, "none", "mean", "sum", "only_first_replica"):
            raise ValueError(
                "Invalid value for argument `aggregation`. Expected one of "
                "`None`, `'none'`, `'mean'`, `'sum'`, `'only_first_replica'`. "
                f"Received: aggregation={aggregation}"
            )
        if aggregation is None:
            aggregation = "none"
        if synchronization not in (None, "none", "on_read", "on_write", "auto"):
            raise ValueError(
                "Invalid value for argument `synchronization`. Expected one of "
                "`None`, `'none'`, `'on_read'`, `'on_write'`, `'auto'`. "
                f"Received: synchronization={synchronization}"
            )
        if synchronization is None:
            synchronization = "none"
        self._name = name
        parent = current_path()
        self._path = f"{parent}/{name}" if parent else name
        self._shape = None
        self._initializer = None
        self._regularizer = None
        self._constraint = None
        self._trainable = bool(trainable)
        self._autocast = bool(autocast)
        self._aggregation = aggregation
        self._synchronization = synchronization
        self._overwrite_with_gradient = False
        self._layout = layout
        self._global_shape = None
        self._shard_slices = None
        self._shard_spec = None
        self._value = None
        self._shadow = None
        if isinstance(initializer, str):
            from keras_b200 import initializers

            initializer = initializers.get(initializer)
        if callable(initializer):
            if shape is None:
                raise ValueError(
                    "When creating a Variable from an initializer, the `shape` argument should be "
                    f"specified. Received: initializer={initializer} and shape={shape}"
                )
        else:
            if not isinstance(initializer, torch.nn.Parameter):  # a Parameter is adopted as the storage itself
                initializer = _as_init_value(initializer, dtype)
            if dtype is None:
                dtype = initializer.dtype
        self._dtype = standardize_dtype(dtype)
        self._torch_dtype = to_torch_dtype(self._dtype)
        self._is_float = self._torch_dtype in _FLOAT_TORCH

        if in_stateless_scope():
            if callable(initializer):
                self._initializer = initializer
                self._shape = self._validate_shape(shape)
                _register_uninitialized(self)
            else:
                raise ValueError(
                    "You are attempting to create a variable while in a stateless scope. This is "
                    "disallowed. Make sure that all variables are created before you start using "
                    "your layer/model objects.\n\nIn some cases, you might be seeing this error "
                    "because you need to implement a `def build(self, input_shape)` method on "
                    "your layer/model, which will create its variables.\n\nIn some other cases, "
                    "you might be seeing this error because you are instantiating a `Variable` "
                    "and assigning it to a layer without going through self.add_variable()/"
                    "self.add_weight(). Always prefer using these methods (with a `shape` and "
                    "`initializer` argument)."
                )
        else:
            if callable(initializer):
                self._shape = self._validate_shape(shape)
                self._initialize_with_initializer(initializer)
            else:
                self._initialize(initializer)
                self._shape = tuple(self._value.shape)
        self._ndim = len(self._shape)

    # -- initialisation ------------------------------------------------------------------
    def _validate_shape(self, shape):
        shape = standardize_shape(shape)
        if None in shape:
            raise ValueError(
                "Shapes used to initialize variables must be fully-defined (no `None` dimensions). "
                f"Received: shape={shape} for variable path='{self._path}'"
            )
        return shape

    def _deferred_initialize(self):
        if self._value is not None:
            raise ValueError(f"Variable {self._path} is already initialized.")
        if in_stateless_scope():
            raise ValueError(
                "You are attempting to initialize a variable while in a stateless scope. "
                "This is disallowed. Make sure that all variables are initialized before you "
                "start using your layer/model objects."
            )
        self._initialize_with_initializer(self._initializer)
        self._initializer = None

    def _initialize_with_initializer(self, initializer):
        from keras_b200.distribution import distribution_lib

        dist = distribution_lib.distribution()
        if dist is not None and self._layout is None:
            self._layout = dist.get_variable_layout(self)
        if self._layout is not None and dist is not None and hasattr(dist, "shard_variable_init"):
            value = dist.shard_variable_init(self, initializer)
            if value is not None:
                self._initialize(value)
                return
        value = initializer(self._shape, dtype=self._dtype)
        self._initialize(value)

    def _initialize(self, value):
        if isinstance(value, torch.nn.Parameter):
            self._value = value
            return
        t = convert_to_tensor(value, dtype=self._torch_dtype)
        dev = get_device()
        if t.device != dev and t.device.type != "meta":
            t = t.to(dev)
        t = t.detach()
        if t.requires_grad or not t.is_contiguous():
            t = t.contiguous()
        self._value = torch.nn.Parameter(t.clone() if t.data_ptr() != 0 and t._base is not None else t,
                                         requires_grad=self._trainable and self._is_float)

    # -- properties ----------------------------------------------------------------------
    name = property(lambda self: self._name)
    path = property(lambda self: self._path)
    shape = property(lambda self: self._shape)
    ndim = property(lambda self: self._ndim)
    dtype = property(lambda self: self._dtype)
    aggregation = property(lambda self: self._aggregation)
    synchronization = property(lambda self: self._synchronization)

    @property
    def global_shape(self):
        """Shape of the logical tensor; differs from ``shape`` for sharded variables."""
        return self._global_shape or self._shape

    @property
    def value(self):
        scope = get_stateless_scope()
        if scope is not None:
            v = scope.get_current_value(self)
            if v is not None:
                return self._maybe_autocast(v)
        if self._value is None:
            # Uninitialized (created in a stateless scope): produce a throw-away value.
            v = self._initializer(self._shape, dtype=self._dtype)
            return self._maybe_autocast(convert_to_tensor(v, dtype=self._torch_dtype))
        if global_state.get_global_attribute("symbolic_scope") is not None:
            # shape inference runs on placeholder tensors of another device (meta, or the CPU fallback): follow it
            dev = global_state.get_global_attribute("torch_device")
            if dev is not None and dev != self._value.device:
                shape = self._global_shape or self._shape
                if dev.type == "meta" or self._shard_slices is not None:
                    return self._maybe_autocast(torch.empty(tuple(shape), dtype=self._value.dtype, device=dev))
                return self._maybe_autocast(self._value.to(dev))
        if self._shard_slices is not None:
            from keras_b200.parallel import tensor_parallel

            if not tensor_parallel.in_local_shards():
                return self._maybe_autocast(tensor_parallel.gather_variable(self))
        return self._maybe_autocast(self._value)

    def _maybe_autocast(self, value):
        if self._autocast and self._is_float:
            scope = global_state.get_global_attribute("autocast_scope")
            if scope is not None and scope.torch_dtype is not None and value.dtype != scope.torch_dtype:
                shadow = self._shadow
                if shadow is not None and value is self._value and shadow[0] == scope.torch_dtype:
                    return shadow[1](value)
                return value.to(scope.torch_dtype)
        return value

    def _direct_assign(self, value):
        with torch.no_grad():
            if self._shard_slices is not None and tuple(value.shape) != tuple(self._value.shape):
                value = value[self._shard_slices]
            self._value.copy_(value)
        if self._shadow is not None:
            self._shadow[2]()

    def assign(self, value):
        value = convert_to_tensor(value, dtype=self._torch_dtype)
        if tuple(value.shape) != tuple(self._shape):
            raise ValueError(
                "The shape of the target variable and the shape of the target value in "
                "`variable.assign(value)` must match. "
                f"variable.shape={tuple(self._shape)}, Received: value.shape={tuple(value.shape)}. "
                f"Target variable: {self}"
            )
        scope = get_stateless_scope()
        if scope is not None:
            scope.add_update((self, value))
        else:
            self._direct_assign(value)
        return value

    def assign_add(self, value):
        return self.assign(self.value_unautocast() + convert_to_tensor(value, dtype=self._torch_dtype))

    def assign_sub(self, value):
        return self.assign(self.value_unautocast() - convert_to_tensor(value, dtype=self._torch_dtype))

    def value_unautocast(self):
        scope = get_stateless_scope()
        if scope is not None:
            v = scope.get_current_value(self)
            if v is not None:
                return v
        if self._value is None:
            return convert_to_tensor(self._initializer(self._shape, dtype=self._dtype), dtype=self._torch_dtype)
        if self._shard_slices is not None:
            from keras_b200.parallel import tensor_parallel

            if not tensor_parallel.in_local_shards():
                return tensor_parallel.gather_variable(self)
        return self._value

    @property
    def trainable(self):
        return self._trainable

    @trainable.setter
    def trainable(self, value):
        self._trainable = bool(value)
        if self._value is not None:
            self._value.requires_grad = self._trainable and self._is_float

    @property
    def overwrite_with_gradient(self):
        return self._overwrite_with_gradient

    @overwrite_with_gradient.setter
    def overwrite_with_gradient(self, value):
        if not isinstance(value, bool):
            raise TypeError(f"`overwrite_with_gradient` must be a boolean. Received: {value}")
        self._overwrite_with_gradient = value

    @property
    def regularizer(self):
        return self._regularizer

    @regularizer.setter
    def regularizer(self, value):
        from keras_b200.regularizers import Regularizer

        if value is not None and not isinstance(value, Regularizer):
            raise ValueError(
                "Invalid value for attribute `regularizer`. Expected an instance of "
                f"`keras.regularizers.Regularizer`, or `None`. Received: regularizer={value}"
            )
        self._regularizer = value

    @property
    def constraint(self):
        return self._constraint

    @constraint.setter
    def constraint(self, value):
        from keras_b200.constraints import Constraint

        if value is not None and not isinstance(value, Constraint):
            raise ValueError(
                "Invalid value for attribute `constraint`. Expected an instance of "
                f"`keras.constraints.Constraint`, or `None`. Received: constraint={value}"
            )
        self._constraint = value

    @property
    def layout(self):
        return self._layout

    @layout.setter
    def layout(self, value):
        self._layout = value

    def numpy(self):
        from keras_b200.core.tensor import convert_to_numpy

        return convert_to_numpy(self.value_unautocast())

    def __repr__(self):
        val = None
        if self._value is not None and not in_stateless_scope():
            try:
                val = self.numpy()
            except Exception:
                val = None
        vs = f", value={val}" if val is not None else ""
        return f"<Variable path={self._path}, shape={self._shape}, dtype={self._dtype}{vs}>"

    def __hash__(self):
        return id(self)

    def __bool__(self):
        raise TypeError("A Keras Variable cannot be used as a boolean.")

    def __array__(self, dtype=None, copy=None):
        arr = self.numpy()
        return arr.astype(dtype) if dtype is not None else arr

    def __getitem__(self, idx):
        return self.value.__getitem__(idx)

    def __int__(self):
        if self._ndim > 0:
            raise TypeError(f"Only scalar arrays can be converted to Python scalars. Got: shape={self._shape}")
        return int(self.value)

    def __float__(self):
        if self._ndim > 0:
            raise TypeError(f"Only scalar arrays can be converted to Python scalars. Got: shape={self._shape}")
        return float(self.value)

    def __len__(self):
        return self._shape[0]

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        args = [a.value if isinstance(a, Variable) else a for a in args]
        kwargs = {k: (v.value if isinstance(v, Variable) else v) for k, v in (kwargs or {}).items()}
        return func(*args, **kwargs)

    def _convert(self, other):
        return other.value if isinstance(other, Variable) else other


def _arith(name, swap=False):
    def method(self, other):
        from keras_b200 import ops

        fn = getattr(ops, name)
        return fn(other, self.value) if swap else fn(self.value, other)

    return method


for _d, _o in {
    "add": "add", "sub": "subtract", "mul": "multiply", "truediv": "divide",
    "floordiv": "floor_divide", "mod": "mod", "pow": "power", "matmul": "matmul",
    "and": "logical_and", "or": "logical_or", "xor": "logical_xor",
}.items():
    setattr(Variable, f"__{_d}__", _arith(_o))
    setattr(Variable, f"__r{_d}__", _arith(_o, swap=True))
for _d, _o in {"lt": "less", "le": "less_equal", "gt": "greater", "ge": "greater_equal", "ne": "not_equal", "eq": "equal"}.items():
    setattr(Variable, f"__{_d}__", _arith(_o))
Variable.__neg__ = lambda self: -self.value
Variable.__pos__ = lambda self: self.value
Variable.__abs__ = lambda self: abs(self.value)
Variable.__invert__ = lambda self: ~self.value
Variable.__round__ = lambda self, ndigits=None: __import__("keras_b200").ops.round(self.value, ndigits or 0)


def _as_init_value(value, dtype):
    if isinstance(value, Variable):
        value = value.value
    if isinstance(value, torch.Tensor):
        return value.detach().to(to_torch_dtype(dtype)) if dtype is not None else value.detach()
    if dtype is None:
        if isinstance(value, float) or (isinstance(value, (list, tuple)) and _all_float(value)):
            dtype = config.floatx()
        elif isinstance(value, np.ndarray) and value.dtype == np.float64:
            dtype = None
    return convert_to_tensor(value, dtype=dtype)


def _all_float(x):
    flat = np.asarray(x)
    return flat.dtype.kind == "f"


def _register_uninitialized(variable):
    pending = global_state.get_global_attribute("uninitialized_variables", default=[], set_to_default=True)
    pending.append(variable)


def initialize_all_variables():
    pending = global_state.get_global_attribute("uninitialized_variables")
    if pending:
        for v in pending:
            v._deferred_initialize()
    global_state.set_global_attribute("uninitialized_variables", [])


class AutocastScope:
    """While active, float variables read as ``dtype`` (keras/src/backend/common/variables.py:677-708)."""

    def __init__(self, dtype):
        if dtype is not None:
            dtype = standardize_dtype(dtype)
            if not (dtype.startswith("float") or dtype == "bfloat16"):
                raise ValueError(
                    "`AutocastScope` can only be used with a floating-point target dtype, such as "
                    f"'float16'. Received: dtype={dtype}"
                )
        self.dtype = dtype
        self.torch_dtype = to_torch_dtype(dtype) if dtype is not None else None
        self._outer = None

    def maybe_cast(self, value):
        if self.torch_dtype is not None and value.dtype in _FLOAT_TORCH and value.dtype != self.torch_dtype:
            return value.to(self.torch_dtype)
        return value

    def __enter__(self):
        self._outer = global_state.get_global_attribute("autocast_scope")
        global_state.set_global_attribute("autocast_scope", self)
        return self

    def __exit__(self, *exc):
        global_state.set_global_attribute("autocast_scope", self._outer)


def get_autocast_scope():
    return global_state.get_global_attribute("autocast_scope")


def shape_equal(a, b):
    a, b = tuple(a), tuple(b)
    if len(a) != len(b):
        return False
    return all(x is None or y is None or x == y for x, y in zip(a, b))
