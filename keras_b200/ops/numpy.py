"""NumPy-API ops (``keras.ops.*`` / ``keras.ops.numpy.*``) on torch tensors.

Function list and dtype rules follow keras/src/ops/numpy.py and keras/src/backend/torch/numpy.py;
implementations are written directly against torch.
"""

import builtins
import math

import numpy as np
import torch

from keras_b200.core import config
from keras_b200.core.dtypes import (
    is_float as _is_float_name,
    result_type,
    standardize_dtype,
    to_torch_dtype,
)
from keras_b200.core.tensor import cast, convert_to_tensor, get_device
from keras_b200.core.variables import Variable
from keras_b200.ops._dispatch import op

_T = torch.Tensor
_FLOATS = (torch.float16, torch.bfloat16, torch.float32, torch.float64)
_COMPLEX = (torch.complex64, torch.complex128)


def _t(x, dtype=None):
    if type(x) is _T and dtype is None:
        return x
    return convert_to_tensor(x, dtype)


def _dt(x):
    """dtype spelling usable by ``result_type``: tensor dtype, or Python type for scalars."""
    if isinstance(x, Variable):
        return x.value.dtype
    if isinstance(x, _T):
        return x.dtype
    if isinstance(x, np.generic):
        return x.dtype  # np.float64 subclasses float, but it carries a dtype: not a weak Python scalar
    if isinstance(x, bool):
        return "bool"
    if isinstance(x, int):
        return int
    if isinstance(x, float):
        return float
    if hasattr(x, "dtype"):
        return x.dtype
    return convert_to_tensor(x).dtype


def _pair(x1, x2):
    """Promote two operands to their common Keras dtype."""
    if type(x1) is _T and type(x2) is _T and x1.dtype == x2.dtype:
        return x1, x2
    if isinstance(x1, Variable):
        x1 = x1.value
    if isinstance(x2, Variable):
        x2 = x2.value
    if type(x1) is _T and type(x2) is _T and x1.dtype == x2.dtype:
        return x1, x2
    d = to_torch_dtype(result_type(_dt(x1), _dt(x2)))
    return convert_to_tensor(x1, d), convert_to_tensor(x2, d)


def _pair_native(x1, x2):
    """Both operands as tensors, promoted by torch's own rule (0-dim operands count as scalars).  The reference hands the
    operands of add, subtract, multiply, power, where, append, kron, outer, mod, gcd, lcm and the bitwise ops to torch
    unpromoted (keras/src/backend/torch/numpy.py:68-71 and the like), so 64-bit operands keep 64 bits there although
    ``result_type`` would narrow them."""
    if isinstance(x1, Variable):
        x1 = x1.value
    if isinstance(x2, Variable):
        x2 = x2.value
    if type(x1) is _T and type(x2) is _T and x1.dtype == x2.dtype:
        return x1, x2
    a, b = convert_to_tensor(x1), convert_to_tensor(x2)
    if a.dtype == b.dtype:
        return a, b
    d = torch.result_type(a, b)
    return a.to(d), b.to(d)


def _dt_converted(x):
    """dtype an operand has once the reference has passed it through ``convert_to_tensor``: a Python int is int32 and a Python
    float is floatx from then on, no longer a weakly typed scalar."""
    if isinstance(x, bool):
        return "bool"
    if isinstance(x, int) and not isinstance(x, np.generic):
        return "int32" if -(2 ** 31) <= x < 2 ** 31 else "int64"
    if isinstance(x, float) and not isinstance(x, np.generic):
        return config.floatx()
    return _dt(x)


def _pair_strict(x1, x2):
    """Both operands cast to ``result_type`` of their dtypes even when the dtypes are equal: ops that resolve their dtype that
    way in the reference (maximum, minimum, floor_divide, the products) turn int64 into int32 and float64 into float32."""
    if isinstance(x1, Variable):
        x1 = x1.value
    if isinstance(x2, Variable):
        x2 = x2.value
    d = to_torch_dtype(result_type(_dt(x1), _dt(x2)))
    return convert_to_tensor(x1, d), convert_to_tensor(x2, d)


def _pair_converted(x1, x2, floating=False):
    """``result_type`` of the operands' dtypes after conversion to tensors (Python scalars typed, see ``_dt_converted``),
    optionally lifted to a float type: arctan2, hypot, logaddexp, nextafter, the dot products, cross, tensordot."""
    if isinstance(x1, Variable):
        x1 = x1.value
    if isinstance(x2, Variable):
        x2 = x2.value
    kinds = (_dt_converted(x1), _dt_converted(x2)) + ((float,) if floating else ())
    d = to_torch_dtype(result_type(*kinds))
    return convert_to_tensor(x1, d), convert_to_tensor(x2, d)


def _pair_full(x1, x2):
    """torch's promotion without the scalar rule (0-dim operands count like any other): what concatenation and the outer /
    Kronecker products apply."""
    if isinstance(x1, Variable):
        x1 = x1.value
    if isinstance(x2, Variable):
        x2 = x2.value
    a, b = convert_to_tensor(x1), convert_to_tensor(x2)
    if a.dtype == b.dtype:
        return a, b
    d = torch.promote_types(a.dtype, b.dtype)
    return a.to(d), b.to(d)


def _narrow64(x):
    """``result_type`` of a single dtype: 64-bit types become their 32-bit counterparts."""
    d = to_torch_dtype(result_type(_dt(x)))
    return x if x.dtype == d else x.to(d)


def _floatize(x):
    """ints/bools → floatx; floats unchanged."""
    x = _t(x)
    if x.dtype in _FLOATS or x.dtype in _COMPLEX:
        return x
    return x.to(to_torch_dtype(config.floatx()))


def _pair_float(x1, x2):
    if isinstance(x1, Variable):
        x1 = x1.value
    if isinstance(x2, Variable):
        x2 = x2.value
    d = to_torch_dtype(result_type(_dt(x1), _dt(x2), float))
    return convert_to_tensor(x1, d), convert_to_tensor(x2, d)


def _axis(axis):
    if axis is None:
        return None
    if isinstance(axis, (list, tuple)):
        return tuple(int(a) for a in axis)
    return int(axis)


def _unary_float(torch_fn):
    def f(x):
        return torch_fn(_floatize(x))

    return f


def _reg_unary_float(name, torch_fn):
    def f(x):
        return torch_fn(_floatize(x))

    f.__name__ = name
    f.__qualname__ = name
    globals()[name] = op("numpy")(f)


for _n, _f in {
    "arccos": torch.arccos, "arccosh": torch.arccosh, "arcsin": torch.arcsin,
    "arcsinh": torch.arcsinh, "arctan": torch.arctan, "arctanh": torch.arctanh,
    "cos": torch.cos, "cosh": torch.cosh, "exp": torch.exp, "exp2": torch.exp2,
    "expm1": torch.expm1, "log": torch.log, "log10": torch.log10, "log1p": torch.log1p,
    "log2": torch.log2, "sin": torch.sin, "sinh": torch.sinh, "sqrt": torch.sqrt,
    "tan": torch.tan, "tanh": torch.tanh, "sinc": torch.sinc, "i0": torch.i0,
    "reciprocal": torch.reciprocal,
}.items():
    _reg_unary_float(_n, _f)


def _reg_angle(name, torch_fn):
    def f(x):
        x = _t(x)
        # int64 degrees / radians come back as float64 (keras/src/backend/torch/numpy.py deg2rad, rad2deg)
        return torch_fn(x.to(torch.float64)) if x.dtype == torch.int64 else torch_fn(_floatize(x))

    f.__name__ = name
    f.__qualname__ = name
    globals()[name] = op("numpy")(f)


_reg_angle("deg2rad", torch.deg2rad)
_reg_angle("rad2deg", torch.rad2deg)


@op("numpy")
def cbrt(x):
    x = _t(x)
    x = x.to(torch.float64) if x.dtype == torch.int64 else _floatize(x)
    return torch.sign(x) * torch.pow(torch.abs(x), 1.0 / 3.0)


# --- elementwise binary -------------------------------------------------------------------

@op("numpy")
def add(x1, x2):
    x1, x2 = _pair_native(x1, x2)
    return torch.add(x1, x2) if x1.dtype != torch.bool else torch.logical_or(x1, x2)


@op("numpy")
def subtract(x1, x2):
    x1, x2 = _pair_native(x1, x2)
    if x1.dtype == torch.bool:
        x1, x2 = x1.to(torch.int32), x2.to(torch.int32)
    return torch.subtract(x1, x2)


@op("numpy")
def multiply(x1, x2):
    x1, x2 = _pair_native(x1, x2)
    return torch.multiply(x1, x2) if x1.dtype != torch.bool else torch.logical_and(x1, x2)


@op("numpy", also=("keras.ops.true_divide", "keras.ops.numpy.true_divide"))
def divide(x1, x2):
    # torch's true division of the operands as they are: float64 stays float64, integer by integer gives floatx
    # (keras/src/backend/torch/numpy.py divide)
    if isinstance(x1, Variable):
        x1 = x1.value
    if isinstance(x2, Variable):
        x2 = x2.value
    if not isinstance(x1, (int, float)):
        x1 = convert_to_tensor(x1)
    if not isinstance(x2, (int, float)):
        x2 = convert_to_tensor(x2)
    if not isinstance(x1, _T) and not isinstance(x2, _T):
        x1 = convert_to_tensor(x1)
    return torch.divide(x1, x2)


true_divide = divide


@op("numpy")
def divide_no_nan(x1, x2):
    x1, x2 = _pair_float(x1, x2)
    return torch.where(x2 == 0, torch.zeros((), dtype=x1.dtype, device=x1.device), x1 / x2)


@op("numpy")
def floor_divide(x1, x2):
    x1, x2 = _pair_strict(x1, x2)
    return torch.floor_divide(x1, x2)


@op("numpy")
def mod(x1, x2):
    x1, x2 = _pair_native(x1, x2)
    if x1.dtype == torch.bool:
        x1, x2 = x1.to(torch.int32), x2.to(torch.int32)
    return torch.remainder(x1, x2)


@op("numpy")
def fmod(x1, x2):
    x1, x2 = _pair_native(x1, x2)
    if x1.dtype == torch.bool:
        x1, x2 = x1.to(torch.int32), x2.to(torch.int32)
    return torch.fmod(x1, x2)


@op("numpy")
def power(x1, x2):
    x1, x2 = _pair_native(x1, x2)
    return torch.pow(x1, x2)


@op("numpy")
def maximum(x1, x2):
    x1, x2 = _pair_strict(x1, x2)
    return torch.maximum(x1, x2)


@op("numpy")
def minimum(x1, x2):
    x1, x2 = _pair_strict(x1, x2)
    return torch.minimum(x1, x2)


@op("numpy")
def fmax(x1, x2):
    x1, x2 = _pair(x1, x2)
    return torch.fmax(x1, x2)


@op("numpy")
def fmin(x1, x2):
    x1, x2 = _pair(x1, x2)
    return torch.fmin(x1, x2)


@op("numpy")
def arctan2(x1, x2):
    x1, x2 = _pair_converted(x1, x2, floating=True)
    return torch.arctan2(x1, x2)


@op("numpy")
def hypot(x1, x2):
    x1, x2 = _pair_converted(x1, x2, floating=True)
    return torch.hypot(x1, x2)


@op("numpy")
def logaddexp(x1, x2):
    x1, x2 = _pair_converted(x1, x2, floating=True)
    return torch.logaddexp(x1, x2)


@op("numpy")
def logaddexp2(x1, x2):
    x1, x2 = _pair_converted(x1, x2, floating=True)
    return torch.logaddexp2(x1, x2)


@op("numpy")
def nextafter(x1, x2):
    x1, x2 = _pair_converted(x1, x2, floating=True)
    return torch.nextafter(x1, x2)


@op("numpy")
def heaviside(x1, x2):
    x1, x2 = _pair_converted(x1, x2)
    if x1.dtype == torch.int64:
        x1, x2 = x1.to(torch.float64), x2.to(torch.float64)
    elif x1.dtype in (torch.int8, torch.int16, torch.int32, torch.uint8):
        f = to_torch_dtype(config.floatx())
        x1, x2 = x1.to(f), x2.to(f)
    return torch.heaviside(x1, x2)


@op("numpy")
def ldexp(x1, x2):
    x1, x2 = _t(x1), _t(x2)
    if x2.dtype in _FLOATS:
        raise TypeError(f"ldexp exponent must be an integer type. Received: x2 dtype={x2.dtype}")
    d = to_torch_dtype(result_type(x1.dtype, x2.dtype, float))
    return torch.ldexp(x1.to(d), x2).to(d)


@op("numpy")
def gcd(x1, x2):
    x1, x2 = _pair_native(x1, x2)
    return torch.gcd(x1, x2)


@op("numpy")
def lcm(x1, x2):
    x1, x2 = _pair_native(x1, x2)
    return torch.lcm(x1, x2)


@op("numpy")
def copysign(x1, x2):
    x1, x2 = _pair_float(x1, x2)
    return torch.copysign(x1, x2)


# comparisons
def _cmp(name, fn):
    def f(x1, x2):
        a, b = _pair(x1, x2)
        return fn(a, b)

    f.__name__ = name
    globals()[name] = op("numpy")(f)


for _n, _f in {
    "equal": torch.eq, "not_equal": torch.ne, "greater": torch.gt,
    "greater_equal": torch.ge, "less": torch.lt, "less_equal": torch.le,
}.items():
    _cmp(_n, _f)


def _logic(name, fn):
    def f(x1, x2):
        return fn(_t(x1).to(torch.bool), _t(x2).to(torch.bool))

    f.__name__ = name
    globals()[name] = op("numpy")(f)


for _n, _f in {"logical_and": torch.logical_and, "logical_or": torch.logical_or, "logical_xor": torch.logical_xor}.items():
    _logic(_n, _f)


@op("numpy")
def logical_not(x):
    return torch.logical_not(_t(x).to(torch.bool))


def _bitwise(name, fn):
    shift = "shift" in name

    def f(x, y):
        if shift and isinstance(y, int) and not isinstance(y, bool):
            return fn(_t(x), y)  # the count stays a Python int, as in keras/src/backend/torch/numpy.py bitwise_left_shift
        a, b = _pair_native(x, y)
        return fn(a, b)

    f.__name__ = name
    globals()[name] = op("numpy")(f)


for _n, _f in {
    "bitwise_and": torch.bitwise_and, "bitwise_or": torch.bitwise_or, "bitwise_xor": torch.bitwise_xor,
    "bitwise_left_shift": torch.bitwise_left_shift, "bitwise_right_shift": torch.bitwise_right_shift,
    "left_shift": torch.bitwise_left_shift, "right_shift": torch.bitwise_right_shift,
}.items():
    _bitwise(_n, _f)


@op("numpy", also=("keras.ops.bitwise_not", "keras.ops.numpy.bitwise_not"))
def bitwise_invert(x):
    return torch.bitwise_not(_t(x))


bitwise_not = bitwise_invert


# --- elementwise unary --------------------------------------------------------------------

@op("numpy", also=("keras.ops.abs", "keras.ops.numpy.abs"))
def absolute(x):
    x = _t(x)
    return x if x.dtype in (torch.uint8, torch.bool) else torch.abs(x)


abs = absolute


@op("numpy")
def fabs(x):
    return torch.abs(_floatize(x))


@op("numpy")
def negative(x):
    return torch.negative(_t(x))


@op("numpy")
def square(x):
    x = _t(x)
    if x.dtype == torch.bool:
        x = x.to(torch.int32)
    return torch.square(x)


@op("numpy")
def sign(x):
    return torch.sign(_t(x))


@op("numpy")
def signbit(x):
    return torch.signbit(_t(x))


@op("numpy")
def ceil(x):
    return torch.ceil(_narrow64(_floatize(x)))


@op("numpy")
def floor(x):
    return torch.floor(_narrow64(_floatize(x)))


@op("numpy")
def trunc(x):
    x = _t(x)
    return x if x.dtype not in _FLOATS else torch.trunc(x)


@op("numpy")
def round(x, decimals=0):
    x = _t(x)
    if x.dtype not in _FLOATS:
        if decimals >= 0:
            return x
        f = 10 ** (-decimals)
        return (torch.round(x.to(torch.float64) / f) * f).to(x.dtype)
    return torch.round(x, decimals=decimals)


@op("numpy")
def clip(x, x_min, x_max):
    x = _t(x)
    if x.dtype == torch.bool:
        x = x.to(torch.int32)
    def scalar(b):
        return b is None or (isinstance(b, (int, float)) and not isinstance(b, np.generic))

    if scalar(x_min) and scalar(x_max):
        return torch.clip(x, x_min, x_max)
    # a bound that is an array or a tensor: torch wants both bounds as tensors then
    lo = None if x_min is None else _t(x_min).to(x.dtype)
    hi = None if x_max is None else _t(x_max).to(x.dtype)
    return torch.clip(x, lo, hi)


@op("numpy")
def isfinite(x):
    return torch.isfinite(_t(x))


@op("numpy")
def isinf(x):
    return torch.isinf(_t(x))


@op("numpy")
def isnan(x):
    return torch.isnan(_t(x))


@op("numpy")
def isneginf(x):
    return torch.isneginf(_t(x))


@op("numpy")
def isposinf(x):
    return torch.isposinf(_t(x))


@op("numpy")
def isreal(x):
    return torch.isreal(_t(x))


@op("numpy")
def real(x):
    x = _t(x)
    return torch.real(x) if x.is_complex() else x


@op("numpy")
def imag(x):
    x = _t(x)
    return torch.imag(x) if x.is_complex() else torch.zeros_like(x)


@op("numpy", also=("keras.ops.conj", "keras.ops.numpy.conj"))
def conjugate(x):
    x = _t(x)
    return torch.conj(x).resolve_conj() if x.is_complex() else x


conj = conjugate


@op("numpy")
def angle(x):
    return torch.angle(_floatize(x))


@op("numpy")
def nan_to_num(x, nan=0.0, posinf=None, neginf=None):
    return torch.nan_to_num(_t(x), nan=nan, posinf=posinf, neginf=neginf)


# --- reductions ---------------------------------------------------------------------------

def _promote_sum_dtype(x):
    if x.dtype == torch.bool:
        return x.to(torch.int32)
    if x.dtype in (torch.int8, torch.int16):
        return x.to(torch.int32)
    if x.dtype == torch.uint8:
        return x.to(torch.int32)  # the reference's torch backend has no uint32 and uses int32
    return x


@op("numpy")
def sum(x, axis=None, keepdims=False):
    x = _promote_sum_dtype(_t(x))
    if axis is None:
        r = torch.sum(x, dtype=x.dtype)
        return r.reshape((1,) * x.ndim) if keepdims else r
    if axis == ():
        return x
    return torch.sum(x, dim=_axis(axis), keepdim=keepdims, dtype=x.dtype)


@op("numpy")
def prod(x, axis=None, keepdims=False, dtype=None):
    x = _promote_sum_dtype(_t(x))
    if dtype is not None:
        x = x.to(to_torch_dtype(dtype))
    else:
        x = _narrow64(x)  # result_type of the input's dtype (keras/src/backend/torch/numpy.py prod)
    if axis is None:
        r = torch.prod(x, dtype=x.dtype)
        return r.reshape((1,) * x.ndim) if keepdims else r
    if not isinstance(axis, (list, tuple)):
        axis = (axis,)
    for a in sorted([a % x.ndim for a in axis], reverse=True):
        x = torch.prod(x, dim=a, keepdim=keepdims, dtype=x.dtype)
    return x


@op("numpy")
def mean(x, axis=None, keepdims=False):
    x = _t(x)
    if isinstance(axis, (list, tuple)) and len(axis) == 0:
        return x
    ori = x.dtype
    if ori in _FLOATS:
        compute = torch.float32 if ori in (torch.float16, torch.bfloat16) else ori
        out_dtype = ori
    else:
        compute = out_dtype = to_torch_dtype(config.floatx())
        if ori == torch.int64:
            pass
    r = torch.mean(x.to(compute), dim=_axis(axis), keepdim=keepdims) if axis is not None else torch.mean(x.to(compute))
    if axis is None and keepdims:
        r = r.reshape((1,) * x.ndim)
    return r.to(out_dtype)


def _minmax(fn_all, fn_dim, x, axis, keepdims, initial):
    x = _t(x)
    if x.numel() == 0 and initial is not None:
        shape = [1 if keepdims else None for _ in x.shape] if axis is None else None
        return torch.full((), initial, dtype=x.dtype, device=x.device)
    if axis is None:
        r = fn_all(x)
        if keepdims:
            r = r.reshape((1,) * x.ndim)
    else:
        if axis == () or axis == []:
            r = x
        else:
            r = fn_dim(x, dim=_axis(axis), keepdim=keepdims)
    if initial is not None:
        init = torch.as_tensor(initial, dtype=r.dtype, device=r.device)
        r = torch.maximum(r, init) if fn_all is torch.max else torch.minimum(r, init)
    return r


@op("numpy", also=("keras.ops.amax", "keras.ops.numpy.amax"))
def max(x, axis=None, keepdims=False, initial=None):
    return _minmax(torch.max, torch.amax, x, axis, keepdims, initial)


@op("numpy", also=("keras.ops.amin", "keras.ops.numpy.amin"))
def min(x, axis=None, keepdims=False, initial=None):
    return _minmax(torch.min, torch.amin, x, axis, keepdims, initial)


def amax(x, axis=None, keepdims=False):
    return max(x, axis=axis, keepdims=keepdims)


def amin(x, axis=None, keepdims=False):
    return min(x, axis=axis, keepdims=keepdims)


@op("numpy")
def ptp(x, axis=None, keepdims=False):
    x = _t(x)
    return _minmax(torch.max, torch.amax, x, axis, keepdims, None) - _minmax(torch.min, torch.amin, x, axis, keepdims, None)


@op("numpy")
def all(x, axis=None, keepdims=False):
    x = _t(x).to(torch.bool)
    if axis is None:
        r = torch.all(x)
        return r.reshape((1,) * x.ndim) if keepdims else r
    if not isinstance(axis, (list, tuple)):
        axis = (axis,)
    for a in sorted([a % x.ndim for a in axis], reverse=True):
        x = torch.all(x, dim=a, keepdim=keepdims)
    return x


@op("numpy")
def any(x, axis=None, keepdims=False):
    x = _t(x).to(torch.bool)
    if axis is None:
        r = torch.any(x)
        return r.reshape((1,) * x.ndim) if keepdims else r
    if not isinstance(axis, (list, tuple)):
        axis = (axis,)
    for a in sorted([a % x.ndim for a in axis], reverse=True):
        x = torch.any(x, dim=a, keepdim=keepdims)
    return x


def _var_like(fn, x, axis, keepdims):
    x = _t(x)
    ori = x.dtype
    if ori in _FLOATS:
        compute, out = (torch.float32 if ori in (torch.float16, torch.bfloat16) else ori), ori
    else:
        compute = out = to_torch_dtype(config.floatx())
    xc = x.to(compute)
    if axis is None:
        r = fn(xc, correction=0)
        if keepdims:
            r = r.reshape((1,) * x.ndim)
    else:
        r = fn(xc, dim=_axis(axis), correction=0, keepdim=keepdims)
    return r.to(out)


@op("numpy")
def var(x, axis=None, keepdims=False):
    x = _t(x)
    return _var_like(torch.var, x.to(torch.float32) if x.dtype == torch.float64 else x, axis, keepdims)


@op("numpy")
def std(x, axis=None, keepdims=False):
    return _var_like(torch.std, x, axis, keepdims)


@op("numpy")
def argmax(x, axis=None, keepdims=False):
    x = _t(x)
    if x.dtype == torch.bool:
        x = x.to(torch.uint8)
    return torch.argmax(x, dim=axis, keepdim=keepdims).to(torch.int32)


@op("numpy")
def argmin(x, axis=None, keepdims=False):
    x = _t(x)
    if x.dtype == torch.bool:
        x = x.to(torch.uint8)
    return torch.argmin(x, dim=axis, keepdim=keepdims).to(torch.int32)


@op("numpy")
def count_nonzero(x, axis=None):
    x = _t(x)
    if axis == () or axis == []:
        return (x != 0).to(torch.int32)
    return torch.count_nonzero(x, dim=_axis(axis)).to(torch.int32)


@op("numpy")
def cumsum(x, axis=None, dtype=None):
    x = _t(x)
    if axis is None:
        x, axis = x.flatten(), 0
    d = to_torch_dtype(result_type(dtype if dtype is not None else _dt(x)))  # 64-bit narrows, as result_type says
    d = torch.int32 if d == torch.bool else d
    return torch.cumsum(x, dim=axis, dtype=d)


@op("numpy")
def cumprod(x, axis=None, dtype=None):
    x = _t(x)
    if axis is None:
        x, axis = x.flatten(), 0
    d = to_torch_dtype(result_type(dtype if dtype is not None else _dt(x)))
    d = torch.int32 if d == torch.bool else d
    return torch.cumprod(x, dim=axis, dtype=d)


@op("numpy")
def average(x, axis=None, weights=None):
    x = _t(x)
    dts = [x.dtype, float]
    if weights is not None:
        weights = _t(weights)
        dts.append(weights.dtype)
    d = to_torch_dtype(result_type(*dts))
    x = x.to(d)
    if weights is None:
        return torch.mean(x, dim=_axis(axis)) if axis is not None else torch.mean(x)
    weights = weights.to(d)
    if weights.shape != x.shape and axis is not None and weights.ndim == 1:
        shape = [1] * x.ndim
        shape[axis] = -1
        weights = weights.reshape(shape)
    if axis is None:
        return torch.sum(x * weights) / torch.sum(weights)
    return torch.sum(x * weights, dim=_axis(axis)) / torch.sum(weights.expand_as(x) if weights.ndim == x.ndim else weights, dim=_axis(axis))


@op("numpy")
def median(x, axis=None, keepdims=False):
    return quantile(x, 0.5, axis=axis, keepdims=keepdims)


@op("numpy")
def quantile(x, q, axis=None, method="linear", keepdims=False):
    x = _t(x)
    ori = to_torch_dtype(result_type(_dt(x), float))  # float64 narrows to float32 here, as in the reference
    compute = torch.float32 if ori in (torch.float16, torch.bfloat16) else ori
    xq = x.to(compute)
    qt = _t(q).to(compute)
    if axis is None:
        y = xq.flatten()
        r = torch.quantile(y, qt, dim=0, interpolation=method)
        if keepdims:
            r = r.reshape(tuple(qt.shape) + (1,) * x.ndim)
        return r.to(ori)
    if isinstance(axis, (list, tuple)):
        axes = sorted(a % x.ndim for a in axis)
        keep = [i for i in range(x.ndim) if i not in axes]
        y = xq.permute(keep + axes).reshape([x.shape[i] for i in keep] + [-1])
        r = torch.quantile(y, qt, dim=-1, interpolation=method)
        if keepdims:
            shape = [1 if i in axes else x.shape[i] for i in range(x.ndim)]
            r = r.reshape(tuple(qt.shape) + tuple(shape))
        return r.to(ori)
    return torch.quantile(xq, qt, dim=axis, keepdim=keepdims, interpolation=method).to(ori)


@op("numpy")
def percentile(x, q, axis=None, method="linear", keepdims=False):
    return quantile(x, _t(q).to(torch.float32) / 100.0 if not isinstance(q, (int, float)) else q / 100.0, axis=axis, method=method, keepdims=keepdims)


def _nan_reduce(name, body):
    body.__name__ = name
    globals()[name] = op("numpy")(body)


@op("numpy")
def nansum(x, axis=None, keepdims=False):
    x = _promote_sum_dtype(_t(x))
    if axis is None:
        r = torch.nansum(x, dtype=x.dtype)
        return r.reshape((1,) * x.ndim) if keepdims else r
    return torch.nansum(x, dim=_axis(axis), keepdim=keepdims, dtype=x.dtype)


@op("numpy")
def nanmean(x, axis=None, keepdims=False):
    x = _floatize(x)
    compute = torch.float32 if x.dtype in (torch.float16, torch.bfloat16) else x.dtype
    if axis is None:
        r = torch.nanmean(x.to(compute))
        r = r.reshape((1,) * x.ndim) if keepdims else r
    else:
        r = torch.nanmean(x.to(compute), dim=_axis(axis), keepdim=keepdims)
    return r.to(x.dtype)


@op("numpy")
def nanprod(x, axis=None, keepdims=False):
    x = _t(x)
    if x.dtype in _FLOATS:
        x = torch.where(torch.isnan(x), torch.ones((), dtype=x.dtype, device=x.device), x)
    return prod(x, axis=axis, keepdims=keepdims)


@op("numpy")
def nanmax(x, axis=None, keepdims=False):
    x = _t(x)
    if x.dtype in _FLOATS:
        allnan = all(torch.isnan(x), axis=axis, keepdims=keepdims)
        y = torch.where(torch.isnan(x), torch.full((), -math.inf, dtype=x.dtype, device=x.device), x)
        r = max(y, axis=axis, keepdims=keepdims)
        return torch.where(allnan, torch.full((), math.nan, dtype=x.dtype, device=x.device), r)
    return max(x, axis=axis, keepdims=keepdims)


@op("numpy")
def nanmin(x, axis=None, keepdims=False):
    x = _t(x)
    if x.dtype in _FLOATS:
        allnan = all(torch.isnan(x), axis=axis, keepdims=keepdims)
        y = torch.where(torch.isnan(x), torch.full((), math.inf, dtype=x.dtype, device=x.device), x)
        r = min(y, axis=axis, keepdims=keepdims)
        return torch.where(allnan, torch.full((), math.nan, dtype=x.dtype, device=x.device), r)
    return min(x, axis=axis, keepdims=keepdims)


@op("numpy")
def nanvar(x, axis=None, keepdims=False):
    x = _floatize(x)
    compute = torch.float32 if x.dtype in (torch.float16, torch.bfloat16) else x.dtype
    xc = x.to(compute)
    m = nanmean(xc, axis=axis, keepdims=True)
    sq = torch.where(torch.isnan(xc), torch.full((), math.nan, dtype=compute, device=x.device), (xc - m) ** 2)
    return nanmean(sq, axis=axis, keepdims=keepdims).to(x.dtype)


@op("numpy")
def nanstd(x, axis=None, keepdims=False):
    return torch.sqrt(nanvar(x, axis=axis, keepdims=keepdims))


@op("numpy")
def nanargmax(x, axis=None, keepdims=False):
    x = _t(x)
    if x.dtype in _FLOATS:
        x = torch.where(torch.isnan(x), torch.full((), -math.inf, dtype=x.dtype, device=x.device), x)
    return argmax(x, axis=axis, keepdims=keepdims)


@op("numpy")
def nanargmin(x, axis=None, keepdims=False):
    x = _t(x)
    if x.dtype in _FLOATS:
        x = torch.where(torch.isnan(x), torch.full((), math.inf, dtype=x.dtype, device=x.device), x)
    return argmin(x, axis=axis, keepdims=keepdims)


@op("numpy")
def nancumsum(x, axis=None, dtype=None):
    x = _t(x)
    if x.dtype in _FLOATS:
        x = torch.nan_to_num(x, nan=0.0, posinf=math.inf, neginf=-math.inf)
    return cumsum(x, axis=axis, dtype=dtype)


@op("numpy")
def nancumprod(x, axis=None, dtype=None):
    x = _t(x)
    if x.dtype in _FLOATS:
        x = torch.where(torch.isnan(x), torch.ones((), dtype=x.dtype, device=x.device), x)
    return cumprod(x, axis=axis, dtype=dtype)


@op("numpy")
def nanmedian(x, axis=None, keepdims=False):
    return nanquantile(x, 0.5, axis=axis, keepdims=keepdims)


@op("numpy")
def nanquantile(x, q, axis=None, method="linear", keepdims=False):
    x = _floatize(x)
    ori = x.dtype
    compute = torch.float32 if ori in (torch.float16, torch.bfloat16) else ori
    xq = x.to(compute)
    qt = _t(q).to(compute)
    if axis is None:
        r = torch.nanquantile(xq.flatten(), qt, dim=0, interpolation=method)
        if keepdims:
            r = r.reshape(tuple(qt.shape) + (1,) * x.ndim)
        return r.to(ori)
    if isinstance(axis, (list, tuple)):
        axes = sorted(a % x.ndim for a in axis)
        keep = [i for i in range(x.ndim) if i not in axes]
        y = xq.permute(keep + axes).reshape([x.shape[i] for i in keep] + [-1])
        r = torch.nanquantile(y, qt, dim=-1, interpolation=method)
        if keepdims:
            r = r.reshape(tuple(qt.shape) + tuple(1 if i in axes else x.shape[i] for i in range(x.ndim)))
        return r.to(ori)
    return torch.nanquantile(xq, qt, dim=axis, keepdim=keepdims, interpolation=method).to(ori)


@op("numpy")
def nanpercentile(x, q, axis=None, method="linear", keepdims=False):
    qq = q / 100.0 if isinstance(q, (int, float)) else _t(q).to(torch.float32) / 100.0
    return nanquantile(x, qq, axis=axis, method=method, keepdims=keepdims)


# --- linear algebra-ish -------------------------------------------------------------------

@op("numpy")
def matmul(x1, x2):
    x1, x2 = _t(x1), _t(x2)
    if x1.dtype == torch.int8 and x2.dtype == torch.int8:
        # int8 x int8 accumulates in int32 (keras/src/backend/torch/numpy.py:101-160).
        if x1.is_cuda and x1.ndim == 2 and x2.ndim == 2 and x1.shape[0] > 16 and x1.shape[1] % 8 == 0 and x2.shape[1] % 8 == 0 and x1.shape[0] % 8 == 0:
            return torch._int_mm(x1, x2)
        if x1.is_cuda:
            return torch.matmul(x1.to(torch.float32), x2.to(torch.float32)).to(torch.int32)
        return torch.matmul(x1.to(torch.int32), x2.to(torch.int32))
    if x1.dtype != x2.dtype or x1.dtype in (torch.int64, torch.float64):
        d = to_torch_dtype(result_type(x1.dtype, x2.dtype))  # also narrows a pair of 64-bit operands, as the reference does
        x1, x2 = x1.to(d), x2.to(d)
    if x1.dtype == torch.bool:
        # computed in floatx and cast back to bool (keras/src/backend/torch/numpy.py matmul)
        f = to_torch_dtype(config.floatx())
        return torch.matmul(x1.to(f), x2.to(f)).to(torch.bool)
    from keras_b200.kernels import dispatch

    out = dispatch.matmul(x1, x2)
    if out is not None:
        return out
    return torch.matmul(x1, x2)


def _float_product(x1, x2, body):
    """dot / inner / vdot: operands promoted by ``result_type``, the product formed in a float type and cast back to that
    dtype (keras/src/backend/torch/numpy.py dot, inner, vdot: integer and bool operands give integer and bool results)."""
    x1, x2 = _pair_converted(x1, x2)
    out = x1.dtype
    compute = to_torch_dtype(result_type(_dt(x1), float))
    if compute == torch.float16 and not x1.is_cuda:
        compute = torch.float32
    r = body(x1.to(compute), x2.to(compute))
    return r if r.dtype == out else r.to(out)


@op("numpy")
def dot(x1, x2):
    def body(a, b):
        if a.ndim == 0 or b.ndim == 0:
            return a * b
        if b.ndim <= 2:
            return torch.matmul(a, b)
        return torch.tensordot(a, b, dims=([-1], [-2]))

    return _float_product(x1, x2, body)


@op("numpy")
def vdot(x1, x2):
    return _float_product(x1, x2, lambda a, b: torch.vdot(a.flatten(), b.flatten()))


@op("numpy")
def inner(x1, x2):
    return _float_product(x1, x2, torch.inner)


@op("numpy")
def outer(x1, x2):
    x1, x2 = _pair_full(x1, x2)
    return torch.outer(x1.flatten(), x2.flatten())


@op("numpy")
def tensordot(x1, x2, axes=2):
    x1, x2 = _pair_converted(x1, x2)
    if isinstance(axes, (list, tuple)):
        a, b = axes
        a = [a] if isinstance(a, int) else list(a)
        b = [b] if isinstance(b, int) else list(b)
        return torch.tensordot(x1, x2, dims=(a, b))
    return torch.tensordot(x1, x2, dims=axes)


@op("numpy")
def einsum(subscripts, *operands, **kwargs):
    ts = [_t(o) for o in operands]
    dts = {t.dtype for t in ts}
    if len(dts) > 1:
        d = to_torch_dtype(result_type(*[t.dtype for t in ts]))
        ts = [t.to(d) for t in ts]
    elif ts and ts[0].dtype == torch.int8:
        if ts[0].is_cuda:
            return torch.einsum(subscripts, *[t.to(torch.float32) for t in ts]).to(torch.int32)
        ts = [t.to(torch.int32) for t in ts]
    return torch.einsum(subscripts, *ts)


@op("numpy")
def kron(x1, x2):
    x1, x2 = _pair_full(x1, x2)
    return torch.kron(x1, x2)


@op("numpy")
def cross(x1, x2, axisa=-1, axisb=-1, axisc=-1, axis=None):
    x1, x2 = _pair_converted(x1, x2)
    if axis is not None:
        axisa = axisb = axisc = axis
    a = torch.movedim(x1, axisa, -1)
    b = torch.movedim(x2, axisb, -1)
    if a.shape[-1] == 2 and b.shape[-1] == 2:
        return a[..., 0] * b[..., 1] - a[..., 1] * b[..., 0]
    if a.shape[-1] == 2:
        a = torch.cat([a, torch.zeros_like(a[..., :1])], -1)
    if b.shape[-1] == 2:
        b = torch.cat([b, torch.zeros_like(b[..., :1])], -1)
    return torch.movedim(torch.linalg.cross(a, b, dim=-1), -1, axisc)


@op("numpy")
def trace(x, offset=0, axis1=0, axis2=1):
    x = _t(x)
    if x.dtype in (torch.int8, torch.int16, torch.uint8, torch.bool):
        x = x.to(torch.int32)
    return torch.sum(torch.diagonal(x, offset, axis1, axis2), dim=-1, dtype=x.dtype)


@op("numpy")
def diagonal(x, offset=0, axis1=0, axis2=1):
    return torch.diagonal(_t(x), offset=offset, dim1=axis1, dim2=axis2)


@op("numpy")
def diag(x, k=0):
    return torch.diag(_t(x), diagonal=k)


@op("numpy")
def diagflat(x, k=0):
    return torch.diagflat(_t(x), offset=k)


@op("numpy")
def tril(x, k=0):
    return torch.tril(_t(x), diagonal=k)


@op("numpy")
def triu(x, k=0):
    return torch.triu(_t(x), diagonal=k)


@op("numpy")
def slogdet(x):
    r = torch.linalg.slogdet(_floatize(x))
    return r.sign, r.logabsdet


@op("numpy")
def correlate(x1, x2, mode="valid"):
    x1, x2 = _pair_float(x1, x2)
    n, m = x1.shape[0], x2.shape[0]
    if mode == "full":
        pad = (m - 1, m - 1)
    elif mode == "same":
        total = m - 1
        pad = (total // 2, total - total // 2) if n >= m else (total // 2, total - total // 2)
    else:
        pad = (0, 0)
    if mode == "valid" and m > n:
        x1, x2 = x2, x1
        flip = True
    else:
        flip = False
    xi = torch.nn.functional.pad(x1[None, None], pad)
    out = torch.nn.functional.conv1d(xi.to(torch.float32) if x1.dtype in (torch.float16, torch.bfloat16) and not x1.is_cuda else xi, x2[None, None].to(xi.dtype))[0, 0]
    if mode == "same":
        out = out[: builtins.max(n, m)]
    if flip:
        out = out.flip(0)
    return out.to(x1.dtype)


@op("numpy")
def corrcoef(x):
    return torch.corrcoef(_floatize(x))


@op("numpy")
def vander(x, N=None, increasing=False):
    x = _t(x)
    d = x.dtype if x.dtype != torch.bool else torch.int32
    return torch.vander(x.to(d), N=N, increasing=increasing)


# --- creation -----------------------------------------------------------------------------

def _cdt(dtype):
    return to_torch_dtype(dtype if dtype is not None else config.floatx())


@op("numpy")
def zeros(shape, dtype=None):
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    return torch.zeros(shape, dtype=_cdt(dtype), device=get_device())


@op("numpy")
def ones(shape, dtype=None):
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    return torch.ones(shape, dtype=_cdt(dtype), device=get_device())


@op("numpy")
def empty(shape, dtype=None):
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    return torch.empty(shape, dtype=_cdt(dtype), device=get_device())


@op("numpy")
def full(shape, fill_value, dtype=None):
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    if isinstance(fill_value, (_T, np.ndarray, Variable)):
        fv = _t(fill_value)
        d = to_torch_dtype(dtype if dtype is not None else config.floatx())  # no dtype: floatx here too, not the array's type
        return torch.broadcast_to(fv.to(d), shape).clone()
    d = to_torch_dtype(dtype if dtype is not None else config.floatx())  # no dtype: floatx, whatever the scalar's type
    return torch.full(shape, fill_value, dtype=d, device=get_device())


@op("numpy")
def zeros_like(x, dtype=None):
    x = _t(x)
    return torch.zeros_like(x, dtype=to_torch_dtype(dtype) if dtype is not None else None)


@op("numpy")
def ones_like(x, dtype=None):
    x = _t(x)
    return torch.ones_like(x, dtype=to_torch_dtype(dtype) if dtype is not None else None)


@op("numpy")
def empty_like(x, dtype=None):
    x = _t(x)
    return torch.empty_like(x, dtype=to_torch_dtype(dtype) if dtype is not None else None)


@op("numpy")
def full_like(x, fill_value, dtype=None):
    x = _t(x)
    d = to_torch_dtype(dtype) if dtype is not None else x.dtype
    if isinstance(fill_value, (_T, np.ndarray, Variable)):
        return torch.broadcast_to(_t(fill_value).to(d), x.shape).clone()
    return torch.full_like(x, fill_value, dtype=d)


@op("numpy")
def eye(N, M=None, k=0, dtype=None):
    M = N if M is None else M
    d = _cdt(dtype)
    if k == 0:
        return torch.eye(N, M, dtype=d, device=get_device())
    out = torch.zeros((N, M), dtype=d, device=get_device())
    diag_len = builtins.max(0, builtins.min(N, M - k) if k >= 0 else builtins.min(N + k, M))
    if diag_len > 0:
        idx = torch.arange(diag_len, device=get_device())
        rows = idx if k >= 0 else idx - k
        cols = idx + k if k >= 0 else idx
        out[rows, cols] = 1
    return out


@op("numpy")
def identity(n, dtype=None):
    return torch.eye(n, dtype=_cdt(dtype), device=get_device())


@op("numpy")
def tri(N, M=None, k=0, dtype=None):
    M = N if M is None else M
    return torch.tril(torch.ones((N, M), dtype=_cdt(dtype), device=get_device()), diagonal=k)


@op("numpy")
def arange(start, stop=None, step=None, dtype=None):
    if dtype is None:
        parts = [start] + ([stop] if stop is not None else []) + ([step] if step is not None else [])
        d = result_type(*[_dt(p) for p in parts])
        if builtins.all(isinstance(p, int) for p in parts):
            d = "int32"
        dtype = d
    td = to_torch_dtype(dtype)
    conv = lambda v: v.item() if isinstance(v, _T) else v
    start, stop, step = conv(start), (conv(stop) if stop is not None else None), (conv(step) if step is not None else 1)
    if stop is None:
        return torch.arange(start, dtype=td, device=get_device())
    return torch.arange(start, stop, step, dtype=td, device=get_device())


@op("numpy")
def linspace(start, stop, num=50, endpoint=True, retstep=False, dtype=None, axis=0):
    if dtype is None:
        dtype = result_type(_dt(start), _dt(stop), float)
    td = to_torch_dtype(dtype)
    compute = torch.float32 if td in (torch.float16, torch.bfloat16) or td not in _FLOATS else td
    s, e = _t(start).to(compute), _t(stop).to(compute)
    div = (num - 1) if endpoint else num
    step = (e - s) / div if div > 0 else torch.full_like(e - s, math.nan)
    idx = torch.arange(num, dtype=compute, device=s.device).reshape((-1,) + (1,) * builtins.max(s.ndim, e.ndim))
    out = s + idx * step if div > 0 else s + idx * 0
    if endpoint and num > 1:
        out[-1] = torch.broadcast_to(e, out[-1].shape)
    if axis != 0:
        out = torch.movedim(out, 0, axis)
    out = out.to(td) if td in _FLOATS else torch.floor(out).to(td)
    return (out, step) if retstep else out


@op("numpy")
def logspace(start, stop, num=50, endpoint=True, base=10, dtype=None, axis=0):
    if dtype is None:
        dtype = result_type(_dt(start), _dt(stop), float)
    y = linspace(start, stop, num=num, endpoint=endpoint, dtype="float32" if dtype != "float64" else dtype, axis=axis)
    return torch.pow(_t(base).to(y.dtype), y).to(to_torch_dtype(dtype))


@op("numpy")
def geomspace(start, stop, num=50, endpoint=True, dtype=None, axis=0):
    if dtype is None:
        dtype = result_type(_dt(start), _dt(stop), float)
    s, e = _t(start).to(torch.float64), _t(stop).to(torch.float64)
    sign = torch.sign(s)
    y = linspace(torch.log(torch.abs(s)), torch.log(torch.abs(e)), num=num, endpoint=endpoint, dtype="float64", axis=axis)
    return (torch.exp(y) * sign).to(to_torch_dtype(dtype))


@op("numpy")
def array(x, dtype=None):
    return convert_to_tensor(x, dtype=dtype)


@op("numpy")
def copy(x):
    return _t(x).clone()


@op("numpy")
def meshgrid(*x, indexing="xy"):
    return tuple(torch.meshgrid(*[_t(e) for e in x], indexing=indexing))


def _window(fn, x, **kw):
    n = int(x.item()) if isinstance(x, _T) else int(x)
    return fn(n, periodic=False, dtype=to_torch_dtype(config.floatx()), device=get_device(), **kw)


@op("numpy")
def bartlett(x):
    return _window(torch.bartlett_window, x)


@op("numpy")
def blackman(x):
    return _window(torch.blackman_window, x)


@op("numpy")
def hamming(x):
    return _window(torch.hamming_window, x)


@op("numpy")
def hanning(x):
    return _window(torch.hann_window, x)


@op("numpy")
def kaiser(x, beta):
    return _window(torch.kaiser_window, x, beta=float(beta))


# --- shape manipulation -------------------------------------------------------------------

@op("numpy")
def reshape(x, newshape):
    if not isinstance(newshape, (list, tuple)):
        newshape = (newshape,)
    return torch.reshape(_t(x), tuple(int(d) for d in newshape))


@op("numpy")
def transpose(x, axes=None):
    x = _t(x)
    if axes is None:
        return x.permute(*reversed(range(x.ndim)))
    return x.permute(*axes)


@op("numpy")
def swapaxes(x, axis1, axis2):
    return torch.swapaxes(_t(x), axis1, axis2)


@op("numpy")
def moveaxis(x, source, destination):
    return torch.moveaxis(_t(x), source, destination)


@op("numpy")
def expand_dims(x, axis):
    x = _t(x)
    if isinstance(axis, (list, tuple)):
        out_ndim = x.ndim + len(axis)
        for a in sorted(a % out_ndim for a in axis):
            x = torch.unsqueeze(x, a)
        return x
    return torch.unsqueeze(x, axis)


@op("numpy")
def squeeze(x, axis=None):
    x = _t(x)
    if axis is None:
        return torch.squeeze(x)
    axes = (axis,) if isinstance(axis, int) else tuple(axis)
    return torch.squeeze(x, dim=axes)  # an axis whose extent is not 1 is left alone (eager torch semantics)


@op("numpy")
def ravel(x):
    return torch.ravel(_t(x))


@op("numpy")
def flip(x, axis=None):
    x = _t(x)
    if axis is None:
        axis = tuple(range(x.ndim))
    return torch.flip(x, dims=(axis,) if isinstance(axis, int) else tuple(axis))


@op("numpy")
def fliplr(x):
    return torch.fliplr(_t(x))


@op("numpy")
def flipud(x):
    return torch.flipud(_t(x))


@op("numpy")
def rot90(array, k=1, axes=(0, 1)):
    array = _t(array)
    if array.ndim < 2:
        raise ValueError(f"Input array must have at least 2 dimensions. Received: array.ndim={array.ndim}")
    if len(axes) != 2 or axes[0] == axes[1]:
        raise ValueError(f"Invalid axes: {axes}. Axes must be a tuple of two different dimensions.")
    return torch.rot90(array, k=k, dims=tuple(a % array.ndim for a in axes))


@op("numpy")
def roll(x, shift, axis=None):
    return torch.roll(_t(x), shift, axis)


@op("numpy")
def broadcast_to(x, shape):
    return torch.broadcast_to(_t(x), tuple(shape))


def _seq(xs):
    ts = [_t(x) for x in xs]
    if len({t.dtype for t in ts}) > 1:
        d = to_torch_dtype(result_type(*[t.dtype for t in ts]))
        ts = [t.to(d) for t in ts]
    return ts


@op("numpy")
def concatenate(xs, axis=0):
    return torch.cat(_seq(xs), dim=axis)


@op("numpy")
def stack(x, axis=0):
    return torch.stack(_seq(x), dim=axis)


@op("numpy")
def hstack(xs):
    return torch.hstack(_seq(xs))


@op("numpy")
def vstack(xs):
    return torch.vstack(_seq(xs))


@op("numpy")
def dstack(xs):
    return torch.dstack(_seq(xs))


@op("numpy")
def column_stack(xs):
    return torch.column_stack(_seq(xs))


@op("numpy")
def append(x1, x2, axis=None):
    x1, x2 = _pair_full(x1, x2)
    if axis is None:
        return torch.cat([x1.flatten(), x2.flatten()])
    return torch.cat([x1, x2], dim=axis)


def _split_sizes(n, spec):
    if isinstance(spec, int):
        if n % spec != 0:
            raise ValueError(f"Split does not result in an equal division. Received: dim={n}, indices_or_sections={spec}")
        return [n // spec] * spec
    idx = [int(i) for i in (spec.tolist() if isinstance(spec, (_T, np.ndarray)) else spec)]
    bounds = [0] + [builtins.min(builtins.max(i, 0), n) for i in idx] + [n]
    return [builtins.max(bounds[i + 1] - bounds[i], 0) for i in range(len(bounds) - 1)]


@op("numpy")
def split(x, indices_or_sections, axis=0):
    x = _t(x)
    return list(torch.split(x, _split_sizes(x.shape[axis], indices_or_sections), dim=axis))


@op("numpy")
def array_split(x, indices_or_sections, axis=0):
    x = _t(x)
    if isinstance(indices_or_sections, int):
        return list(torch.tensor_split(x, indices_or_sections, dim=axis))
    return split(x, indices_or_sections, axis=axis)


@op("numpy")
def hsplit(x, indices_or_sections):
    x = _t(x)
    return split(x, indices_or_sections, axis=0 if x.ndim == 1 else 1)


@op("numpy")
def vsplit(x, indices_or_sections):
    return split(x, indices_or_sections, axis=0)


@op("numpy")
def dsplit(x, indices_or_sections):
    return split(x, indices_or_sections, axis=2)


@op("numpy")
def tile(x, repeats):
    x = _t(x)
    repeats = (repeats,) if isinstance(repeats, int) else tuple(int(r) for r in repeats)
    if len(repeats) < x.ndim:
        repeats = (1,) * (x.ndim - len(repeats)) + repeats
    return torch.tile(x, repeats)


@op("numpy")
def repeat(x, repeats, axis=None):
    x = _t(x)
    if isinstance(repeats, (list, tuple, np.ndarray)):
        repeats = torch.as_tensor(np.asarray(repeats), device=x.device)
    if isinstance(repeats, _T) and repeats.ndim == 0:
        repeats = int(repeats)
    return torch.repeat_interleave(x, repeats, dim=axis)


@op("numpy")
def pad(x, pad_width, mode="constant", constant_values=None):
    x = _t(x)
    if isinstance(pad_width, int):
        pad_width = [(pad_width, pad_width)] * x.ndim
    pw = [tuple(int(v) for v in (p if isinstance(p, (list, tuple)) else (p, p))) for p in (pad_width.tolist() if isinstance(pad_width, (np.ndarray, _T)) else pad_width)]
    if len(pw) == 1 and x.ndim > 1:
        pw = pw * x.ndim
    if mode != "constant" and constant_values is not None:
        raise ValueError(f"Argument `constant_values` can only be provided when `mode == 'constant'`. Received: mode={mode}")
    mode_t = {"symmetric": "replicate_sym", "wrap": "circular", "edge": "replicate"}.get(mode, mode)
    # drop leading dims with zero padding so torch's N-d limits are met
    flat = []
    for lo, hi in reversed(pw):
        flat.extend([lo, hi])
    while len(flat) > 2 and flat[-1] == 0 and flat[-2] == 0:
        flat = flat[:-2]
    if mode_t == "constant":
        cv = 0 if constant_values is None else (constant_values.item() if isinstance(constant_values, _T) else constant_values)
        if x.dtype == torch.bool:
            return torch.nn.functional.pad(x.to(torch.uint8), flat, value=int(bool(cv))).to(torch.bool)
        return torch.nn.functional.pad(x, flat, mode="constant", value=cv)
    if mode_t == "replicate_sym":
        out = x
        for d, (lo, hi) in enumerate(pw):
            if lo == 0 and hi == 0:
                continue
            n = out.shape[d]
            idx = torch.arange(-lo, n + hi, device=x.device)
            period = 2 * n
            idx = torch.remainder(idx, period)
            idx = torch.where(idx >= n, period - 1 - idx, idx)
            out = torch.index_select(out, d, idx)
        return out
    if mode_t == "reflect":
        out = x
        for d, (lo, hi) in enumerate(pw):
            if lo == 0 and hi == 0:
                continue
            n = out.shape[d]
            idx = torch.arange(-lo, n + hi, device=x.device)
            if n == 1:
                idx = torch.zeros_like(idx)
            else:
                period = 2 * (n - 1)
                idx = torch.remainder(idx, period)
                idx = torch.where(idx >= n, period - idx, idx)
            out = torch.index_select(out, d, idx)
        return out
    if mode_t == "circular":
        out = x
        for d, (lo, hi) in enumerate(pw):
            if lo == 0 and hi == 0:
                continue
            n = out.shape[d]
            idx = torch.remainder(torch.arange(-lo, n + hi, device=x.device), n)
            out = torch.index_select(out, d, idx)
        return out
    if mode_t == "replicate":
        out = x
        for d, (lo, hi) in enumerate(pw):
            if lo == 0 and hi == 0:
                continue
            n = out.shape[d]
            idx = torch.clamp(torch.arange(-lo, n + hi, device=x.device), 0, n - 1)
            out = torch.index_select(out, d, idx)
        return out
    raise ValueError(f"Unsupported padding mode: {mode}")


# --- indexing / sorting -------------------------------------------------------------------

@op("numpy")
def get_item(x, key):
    x = _t(x)
    if isinstance(key, tuple):
        key = tuple(_t(k).long() if isinstance(k, (list, np.ndarray)) else k for k in key)
        key = tuple(k.long() if isinstance(k, _T) and k.dtype in (torch.int32, torch.int16, torch.int8, torch.uint8) and k.dtype != torch.bool else k for k in key)
    elif isinstance(key, (list, np.ndarray)):
        key = _t(key)
    if isinstance(key, _T) and key.dtype not in (torch.bool, torch.int64):
        key = key.long()
    return x[key]


@op("numpy")
def take(x, indices, axis=None):
    x = _t(x)
    indices = _t(indices)
    if indices.dtype in _FLOATS:
        indices = indices.long()
    elif indices.dtype != torch.int64:
        indices = indices.long()
    if axis is None:
        x, axis = x.flatten(), 0
    n = x.shape[axis]
    indices = torch.where(indices < 0, indices + n, indices)
    if x.ndim == 2 and axis == 0:
        # embedding lookup: autograd-friendly gather with dense scatter-add backward
        return torch.nn.functional.embedding(indices, x)
    out = torch.index_select(x, axis, indices.reshape(-1))
    new_shape = tuple(x.shape[: axis % x.ndim]) + tuple(indices.shape) + tuple(x.shape[axis % x.ndim + 1:])
    return out.reshape(new_shape)


@op("numpy")
def take_along_axis(x, indices, axis=None):
    x = _t(x)
    indices = _t(indices).long()
    if axis is None:
        return torch.take_along_dim(x.flatten(), indices.flatten(), 0)
    n = x.shape[axis]
    indices = torch.where(indices < 0, indices + n, indices)
    return torch.take_along_dim(x, indices, dim=axis)


@op("numpy")
def where(condition, x1=None, x2=None):
    condition = _t(condition).to(torch.bool)
    if x1 is None and x2 is None:
        return torch.where(condition)
    if x1 is None or x2 is None:
        raise ValueError("`x1` and `x2` either both should be `None` or both should have non-None value.")
    x1, x2 = _pair_native(x1, x2)
    return torch.where(condition, x1, x2)


@op("numpy")
def select(condlist, choicelist, default=0):
    choices = _seq(choicelist)
    out = torch.full_like(choices[0], default) if not isinstance(default, _T) else default.to(choices[0].dtype)
    shape = torch.broadcast_shapes(*[c.shape for c in choices], *[_t(c).shape for c in condlist])
    out = torch.broadcast_to(out, shape)
    for cond, choice in reversed(list(zip(condlist, choices))):
        out = torch.where(_t(cond).to(torch.bool), choice, out)
    return out


@op("numpy")
def nonzero(x):
    return tuple(t.to(torch.int32) for t in torch.nonzero(_t(x), as_tuple=True))


@op("numpy")
def sort(x, axis=-1):
    x = _t(x)
    if x.dtype == torch.bool:
        return torch.sort(x.to(torch.uint8), dim=axis).values.to(torch.bool)
    return torch.sort(x, dim=axis, stable=True).values


@op("numpy")
def argsort(x, axis=-1):
    x = _t(x)
    if x.dtype == torch.bool:
        x = x.to(torch.uint8)
    if axis is None:
        x, axis = x.flatten(), -1
    return torch.argsort(x, dim=axis, stable=True).to(torch.int32)


@op("numpy")
def argpartition(x, kth, axis=-1):
    # Same selection steps as keras/src/backend/torch/numpy.py:2421-2452 (values are compared as int32, the remaining
    # indices come from a top-k over a 0/1 marker), so that ties and the order inside both halves agree with it.
    x = _t(x).to(torch.int32)
    if axis is None:
        x, axis, flat = x.flatten(), 0, True
    else:
        flat = False
    x = torch.transpose(x, axis, -1)
    n = x.shape[-1]
    lowest = torch.topk(-x, kth + 1).indices
    marker = torch.ones_like(x, dtype=torch.int32).scatter_(-1, lowest, 0)
    others = torch.topk(marker, n - kth - 1).indices
    out = torch.cat([lowest, others], dim=-1)
    if flat:
        return out.to(torch.int32)
    return torch.transpose(out, -1, axis).to(torch.int32)


@op("numpy")
def searchsorted(sorted_sequence, values, side="left"):
    s, v = _t(sorted_sequence), _t(values)
    if s.ndim != 1:
        raise ValueError(f"`searchsorted` only supports 1-D sorted sequences. You can use `keras.ops.vectorized_map` to extend it to N-D sequences. Received: sorted_sequence.shape={tuple(s.shape)}")
    d = to_torch_dtype(result_type(s.dtype, v.dtype))
    out = torch.searchsorted(s.to(d), v.to(d).contiguous(), side=side)
    return out.to(torch.int32) if s.shape[0] < 2**31 else out


@op("numpy")
def digitize(x, bins):
    x, bins = _t(x), _t(bins)
    d = to_torch_dtype(result_type(x.dtype, bins.dtype))
    return torch.bucketize(x.to(d), bins.to(d), right=True).to(torch.int32)


@op("numpy")
def bincount(x, weights=None, minlength=0, sparse=False):
    x = _t(x)
    w = _t(weights) if weights is not None else None
    if w is not None:
        d = to_torch_dtype(result_type(x.dtype, w.dtype))
        w = w.to(d)
    if x.ndim == 2:
        rows = [torch.bincount(x[i].long(), weights=(w[i] if w is not None else None), minlength=minlength) for i in range(x.shape[0])]
        n = builtins.max(r.shape[0] for r in rows)
        rows = [torch.nn.functional.pad(r, (0, n - r.shape[0])) for r in rows]
        out = torch.stack(rows)
    else:
        out = torch.bincount(x.long(), weights=w, minlength=minlength)
    return out.to(torch.int32) if w is None else out.to(w.dtype)


@op("numpy")
def unique(x, return_index=False, return_inverse=False, return_counts=False, axis=None, size=None, fill_value=None):
    x = _t(x)
    if axis is None:
        flat = x.flatten()
        values, inverse, counts = torch.unique(flat, return_inverse=True, return_counts=True)
        inverse = inverse.reshape(x.shape)
    else:
        values, inverse, counts = torch.unique(x, return_inverse=True, return_counts=True, dim=axis)
    outs = [values]
    if return_index:
        n = inverse.numel()
        inv_flat = inverse.flatten()
        first = torch.full((values.shape[0 if axis is None else axis],), n, dtype=torch.int64, device=x.device)
        first = first.scatter_reduce(0, inv_flat, torch.arange(n, device=x.device), reduce="amin")
        outs.append(first.to(torch.int32))
    if return_inverse:
        outs.append(inverse.to(torch.int32))
    if return_counts:
        outs.append(counts.to(torch.int32))
    if size is not None:
        def fit(t, dim=0, fv=0):
            cur = t.shape[dim]
            if cur >= size:
                return t.narrow(dim, 0, size)
            padshape = list(t.shape)
            padshape[dim] = size - cur
            return torch.cat([t, torch.full(padshape, fv, dtype=t.dtype, device=t.device)], dim=dim)

        fv = fill_value if fill_value is not None else (values.flatten()[0].item() if values.numel() else 0)
        outs[0] = fit(outs[0], 0 if axis is None else axis, fv)
        k = 1
        if return_index:
            outs[k] = fit(outs[k]); k += 1
        if return_inverse:
            k += 1
        if return_counts:
            outs[k] = fit(outs[k])
    return outs[0] if len(outs) == 1 else tuple(outs)


@op("numpy")
def isin(x1, x2, assume_unique=False, invert=False):
    x1, x2 = _pair(x1, x2)
    return torch.isin(x1, x2, assume_unique=assume_unique, invert=invert)


@op("numpy")
def isclose(x1, x2, rtol=1e-5, atol=1e-8, equal_nan=False):
    x1, x2 = _pair(x1, x2)
    if x1.dtype not in _FLOATS:
        x1, x2 = x1.to(torch.float32), x2.to(torch.float32)
    return torch.isclose(x1, x2, rtol=rtol, atol=atol, equal_nan=equal_nan)


@op("numpy")
def allclose(x1, x2, rtol=1e-5, atol=1e-8, equal_nan=False):
    return torch.all(isclose(x1, x2, rtol, atol, equal_nan))


@op("numpy")
def diff(a, n=1, axis=-1):
    return torch.diff(_t(a), n=n, dim=axis)


@op("numpy")
def trapezoid(y, x=None, dx=1.0, axis=-1):
    y = _floatize(y)
    if x is not None:
        return torch.trapezoid(y, _t(x).to(y.dtype), dim=axis)
    return torch.trapezoid(y, dx=dx, dim=axis)


@op("numpy")
def histogram(x, bins=10, range=None):
    x = _floatize(x)
    if x.ndim != 1:
        raise ValueError(f"Input tensor must be 1-dimensional. Received: input.shape={tuple(x.shape)}")
    if range is None:
        lo, hi = x.min().item(), x.max().item()
    else:
        lo, hi = range
    xc = x.cpu().to(torch.float32)
    hist, edges = torch.histogram(xc, bins=bins, range=(float(lo), float(hi)))
    return hist.to(x.dtype).to(x.device), edges.to(x.dtype).to(x.device)


@op("numpy")
def unravel_index(indices, shape):
    indices = _t(indices)
    return tuple(t.to(indices.dtype) for t in torch.unravel_index(indices.long(), tuple(shape)))


@op("numpy")
def view(x, dtype=None):
    x = _t(x)
    return x.view(to_torch_dtype(dtype if dtype is not None else config.floatx()))


@op("numpy")
def ndim(x):
    return _t(x).ndim


@op("numpy")
def size(x):
    return _t(x).numel()


def shape(x):
    return tuple(x.shape)


@op("numpy")
def vectorize(pyfunc, *, excluded=None, signature=None):
    from keras_b200.ops.core import vectorized_map

    def wrapped(*args):
        return vectorized_map(lambda a: pyfunc(*a) if isinstance(a, tuple) else pyfunc(a), args if len(args) > 1 else args[0])

    return wrapped
