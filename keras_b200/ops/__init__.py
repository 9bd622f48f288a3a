"""``keras.ops``: the public op namespace."""

from keras_b200.ops import core, einops, image, linalg, math, nn, numpy  # noqa: F401
from keras_b200.ops.core import *  # noqa: F401,F403
from keras_b200.ops.core import (
    associative_scan, cast, cond, convert_to_numpy, convert_to_tensor, custom_gradient, dtype,
    fori_loop, is_tensor, map, saturate_cast, scan, scatter, scatter_update, shape, slice,
    slice_update, stop_gradient, switch, unstack, vectorized_map, while_loop,
)
from keras_b200.ops.einops import rearrange
from keras_b200.ops.function import Function  # noqa: F401
from keras_b200.ops.operation import Operation  # noqa: F401


def _reexport(module, skip=()):
    g = globals()
    for name in dir(module):
        if name.startswith("_") or name in skip:
            continue
        obj = getattr(module, name)
        if callable(obj) and getattr(obj, "_op_class", None) is not None:
            g[name] = obj


_reexport(numpy, skip=("shape",))
_reexport(nn)
_reexport(math)
_reexport(linalg)
_reexport(image)
from keras_b200.ops.linalg import jvp  # noqa: E402,F401
from keras_b200.ops.numpy import amax, amin, vectorize  # noqa: E402,F401
