"""dtype names, torch mapping and the implicit promotion rules.

Promotion reproduces the observable results of keras/src/backend/common/dtypes.py:61-324
(JAX-style: Python scalars are *weak*, 64-bit results fold to 32-bit, bf16+f16→f32, no implicit
float8 conversions) but is computed from (kind, width) rules instead of a lattice search.
"""

import functools

import numpy as np
import torch

from keras_b200.core import config
from keras_b200.core.export_registry import keras_export

BOOL_TYPES = ("bool",)
INT_TYPES = ("uint8", "uint16", "uint32", "uint64", "int8", "int16", "int32", "int64")
FLOAT_TYPES = ("bfloat16", "float16", "float32", "float64")
COMPLEX_TYPES = ("complex64", "complex128")
FLOAT8_TYPES = ("float8_e4m3fn", "float8_e5m2")
WEAK_TYPES = ("int", "float")
ALLOWED_DTYPES = (
    FLOAT_TYPES + INT_TYPES + BOOL_TYPES + ("string",) + FLOAT8_TYPES + COMPLEX_TYPES
)

TORCH_DTYPES = {
    "float16": torch.float16,
    "float32": torch.float32,
    "float64": torch.float64,
    "bfloat16": torch.bfloat16,
    "uint8": torch.uint8,
    # torch has only partial kernels for wide unsigned types: store them one size up
    # (keras/src/backend/torch/core.py:52-75 makes the same choice).
    "uint16": torch.int32,
    "uint32": torch.int64,
    "int8": torch.int8,
    "int16": torch.int16,
    "int32": torch.int32,
    "int64": torch.int64,
    "bool": torch.bool,
    "float8_e4m3fn": torch.float8_e4m3fn,
    "float8_e5m2": torch.float8_e5m2,
    "complex64": torch.complex64,
    "complex128": torch.complex128,
}
_TORCH_TO_NAME = {
    torch.float16: "float16", torch.float32: "float32", torch.float64: "float64",
    torch.bfloat16: "bfloat16", torch.uint8: "uint8", torch.int8: "int8",
    torch.int16: "int16", torch.int32: "int32", torch.int64: "int64", torch.bool: "bool",
    torch.float8_e4m3fn: "float8_e4m3fn", torch.float8_e5m2: "float8_e5m2",
    torch.complex64: "complex64", torch.complex128: "complex128",
    torch.uint16: "uint16", torch.uint32: "uint32", torch.uint64: "uint64",
}
_PY_TYPES = {bool: "bool", int: "int32", float: "float32", str: "string", complex: "complex64"}


@keras_export(["keras.backend.standardize_dtype", "keras.utils.standardize_dtype"])
def standardize_dtype(dtype):
    """Any dtype spelling (str, torch/numpy dtype, Python type, None) → canonical name."""
    if dtype is None:
        return config.floatx()
    if type(dtype) is str:
        if dtype in _ALLOWED_SET:
            return dtype
        if dtype == "int":
            return "int32"
        if dtype == "float":
            return "float32"
    name = _TORCH_TO_NAME.get(dtype)
    if name is not None:
        return name
    if dtype in _PY_TYPES:
        return _PY_TYPES[dtype]
    if hasattr(dtype, "name"):
        cand = dtype.name
    elif hasattr(dtype, "__name__"):
        cand = dtype.__name__
    else:
        cand = str(dtype)
    if cand.startswith("torch."):
        cand = cand[6:]
    if cand == "str" or cand.startswith("str") or cand.startswith("<U"):
        cand = "string"
    if cand not in _ALLOWED_SET:
        try:
            cand = np.dtype(dtype).name
        except TypeError:
            pass
    if cand not in _ALLOWED_SET:
        raise ValueError(f"Invalid dtype: {dtype}")
    return cand


_ALLOWED_SET = frozenset(ALLOWED_DTYPES)


def to_torch_dtype(dtype):
    if isinstance(dtype, torch.dtype):
        return dtype
    name = standardize_dtype(dtype)
    if name == "string":
        raise ValueError("String tensors are not representable as torch tensors.")
    return TORCH_DTYPES[name]


def is_float(dtype):
    name = standardize_dtype(dtype)
    return name.startswith("float") or name == "bfloat16"


def is_int(dtype):
    name = standardize_dtype(dtype)
    return name.startswith("int") or name.startswith("uint")


# --- promotion ---------------------------------------------------------------------------

def _describe(name):
    """name → (kind, bits, weak). kinds: b < u < i < f < c."""
    if name == "bool":
        return ("b", 1, False)
    if name == "int":
        return ("i", 0, True)
    if name == "float":
        return ("f", 0, True)
    if name == "bfloat16":
        return ("f", 16, False)
    if name.startswith("uint"):
        return ("u", int(name[4:]), False)
    if name.startswith("int"):
        return ("i", int(name[3:]), False)
    if name.startswith("float"):
        return ("f", int(name[5:]), False)
    if name.startswith("complex"):
        return ("c", int(name[7:]), False)
    raise ValueError(f"dtype={name!r} is not a valid dtype for type promotion.")


def _join(a, b):
    """Least common type of two names (may return a weak name)."""
    if a == b:
        return a
    ka, wa, weak_a = _describe(a)
    kb, wb, weak_b = _describe(b)
    order = "buifc"
    if order.index(ka) > order.index(kb):
        a, b, ka, kb, wa, wb, weak_a, weak_b = b, a, kb, ka, wb, wa, weak_b, weak_a
    # now kind(a) <= kind(b)
    if ka == "b":
        return b
    if kb == "c":
        if ka == "c":
            return "complex128" if max(wa, wb) == 128 else "complex64"
        if ka == "f" and wa == 64:
            return "complex128"
        if ka in "ui" and wa == 64 and not weak_a:
            # 64-bit integers reach complex through weak float → complex64
            return b
        return b
    if kb == "f":
        if ka == "f":
            if weak_a:
                return b
            if weak_b:
                return a
            if wa == wb:  # bfloat16 vs float16
                return "float32"
            return a if wa > wb else b
        # integer (weak or not) with float: the float wins, weakness kept
        return b
    # both integer kinds
    if weak_a and weak_b:
        return "int"
    if weak_a:
        return b
    if weak_b:
        return a
    if ka == kb:
        return a if wa > wb else b
    # unsigned a with signed b
    if wa < wb:
        return b
    need = wa * 2
    if need > 64:
        return "float"  # uint64 with a signed type: only a (weak) float holds both
    return f"int{need}"


_FOLD_64 = {"int64": "int32", "uint64": "uint32", "float64": "float32", "complex128": "complex64"}


@functools.lru_cache(maxsize=4096)
def _result_type_cached(floatx, entries):
    names = []
    for dtype, weak in entries:
        if weak and dtype != "bool":
            k = _describe(dtype)[0]
            dtype = {"f": "float", "i": "int", "u": "int", "c": "complex"}.get(k, dtype)
        names.append(dtype)
    if len(entries) > 1 and len({d for d, _ in entries}) == 1 and not all(w for _, w in entries):
        out = entries[0][0]
    elif all(w for _, w in entries):
        strong = [d for d, _ in entries]
        out = functools.reduce(_join, strong)
        k = _describe(out)[0]
        if out != "bool":
            out = {"f": "float", "i": "int", "u": "int"}.get(k, out)
    else:
        out = functools.reduce(_join, names)
    if out in WEAK_TYPES:
        bits = floatx[-2:]
        out = f"int{bits}" if out == "int" else f"float{bits}"
    return _FOLD_64.get(out, out)


@keras_export("keras.backend.result_type")
def result_type(*dtypes):
    """Result dtype of combining the given dtypes / Python scalar types."""
    if not dtypes:
        return config.floatx()
    entries = []
    for d in dtypes:
        if d is None:
            d = config.floatx()
        weak = d is int or d is float
        name = standardize_dtype(d)
        if name in FLOAT8_TYPES and len(dtypes) > 1:
            raise ValueError(
                "There is no implicit conversions from float8 dtypes to others. "
                f"You must cast it internally. Received: {dtypes}"
            )
        entries.append((name, weak))
    return _result_type_cached(config.floatx(), tuple(entries))
