"""Tensor runtime: device policy, conversion, casting, shape inference on the meta device.

The compute layer is PyTorch.  Reference behaviour: keras/src/backend/torch/core.py:31-107
(device policy), :198-285 (conversion), :318-392 (``compute_output_spec``).
"""

import contextlib
import os

import numpy as np
import torch

from keras_b200.core import config, global_state
from keras_b200.core.dtypes import TORCH_DTYPES, result_type, standardize_dtype, to_torch_dtype
from keras_b200.core.export_registry import keras_export

IS_THREAD_SAFE = True
SUPPORTS_SPARSE_TENSORS = False
SUPPORTS_RAGGED_TENSORS = False

if "KERAS_TORCH_DEVICE" in os.environ:
    _DEFAULT_DEVICE = os.environ["KERAS_TORCH_DEVICE"]
elif torch.cuda.is_available():
    _DEFAULT_DEVICE = "cuda"
else:
    _DEFAULT_DEVICE = "cpu"


def _parse_device(name):
    if isinstance(name, torch.device):
        return name
    name = str(name).lower()
    if name.startswith("gpu"):
        name = "cuda" + name[3:]
    return torch.device(name)


def get_device():
    dev = global_state.get_global_attribute("torch_device")
    if dev is None:
        if _DEFAULT_DEVICE == "cuda":
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device(_DEFAULT_DEVICE)
    return dev


def set_default_device(name):
    global _DEFAULT_DEVICE
    _DEFAULT_DEVICE = str(name)


@contextlib.contextmanager
def device_scope(device_name):
    prev = global_state.get_global_attribute("torch_device")
    global_state.set_global_attribute("torch_device", _parse_device(device_name))
    try:
        yield
    finally:
        global_state.set_global_attribute("torch_device", prev)


keras_export("keras.device")(device_scope)


def is_tensor(x):
    return isinstance(x, torch.Tensor)


def _python_dtype(x):
    """dtype name for Python scalars / nested lists of scalars (weak-typed → 32 bit)."""
    if isinstance(x, bool):
        return "bool"
    if isinstance(x, int):
        return "int32" if -(2**31) <= x < 2**31 else "int64"
    if isinstance(x, float):
        return config.floatx()
    if isinstance(x, complex):
        return "complex64"
    return None


def convert_to_tensor(x, dtype=None, sparse=None, ragged=None):
    """Anything array-like → ``torch.Tensor`` on the current device."""
    if type(x) is torch.Tensor or isinstance(x, torch.Tensor):
        if dtype is not None:
            td = dtype if isinstance(dtype, torch.dtype) else to_torch_dtype(dtype)
            if x.dtype != td:
                x = x.to(td)
        dev = get_device()
        if x.device != dev:
            if x.device.type == "meta" or dev.type == "meta":
                return x
            if x.device.type == dev.type and dev.index is None:
                return x
            x = x.to(dev)
        return x
    from keras_b200.core.variables import Variable

    if isinstance(x, Variable):
        v = x.value
        if dtype is not None:
            td = to_torch_dtype(dtype)
            if v.dtype != td:
                v = v.to(td)
        return v
    from keras_b200.core.keras_tensor import KerasTensor

    if isinstance(x, KerasTensor):
        raise ValueError(
            "A KerasTensor is symbolic: it is a placeholder for a shape and a dtype and has no "
            "value. It cannot be converted to a tensor; use it to build Functional models or "
            "call `keras.ops` functions on it."
        )
    td = to_torch_dtype(dtype) if dtype is not None else None
    if isinstance(x, (bool, int, float, complex)):
        if td is None:
            td = TORCH_DTYPES[_python_dtype(x)]
        dev = get_device()
        if dev.type == "cuda":
            # a fill kernel instead of a copy from pageable host memory: asynchronous, and legal while a CUDA graph is recorded
            return torch.full((), x, dtype=td, device=dev)
        return torch.as_tensor(x, dtype=td, device=dev)
    if isinstance(x, np.ndarray) or isinstance(x, np.generic):
        if x.dtype == np.uint16:
            x = x.astype(np.int32)
        elif x.dtype == np.uint32:
            x = x.astype(np.int64)
        elif x.dtype == np.uint64:
            x = x.astype(np.int64)
        if x.dtype.kind in "OUS":
            raise ValueError("String/object arrays cannot be converted to tensors.")
        if td is None and x.dtype == np.float64 and False:
            pass
        if isinstance(x, np.ndarray):
            if x.ndim and not x.flags.c_contiguous:
                x = np.ascontiguousarray(x)
            if not x.flags.writeable:
                x = x.copy()
        t = torch.as_tensor(x)
        return t.to(device=get_device(), dtype=td) if (td is not None or t.device != get_device()) else t
    if isinstance(x, (list, tuple)):
        flat_tensors = any(isinstance(e, torch.Tensor) for e in x)
        if flat_tensors or any(isinstance(e, Variable) for e in x):
            parts = [convert_to_tensor(e) for e in x]
            out_dtype = td
            if out_dtype is None:
                out_dtype = to_torch_dtype(result_type(*[p.dtype for p in parts]))
            return torch.stack([p.to(out_dtype) for p in parts])
        if td is None:
            arr = np.asarray(x)
            if arr.dtype == np.float64:
                arr = arr.astype(config.floatx() if config.floatx() != "bfloat16" else "float32")
                t = torch.as_tensor(arr, device=get_device())
                return t.to(to_torch_dtype(config.floatx()))
            if arr.dtype == np.int64:
                if arr.size == 0 or (arr.min() >= -(2**31) and arr.max() < 2**31):
                    arr = arr.astype(np.int32)
            if arr.dtype == object:
                raise ValueError(f"Cannot convert ragged/nested input to a tensor: {x!r}")
            return torch.as_tensor(arr, device=get_device())
        return torch.as_tensor(np.asarray(x), device=get_device()).to(td)
    if hasattr(x, "__array__"):
        return convert_to_tensor(np.asarray(x), dtype=dtype)
    if x is None:
        raise ValueError("Cannot convert `None` to a tensor.")
    return torch.as_tensor(x, dtype=td, device=get_device())


_PINNED_READBACK_BYTES = 1 << 20


def convert_to_numpy(x):
    from keras_b200.core.variables import Variable

    if isinstance(x, Variable):
        x = x.value
    if isinstance(x, torch.Tensor):
        x = x.detach()
        if x.device.type == "cuda" and x.numel() * x.element_size() >= _PINNED_READBACK_BYTES:
            # Large results go through page-locked memory: the copy engine writes it at PCIe speed, where a copy into pageable
            # memory is staged by the driver in small pieces.  The array keeps the page-locked block alive and the block goes
            # back to torch's host cache when the array is dropped, so a predict loop allocates it once.
            host = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
            host.copy_(x, non_blocking=True)
            torch.cuda.current_stream(x.device).synchronize()
            x = host
        elif x.device.type != "cpu":
            x = x.cpu()
        if x.dtype == torch.bfloat16:
            import ml_dtypes

            return x.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
        if x.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            import ml_dtypes

            nd = ml_dtypes.float8_e4m3fn if x.dtype == torch.float8_e4m3fn else ml_dtypes.float8_e5m2
            return x.view(torch.uint8).numpy().view(nd)
        if x.is_conj():
            x = x.resolve_conj()
        return x.numpy()
    if isinstance(x, (list, tuple)) and any(isinstance(e, torch.Tensor) for e in x):
        return np.array([convert_to_numpy(e) for e in x])
    return np.asarray(x)


def cast(x, dtype):
    from keras_b200.core.keras_tensor import KerasTensor

    if isinstance(x, KerasTensor):
        return KerasTensor(x.shape, dtype=standardize_dtype(dtype), sparse=x.sparse)
    td = to_torch_dtype(dtype)
    if isinstance(x, torch.Tensor):
        return x if x.dtype == td else x.to(td)
    return convert_to_tensor(x, dtype=td)


def shape(x):
    return tuple(x.shape)


def dtype_name(x):
    """Canonical dtype name of a tensor-like or Python scalar."""
    if isinstance(x, torch.Tensor):
        return standardize_dtype(x.dtype)
    if hasattr(x, "dtype"):
        return standardize_dtype(x.dtype)
    pd = _python_dtype(x)
    if pd is not None:
        return pd
    return standardize_dtype(convert_to_tensor(x).dtype)


# Placeholder extents used for `None` dimensions while tracing on the meta device.  Two passes
# with different primes tell static output dims from ones that follow a dynamic input dim.
_FILL_A, _FILL_B = 83, 89


def compute_output_spec(fn, *args, **kwargs):
    """Trace ``fn`` on meta tensors and return KerasTensors describing its outputs."""
    from keras_b200 import tree
    from keras_b200.core.keras_tensor import KerasTensor
    from keras_b200.core.scopes import StatelessScope, SymbolicScope

    def has_none(x):
        return isinstance(x, KerasTensor) and any(d is None for d in x.shape)

    any_none = any(has_none(x) for x in tree.flatten((args, kwargs)))

    def materialise(fill, device):
        def conv(x):
            if isinstance(x, KerasTensor):
                shp = tuple(fill if d is None else d for d in x.shape)
                return torch.ones(shp, dtype=to_torch_dtype(x.dtype), device=device)
            if isinstance(x, KerasShapeToken):
                return fill
            return x

        return conv

    def run(fill, device):
        a, k = tree.map_structure(materialise(fill, device), (args, kwargs))
        with device_scope(device):
            return fn(*a, **k)

    with StatelessScope(initialize_variables=False), SymbolicScope(), torch.no_grad():
        try:
            out_a = run(_FILL_A, "meta")
            out_b = run(_FILL_B, "meta") if any_none else None
        except Exception:
            # Some ops have no meta kernels or inspect values: fall back to real tensors.
            out_a = run(_FILL_A, "cpu")
            out_b = run(_FILL_B, "cpu") if any_none else None

    def to_spec(a, b=None):
        if isinstance(a, torch.Tensor):
            shp = list(a.shape)
            if b is not None:
                for i, (da, db) in enumerate(zip(a.shape, b.shape)):
                    if da != db:
                        shp[i] = None
            return KerasTensor(tuple(shp), dtype=standardize_dtype(a.dtype))
        return a

    if out_b is not None:
        return tree.map_structure(to_spec, out_a, out_b)
    return tree.map_structure(to_spec, out_a)


class KerasShapeToken:
    """Stand-in for a dynamic dimension value inside symbolic arguments."""
