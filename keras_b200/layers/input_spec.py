"""``InputSpec``: declarative constraints on a layer's inputs (keras/src/layers/input_spec.py)."""

from keras_b200 import tree
from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.export_registry import keras_export


@keras_export(["keras.InputSpec", "keras.layers.InputSpec"])
class InputSpec:
    def __init__(self, dtype=None, shape=None, ndim=None, max_ndim=None, min_ndim=None, axes=None, allow_last_axis_squeeze=False, name=None, optional=False):
        self.dtype = standardize_dtype(dtype) if dtype is not None else None
        if shape is not None:
            self.shape = tuple(shape)
            self.ndim = len(shape)
        else:
            self.ndim = ndim
            self.shape = None
        self.max_ndim = max_ndim
        self.min_ndim = min_ndim
        self.name = name
        self.optional = optional
        self.allow_last_axis_squeeze = allow_last_axis_squeeze
        try:
            self.axes = {int(k): axes[k] for k in (axes or {})}
        except (ValueError, TypeError):
            raise TypeError(f"Argument `axes` must be a dict with integer keys. Received: axes={axes}")
        if self.axes and (self.ndim is not None or self.max_ndim is not None):
            max_dim = (self.ndim if self.ndim else self.max_ndim) - 1
            max_axis = max(self.axes)
            if max_axis > max_dim:
                raise ValueError(f"Axis {max_axis} is greater than the maximum allowed value: {max_dim}")

    def __repr__(self):
        parts = [f"{k}={getattr(self, k)}" for k in ("dtype", "shape", "ndim", "max_ndim", "min_ndim", "axes") if getattr(self, k)]
        return f"InputSpec({', '.join(parts)})"

    def get_config(self):
        return {"dtype": self.dtype, "shape": self.shape, "ndim": self.ndim, "max_ndim": self.max_ndim, "min_ndim": self.min_ndim, "axes": self.axes}

    @classmethod
    def from_config(cls, config):
        return cls(**config)


def assert_input_compatibility(input_spec, inputs, layer_name):
    if not input_spec:
        return
    specs = tree.flatten(input_spec)
    if isinstance(inputs, dict):
        names = [s.name for s in specs]
        if all(names):
            missing = [n for n in names if n not in inputs and not next(s for s in specs if s.name == n).optional]
            if missing:
                raise ValueError(f'Missing data for input "{missing[0]}". You passed a data dictionary with keys {list(inputs.keys())}. Expected the following keys: {names}')
            inputs = [inputs.get(n) for n in names]
        else:
            inputs = tree.flatten(inputs)
    else:
        inputs = tree.flatten(inputs)
    if len(inputs) != len(specs):
        raise ValueError(f'Layer "{layer_name}" expects {len(specs)} input(s), but it received {len(inputs)} input tensors. Inputs received: {inputs}')
    for i, (x, spec) in enumerate(zip(inputs, specs)):
        if spec is None:
            continue
        if x is None:
            if spec.optional:
                continue
            raise ValueError(f'Layer "{layer_name}" expects input {i} to be a tensor, received None.')
        if not hasattr(x, "shape"):
            raise ValueError(f"Inputs to a layer should be tensors. Got '{x}' (of type {type(x)}) as input for layer '{layer_name}'.")
        shape = tuple(x.shape)
        ndim = len(shape)
        if spec.ndim is not None and not spec.allow_last_axis_squeeze and ndim != spec.ndim:
            raise ValueError(f'Input {i} of layer "{layer_name}" is incompatible with the layer: expected ndim={spec.ndim}, found ndim={ndim}. Full shape received: {shape}')
        if spec.max_ndim is not None and ndim > spec.max_ndim:
            raise ValueError(f'Input {i} of layer "{layer_name}" is incompatible with the layer: expected max_ndim={spec.max_ndim}, found ndim={ndim}')
        if spec.min_ndim is not None and ndim < spec.min_ndim:
            raise ValueError(f'Input {i} of layer "{layer_name}" is incompatible with the layer: expected min_ndim={spec.min_ndim}, found ndim={ndim}. Full shape received: {shape}')
        if spec.dtype is not None and standardize_dtype(x.dtype) != spec.dtype:
            raise ValueError(f'Input {i} of layer "{layer_name}" is incompatible with the layer: expected dtype={spec.dtype}, found dtype={standardize_dtype(x.dtype)}')
        if spec.axes:
            for axis, value in spec.axes.items():
                if value is not None and shape[axis] not in {value, None}:
                    raise ValueError(f'Input {i} of layer "{layer_name}" is incompatible with the layer: expected axis {axis} of input shape to have value {value}, but received input with shape {shape}')
        if spec.shape is not None:
            spec_shape, cmp_shape = spec.shape, shape
            if spec.allow_last_axis_squeeze:
                if cmp_shape and cmp_shape[-1] == 1:
                    cmp_shape = cmp_shape[:-1]
                if spec_shape and spec_shape[-1] == 1:
                    spec_shape = spec_shape[:-1]
            for sd, d in zip(spec_shape, cmp_shape):
                if sd is not None and d is not None and sd != d:
                    raise ValueError(f'Input {i} of layer "{layer_name}" is incompatible with the layer: expected shape={spec.shape}, found shape={shape}')
