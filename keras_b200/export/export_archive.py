"""``ExportArchive``: collect endpoints (functions of tensors closed over tracked variables) and write them out as
``torch.export`` programs (API of keras/src/export/saved_model.py:27-560: ``track``, ``add_endpoint``,
``add_variable_collection``, ``write_out``)."""

import json
import os

import torch

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer
from keras_b200.utils import io_utils

MANIFEST = "keras_export.json"


def _spec_to_tensor(spec, dynamic_batch):
    shape = tuple(spec.shape)
    dtype = getattr(torch, str(spec.dtype) if spec.dtype else "float32")
    concrete = [(dynamic_batch if i == 0 else 1) if d is None else d for i, d in enumerate(shape)]
    if dtype.is_floating_point:
        return torch.zeros(concrete, dtype=dtype)
    return torch.zeros(concrete, dtype=dtype)


def _standardize_signature(signature):
    def one(s):
        if isinstance(s, (KerasTensor, InputSpec)):
            return s
        if isinstance(s, torch.Tensor):
            return InputSpec(shape=(None,) + tuple(s.shape[1:]), dtype=str(s.dtype).replace("torch.", ""))
        if hasattr(s, "shape") and hasattr(s, "dtype"):
            return InputSpec(shape=tuple(s.shape), dtype=str(s.dtype))
        raise TypeError(f"Unsupported type {type(s)} for {s}. Supported types are: `keras.InputSpec`, `keras.KerasTensor` and backend tensor.")

    return tree.map_structure(one, signature)


class _EndpointModule(torch.nn.Module):
    """Wraps a Python endpoint so that ``torch.export`` sees its variables as parameters."""

    def __init__(self, fn, variables):
        super().__init__()
        self._fn = fn
        self.params = torch.nn.ParameterList([v._value if isinstance(v._value, torch.nn.Parameter) else torch.nn.Parameter(v._value, requires_grad=False) for v in variables])

    def forward(self, *args):
        with torch.no_grad():
            out = self._fn(*args)
        return out


@keras_export("keras.export.ExportArchive")
class ExportArchive:
    def __init__(self):
        self._endpoint_names = []
        self._endpoint_signatures = {}
        self._endpoints = {}
        self._tracked = []
        self._variables = []
        self._collections = {}

    @property
    def variables(self):
        return list(self._variables)

    @property
    def trainable_variables(self):
        return [v for v in self._variables if v.trainable]

    @property
    def non_trainable_variables(self):
        return [v for v in self._variables if not v.trainable]

    def track(self, resource):
        """Track the variables of a layer or model so that endpoints closing over them can be exported."""
        if isinstance(resource, Layer) and not resource.built:
            raise ValueError("The layer provided has not yet been built. It must be built before export.")
        self._tracked.append(resource)
        if isinstance(resource, Layer):
            for v in resource.variables:
                if not any(v is w for w in self._variables):
                    self._variables.append(v)

    def add_endpoint(self, name, fn, input_signature=None, **kwargs):
        if name in self._endpoint_names:
            raise ValueError(f"Endpoint name '{name}' is already taken.")
        if input_signature is None:
            raise ValueError(f"You must provide an `input_signature` argument when adding the endpoint '{name}'.")
        signature = _standardize_signature(input_signature)
        if not isinstance(signature, (list, tuple)):
            signature = [signature]
        self._endpoint_names.append(name)
        self._endpoint_signatures[name] = list(signature)
        self._endpoints[name] = fn
        setattr(self, name, fn)
        return fn

    def track_and_add_endpoint(self, name, resource, input_signature, **kwargs):
        self.track(resource)
        return self.add_endpoint(name, resource.__call__ if isinstance(resource, Layer) else resource, input_signature, **kwargs)

    def add_variable_collection(self, name, variables):
        if not isinstance(variables, (list, tuple, set)):
            raise ValueError(f"Expected `variables` to be a list/tuple/set. Received instead object of type '{type(variables)}'.")
        from keras_b200.core.variables import Variable

        if not all(isinstance(v, Variable) for v in variables):
            raise ValueError(f"Expected all elements in `variables` to be `Variable` instances. Found instead the following types: {list(set(type(v) for v in variables))}")
        self._collections[name] = list(variables)

    def write_out(self, filepath, options=None, verbose=True):
        if not self._endpoint_names:
            raise ValueError("No endpoints have been set yet. Call add_endpoint().")
        self._filter_and_track_resources()
        os.makedirs(filepath, exist_ok=True)
        manifest = {"format": "keras_b200.torch_export", "endpoints": {}, "variable_collections": {k: [v.path for v in vs] for k, vs in self._collections.items()}}
        for name in self._endpoint_names:
            fn, signature = self._endpoints[name], self._endpoint_signatures[name]
            flat_specs = tree.flatten(signature)
            example = [_spec_to_tensor(s, 2) for s in flat_specs]
            device = self._variables[0]._value.device if self._variables else torch.device("cpu")
            example = [e.to(device) for e in example]

            def call(*flat_args, _fn=fn, _sig=signature):
                args = tree.pack_sequence_as(_sig, list(flat_args))
                return _fn(*args)

            module = _EndpointModule(call, self._variables).eval()
            dynamic = []
            for s in flat_specs:
                if len(s.shape) > 0 and s.shape[0] is None:
                    dynamic.append({0: torch.export.Dim("batch", min=1)})
                else:
                    dynamic.append(None)
            try:
                program = torch.export.export(module, tuple(example), dynamic_shapes=(tuple(dynamic),) if any(d is not None for d in dynamic) else None, strict=False)
            except Exception:
                program = torch.export.export(module, tuple(example), strict=False)  # static shapes as a fallback
            target = os.path.join(filepath, f"{name}.pt2")
            torch.export.save(program, target)
            manifest["endpoints"][name] = {"file": f"{name}.pt2", "inputs": [{"shape": list(s.shape), "dtype": str(s.dtype)} for s in flat_specs]}
        with open(os.path.join(filepath, MANIFEST), "w") as f:
            json.dump(manifest, f, indent=2)
        if verbose:
            endpoints = "\n\n".join(f"* Endpoint '{n}'\n  inputs: {manifest['endpoints'][n]['inputs']}" for n in self._endpoint_names)
            io_utils.print_msg(f"Saved artifact at '{filepath}'. The following endpoints are available:\n\n{endpoints}")

    def _filter_and_track_resources(self):
        pass


def get_input_signature(model):
    from keras_b200.models import Functional, Sequential

    if not model.built:
        raise ValueError("The model provided has not yet been built. It must be built before export.")
    if isinstance(model, Functional):
        return tree.map_structure(lambda x: InputSpec(shape=tuple(x.shape), dtype=x.dtype), model._inputs_struct)
    if isinstance(model, Sequential):
        return InputSpec(shape=tuple(model.inputs[0].shape), dtype=model.inputs[0].dtype)
    shapes = getattr(model, "_build_shapes_dict", None)
    if shapes:
        return [InputSpec(shape=tuple(s), dtype=model.input_dtype if hasattr(model, "input_dtype") else "float32") for s in shapes.values()]
    raise ValueError("Could not infer the input signature; pass `input_signature`.")


def export_model(model, filepath, format="tf_saved_model", verbose=None, input_signature=None, **kwargs):
    """``Model.export``: ``format`` in ``torch_export`` (native), ``onnx``, ``tf_saved_model``, ``litert``, ``openvino``."""
    verbose = True if verbose is None else verbose
    if format == "tf_saved_model":
        try:
            import tensorflow  # noqa: F401
        except ImportError:
            raise ImportError("`format='tf_saved_model'` needs TensorFlow, which is not installed. Use `format='torch_export'` (native) or `format='onnx'`.")
        raise NotImplementedError("SavedModel export is not available on this runtime; use `format='torch_export'` or `format='onnx'`.")
    if format in ("litert", "tflite"):
        raise ImportError("`format='litert'` needs the `ai-edge-litert`/TensorFlow converter, which is not installed. Use `format='torch_export'` or `format='onnx'`.")
    if format == "openvino":
        raise ImportError("`format='openvino'` needs the `openvino` package, which is not installed. Use `format='torch_export'` or `format='onnx'`.")
    if input_signature is None:
        input_signature = get_input_signature(model)
    if format == "onnx":
        try:
            import onnx  # noqa: F401
        except ImportError:
            raise ImportError("`format='onnx'` needs the `onnx` package (`pip install onnx`).")
        specs = tree.flatten(_standardize_signature(input_signature))
        example = tuple(_spec_to_tensor(s, 2) for s in specs)

        class _Wrapper(torch.nn.Module):
            def forward(self, *args):
                return model(*tree.pack_sequence_as(input_signature, list(args)) if isinstance(input_signature, (list, tuple)) else (args[0],), training=False)

        torch.onnx.export(_Wrapper().eval(), example, filepath, opset_version=kwargs.get("opset_version", 18), dynamo=True)
        if verbose:
            io_utils.print_msg(f"Saved artifact at '{filepath}'.")
        return
    if format != "torch_export":
        raise ValueError(f"Unrecognized format={format}. Supported formats are: ['torch_export', 'onnx', 'tf_saved_model', 'litert', 'openvino'].")
    archive = ExportArchive()
    archive.track(model)
    sig = input_signature if isinstance(input_signature, (list, tuple)) else [input_signature]

    def serve(*args):
        return model(*args, training=False) if model._call_has_training_arg else model(*args)

    archive.add_endpoint("serve", serve, sig)
    archive.write_out(filepath, verbose=verbose)


class _LoadedArchive:
    """Reloaded export: attribute per endpoint, callable on tensors."""

    def __init__(self, path):
        with open(os.path.join(path, MANIFEST)) as f:
            self.manifest = json.load(f)
        self._programs = {}
        for name, info in self.manifest["endpoints"].items():
            program = torch.export.load(os.path.join(path, info["file"]))
            self._programs[name] = program.module()
            setattr(self, name, self._programs[name])

    @property
    def endpoints(self):
        return list(self._programs)


def load_exported(filepath):
    """Load an artefact written with ``format="torch_export"`` / ``ExportArchive.write_out``."""
    return _LoadedArchive(filepath)
