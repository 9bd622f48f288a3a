"""``Model``: a ``Layer`` with training / inference / persistence features.

Behaviour of keras/src/models/model.py:43-1289: ``Model(inputs, outputs)`` reroutes to
``Functional`` (:148-166); ``layers`` / ``get_layer`` / ``summary``; ``save`` / ``save_weights``
/ ``load_weights``; ``quantize`` (:454-699); state-tree API (:1060-1233).
"""

import inspect
import json
import re
import warnings

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.layer import Layer
from keras_b200.trainers.trainer import Trainer


@keras_export(["keras.Model", "keras.models.Model"])
class Model(Trainer, Layer):
    def __new__(cls, *args, **kwargs):
        if functional_init_arguments(args, kwargs) and cls is Model:
            from keras_b200.models.functional import Functional

            return Functional.__new__(Functional, *args, **kwargs)
        return super().__new__(cls, *args, **kwargs)

    def __init__(self, *args, **kwargs):
        Trainer.__init__(self)
        from keras_b200.models import functional

        if functional_init_arguments(args, kwargs):
            inject_functional_model_class(self.__class__)
            functional.Functional.__init__(self, *args, **kwargs)
        else:
            Layer.__init__(self, *args, **kwargs)
            self._init_trainer_state()

    def call(self, *args, **kwargs):
        raise NotImplementedError(f"Model {self.__class__.__name__} does not have a `call()` method implemented.")

    @property
    def layers(self):
        return list(self._flatten_layers(include_self=False, recursive=False))

    @layers.setter
    def layers(self, _):
        raise AttributeError("`Model.layers` attribute is reserved and should not be used. Please use another name.")

    def get_layer(self, name=None, index=None):
        if index is not None and name is not None:
            raise ValueError(f"Provide only a layer name or a layer index. Received: index={index}, name={name}.")
        if index is not None:
            if len(self.layers) <= index:
                raise ValueError(f"Was asked to retrieve layer at index {index} but model only has {len(self.layers)} layers.")
            return self.layers[index]
        if name is not None:
            for layer in self.layers:
                if layer.name == name:
                    return layer
            raise ValueError(f"No such layer: {name}. Existing layers are: {list(layer.name for layer in self.layers)}.")
        raise ValueError("Provide either a layer name or layer index at `get_layer`.")

    def summary(self, line_length=None, positions=None, print_fn=None, expand_nested=False, show_trainable=False, layer_range=None):
        from keras_b200.utils import summary_utils

        summary_utils.print_summary(self, line_length=line_length, positions=positions, print_fn=print_fn,
                                    expand_nested=expand_nested, show_trainable=show_trainable, layer_range=layer_range)

    def save(self, filepath, overwrite=True, zipped=None, **kwargs):
        from keras_b200.saving import saving_api

        return saving_api.save_model(self, filepath, overwrite=overwrite, zipped=zipped, **kwargs)

    def save_weights(self, filepath, overwrite=True, max_shard_size=None):
        from keras_b200.saving import saving_api

        return saving_api.save_weights(self, filepath, overwrite=overwrite, max_shard_size=max_shard_size)

    def load_weights(self, filepath, skip_mismatch=False, **kwargs):
        from keras_b200.saving import saving_api

        saving_api.load_weights(self, filepath, skip_mismatch=skip_mismatch, **kwargs)

    def quantize(self, mode=None, config=None, filters=None, **kwargs):
        """Quantize the weights of every supported leaf layer in place."""
        from keras_b200.quantizers.quantization_config import validate_and_resolve_config

        type_check = kwargs.pop("type_check", True)
        if kwargs:
            raise ValueError(f"Unrecognized keyword arguments passed to {self.__class__.__name__}: {kwargs}")
        config = validate_and_resolve_config(mode, config)
        mode = config.mode
        if type_check and type(self).quantize is not Model.quantize:
            pass
        if filters is not None and not (isinstance(filters, str) or callable(filters) or (isinstance(filters, (list, tuple)) and all(isinstance(f, str) for f in filters))):
            raise ValueError("The `filters` argument must be a regex string, a list of regex strings, or a callable. " f"Received: {type(filters)}")
        if mode in ("gptq", "awq"):
            from keras_b200.quantizers import calibration

            calibration.calibrated_quantize(self, mode, config, filters)
            self._reset_step_functions()
            return
        from keras_b200.quantizers.report import QuantizationReport

        verbose = getattr(self, "_quantize_verbose", False)
        report = QuantizationReport(mode=mode)
        graph_modified = False
        for layer in self._flatten_layers():
            if len(list(layer._flatten_layers())) != 1:
                continue
            path = getattr(layer, "path", None) or layer.name
            if not _should_quantize(layer, filters):
                report.add_skipped(path, QuantizationReport.SKIP_FILTERED)
                continue
            if getattr(layer, "_is_quantized", False):
                report.add_skipped(path, QuantizationReport.SKIP_ALREADY_QUANTIZED)
                continue
            if type(layer).quantize is Layer.quantize:
                if layer.weights:
                    report.add_skipped(path, QuantizationReport.SKIP_NO_SUPPORT)
                continue
            try:
                layer.quantize(mode, type_check=type_check, config=config)
                graph_modified = True
                report.add_quantized(path, mode, getattr(layer.dtype_policy, "name", mode))
            except NotImplementedError as e:
                report.add_skipped(path, QuantizationReport.SKIP_NO_SUPPORT)
                report.add_error(path, e) if "Invalid quantization mode" in str(e) else None
            except AttributeError:
                report.add_skipped(path, QuantizationReport.SKIP_NO_SUPPORT)
        if graph_modified:
            self._reset_step_functions()
        message = report.summary_warning()
        if message and report.errors:
            warnings.warn(message)
        self._quantization_report = report
        return report

    def quantization_summary(self, print_fn=None):
        """Print (and return) the report of the last ``quantize()`` call."""
        from keras_b200.quantizers.report import QuantizationReport
        from keras_b200.utils import io_utils

        report = QuantizationReport.from_model(self)
        (print_fn or io_utils.print_msg)(report.render())
        return report

    def get_quantization_layer_structure(self, mode):
        """Override to describe the model to the calibrated quantisation modes: ``{"pre_block_layers": [...],
        "sequential_blocks": [...]}`` (see ``keras_b200.quantizers.calibration``).  ``None``: the structure must come
        with the config."""
        return None

    def _reset_step_functions(self):
        self.train_function = None
        self.test_function = None
        self.predict_function = None
        self._invalidate()

    def build_from_config(self, config):
        if not config:
            return
        status = False
        if "input_shape" in config:
            if getattr(type(self), "build", None) is not None and not _is_default_build(self):
                status = self._build_by_run_for_single_pos_arg(config["input_shape"]) if False else _try(lambda: self.build(config["input_shape"]))
            else:
                status = self._build_by_run_for_single_pos_arg(config["input_shape"])
        elif "shapes_dict" in config:
            if not _is_default_build(self):
                status = _try(lambda: self.build(**config["shapes_dict"]))
            else:
                status = self._build_by_run_for_kwargs(config["shapes_dict"])
        if not status:
            warnings.warn(
                f"Model '{self.name}' had a build config, but the model cannot be built automatically in "
                "`build_from_config(config)`. You should implement `def build_from_config(self, config)`, and you "
                "might also want to implement the method  that generates the config at saving time, "
                "`def get_build_config(self)`. The method `build_from_config()` is meant to create the state of the "
                "model (i.e. its variables) upon deserialization.",
                stacklevel=2,
            )

    def _build_by_run_for_single_pos_arg(self, input_shape):
        from keras_b200.core.keras_tensor import KerasTensor

        try:
            spec = tree.map_shape_structure(lambda s: KerasTensor(s, dtype=self.input_dtype), input_shape)
            self(spec)
            return True
        except Exception:
            return False

    def _build_by_run_for_kwargs(self, shapes_dict):
        from keras_b200.core.keras_tensor import KerasTensor

        try:
            kwargs = {k[: -len("_shape")] if k.endswith("_shape") else k: tree.map_shape_structure(lambda s: KerasTensor(s, dtype=self.input_dtype), v) for k, v in shapes_dict.items()}
            self(**kwargs)
            return True
        except Exception:
            return False

    def to_json(self, **kwargs):
        from keras_b200.saving import serialization_lib

        return json.dumps(serialization_lib.serialize_keras_object(self), **kwargs)

    def export(self, filepath, format="tf_saved_model", verbose=None, input_signature=None, **kwargs):
        from keras_b200.export import export_model

        return export_model(self, filepath, format=format, verbose=verbose, input_signature=input_signature, **kwargs)

    @classmethod
    def from_config(cls, config, custom_objects=None):
        from keras_b200.models.functional import Functional, functional_from_config

        functional_keys = ["name", "layers", "input_layers", "output_layers"]
        is_functional_config = all(k in config for k in functional_keys)
        argspec = inspect.getfullargspec(cls.__init__)
        functional_init_args = inspect.getfullargspec(Functional.__init__).args[1:]
        revivable_as_functional = cls in {Functional, Model} or argspec.args[1:] == functional_init_args or (argspec.varargs == "args" and argspec.varkw == "kwargs")
        if is_functional_config and revivable_as_functional:
            return functional_from_config(cls, dict(config), custom_objects=custom_objects)
        try:
            return cls(**config)
        except TypeError as e:
            raise TypeError(
                "Unable to revive model from config. When overriding the `get_config()` method, make sure that the "
                "returned config contains all items used as arguments in the  constructor to "
                f"{cls}, which is the default behavior. You can override this default behavior by defining a "
                "`from_config(cls, config)` class method to specify how to create an instance of "
                f"{cls.__name__} from its config.\n\nReceived config={config}\n\nError encountered during deserialization: {e}"
            )

    def _get_variable_map(self):
        store = {}
        map_saveable_variables(self, store=store, visited_saveables=set())
        return store

    def get_state_tree(self, value_format="backend_tensor"):
        """Nested dicts keyed by variable path for trainable / non-trainable / optimizer / metrics variables."""
        assert value_format in ("backend_tensor", "numpy_array")
        out = {
            "trainable_variables": self._create_nested_dict(self.trainable_variables, value_format),
            "non_trainable_variables": self._create_nested_dict(self.non_trainable_variables, value_format),
        }
        if getattr(self, "optimizer", None) is not None:
            out["optimizer_variables"] = self._create_nested_dict(self.optimizer.variables, value_format)
        out["metrics_variables"] = self._create_nested_dict(self.metrics_variables, value_format)
        return out

    def _create_nested_dict(self, variables, value_format):
        flat = {}
        for v in variables:
            if v.path in flat:
                raise ValueError(f"The following variable path is found twice in the model: '{v.path}'. `get_state_tree()` can only be called when all variable paths are unique. Make sure to give unique names to your layers (and other objects).")
            flat[v.path] = v.value_unautocast() if value_format == "backend_tensor" else v.numpy()
        nested = {}
        for path, value in flat.items():
            parts = path.split("/")
            cur = nested
            for p in parts[:-1]:
                cur = cur.setdefault(p, {})
            cur[parts[-1]] = value
        return nested

    def set_state_tree(self, state_tree):
        for k, v in state_tree.items():
            path_value = flatten_nested_dict(v)
            if k == "trainable_variables":
                self._assign_variable_values(self.trainable_variables, path_value)
            elif k == "non_trainable_variables":
                self._assign_variable_values(self.non_trainable_variables, path_value)
            elif k == "optimizer_variables":
                if getattr(self, "optimizer", None) is not None:
                    self._assign_variable_values(self.optimizer.variables, path_value)
            elif k == "metrics_variables":
                self._assign_variable_values(self.metrics_variables, path_value)
            else:
                raise ValueError(f"Unknown variable name: {k}")

    def _assign_variable_values(self, variables, path_value_dict):
        for path, value in path_value_dict.items():
            for v in variables:
                if v.path == path:
                    v.assign(value)

    def _obj_type(self):
        return "Model"


def _try(fn):
    try:
        fn()
        return True
    except Exception:
        return False


def _is_default_build(model):
    b = type(model).build
    return getattr(b, "__wrapped__", b) is getattr(Layer.build, "__wrapped__", Layer.build) or getattr(b, "__wrapped__", b) is getattr(Model.build, "__wrapped__", None)


def _should_quantize(layer, filters):
    if filters is None:
        return True
    if isinstance(filters, str):
        return bool(re.search(filters, layer.name))
    if isinstance(filters, (list, tuple)):
        return any(re.search(p, layer.name) for p in filters)
    if callable(filters):
        return filters(layer)
    return True


def flatten_nested_dict(d, parent=""):
    out = {}
    for k, v in d.items():
        key = f"{parent}/{k}" if parent else k
        if isinstance(v, dict):
            out.update(flatten_nested_dict(v, key))
        else:
            out[key] = v
    return out


def map_saveable_variables(saveable, store, visited_saveables):
    from keras_b200.saving.saving_lib import walk_saveable
    from keras_b200.ops.operation import KerasSaveable

    if id(saveable) in visited_saveables:
        return
    visited_saveables.add(id(saveable))
    variables = []
    if hasattr(saveable, "_trainable_variables"):
        variables += list(saveable._trainable_variables) + list(saveable._non_trainable_variables)
    elif hasattr(saveable, "variables"):
        variables += list(saveable.variables)
    for v in variables:
        if v.path in store:
            raise ValueError(f"The model contains two variables with a duplicate path: path='{v.path}' appears at least twice. This path is used for {v} and for {store[v.path]}. In order to get a variable map, make sure to use unique paths/names for each variable.")
        store[v.path] = v
    for child_attr, child_obj in walk_saveable(saveable):
        if isinstance(child_obj, KerasSaveable):
            map_saveable_variables(child_obj, store, visited_saveables)
        elif isinstance(child_obj, (list, dict, tuple, set)):
            items = child_obj.values() if isinstance(child_obj, dict) else child_obj
            for item in items:
                if isinstance(item, KerasSaveable):
                    map_saveable_variables(item, store, visited_saveables)


def functional_init_arguments(args, kwargs):
    return (len(args) == 2) or (len(args) == 1 and "outputs" in kwargs) or ("inputs" in kwargs and "outputs" in kwargs)


def inject_functional_model_class(cls):
    """Make a user subclass of ``Model`` that is built functionally inherit from ``Functional``."""
    from keras_b200.models import functional

    if cls is Model:
        return functional.Functional
    if cls is object:
        return object
    cls.__bases__ = tuple(inject_functional_model_class(base) for base in cls.__bases__)
    cls.__new__(cls)
    return cls
