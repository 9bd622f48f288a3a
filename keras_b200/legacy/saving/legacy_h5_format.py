"""Whole-model and weights I/O in the Keras 2 HDF5 layout (keras/src/legacy/saving/legacy_h5_format.py):

* root attributes ``keras_version``, ``backend``, ``model_config`` (JSON), ``training_config`` (JSON);
* group ``model_weights`` with attribute ``layer_names``; one sub-group per layer with attribute ``weight_names`` and one
  dataset per weight (trainable first, then non-trainable); ``top_level_model_weights`` for variables owned by the model;
* group ``optimizer_weights`` with ``weight_names`` and one dataset per optimizer variable.
"""

import json
import os
import warnings

import numpy as np

from keras_b200.core import config as core_config
from keras_b200.core.tensor import convert_to_numpy
from keras_b200.legacy.saving import legacy_serialization
from keras_b200.saving import hdf5, object_registration, serialization_lib
from keras_b200.utils import io_utils
from keras_b200.version import __version__ as keras_version


def _legacy_weights(layer):
    return layer.trainable_weights + layer.non_trainable_weights


def _json_default(obj):
    if hasattr(obj, "get_config"):
        return {"class_name": obj.__class__.__name__, "config": obj.get_config()}
    if isinstance(obj, np.ndarray):
        return obj.tolist()
    if isinstance(obj, np.generic):
        return obj.item()
    if callable(obj):
        return obj.__name__
    if isinstance(obj, type):
        return obj.__name__
    raise TypeError(f"Unable to serialize {obj} to JSON. Unrecognized type {type(obj)}.")


def model_metadata(model, include_optimizer=True):
    metadata = {"keras_version": str(keras_version), "backend": core_config.backend(),
                "model_config": {"class_name": model.__class__.__name__, "config": model.get_config()}}
    if getattr(model, "optimizer", None) and include_optimizer and model.compiled:
        raw = getattr(model, "_compile_config", None) or {}
        training = dict(getattr(raw, "config", raw))
        training.pop("optimizer", None)
        training = legacy_serialization.serialize_nested(training)
        training["optimizer_config"] = {"class_name": object_registration.get_registered_name(model.optimizer.__class__),
                                        "config": model.optimizer.get_config()}
        metadata["training_config"] = training
    return metadata


def _write_weights(writer, path, weights):
    names = [str(w.path) for w in weights]
    writer.create_group(path, attrs={"weight_names": np.array(names, dtype=object)} if names else {"weight_names": np.zeros((0,), dtype="S1")})
    for name, w in zip(names, weights):
        writer.create_dataset(f"{path}/{name}", convert_to_numpy(w))


def save_weights_to_hdf5_group(writer, path, model):
    writer.create_group(path, attrs={"layer_names": np.array([layer.name for layer in model.layers], dtype=object),
                                     "backend": core_config.backend(), "keras_version": str(keras_version)})
    for layer in sorted(model.layers, key=lambda x: x.name):
        _write_weights(writer, f"{path}/{layer.name}", _legacy_weights(layer))
    own = [v for v in model._trainable_variables + model._non_trainable_variables if any(v is w for w in model.weights)]
    _write_weights(writer, f"{path}/top_level_model_weights", own)


def save_model_to_hdf5(model, filepath, overwrite=True, include_optimizer=True):
    filepath = str(filepath)
    if not overwrite and os.path.isfile(filepath):
        if not io_utils.ask_to_proceed_with_overwrite(filepath):
            return
    dirpath = os.path.dirname(filepath)
    if dirpath and not os.path.exists(dirpath):
        os.makedirs(dirpath, exist_ok=True)
    writer = hdf5.Writer()
    for k, v in model_metadata(model, include_optimizer).items():
        writer.set_attr("/", k, json.dumps(v, default=_json_default) if isinstance(v, (dict, list, tuple)) else v)
    save_weights_to_hdf5_group(writer, "model_weights", model)
    if include_optimizer and getattr(model, "optimizer", None) is not None:
        variables = list(model.optimizer.variables)
        if variables:
            _write_weights(writer, "optimizer_weights", variables)
    writer.save(filepath)


def _attr_list(group, name):
    """String-array attribute, including the chunked form ``name0, name1, ...`` used for very long lists."""
    attrs = group.attrs
    if name in attrs:
        data = attrs[name]
        vals = data.tolist() if hasattr(data, "tolist") else list(data)
    else:
        vals, i = [], 0
        while f"{name}{i}" in attrs:
            vals.extend(np.asarray(attrs[f"{name}{i}"]).tolist())
            i += 1
    return [v.decode("utf8") if isinstance(v, bytes) else str(v) for v in (vals if isinstance(vals, list) else [vals])]


def load_subset_weights_from_hdf5_group(group):
    return [np.asarray(group[name]) for name in _attr_list(group, "weight_names")]


def _set_weights(instance, symbolic_weights, weight_values, name, skip_mismatch=False):
    for i, value in enumerate(weight_values):
        expected = tuple(symbolic_weights[i].shape)
        if expected != tuple(value.shape):
            if skip_mismatch:
                warnings.warn(f"Skipping loading weights for {name} due to mismatch in shape for weight {symbolic_weights[i].path}. "
                              f"Weight expects shape {expected}. Received saved weight with shape {value.shape}", stacklevel=2)
                continue
            raise ValueError(f"Shape mismatch in {name} for weight {symbolic_weights[i].path}. Weight expects shape {expected}. "
                             f"Received saved weight with shape {value.shape}")
        symbolic_weights[i].assign(value)
    if hasattr(instance, "finalize_state") and symbolic_weights:
        instance.finalize_state()


def load_weights_from_hdf5_group(group, model, skip_mismatch=False):
    filtered = [layer for layer in model.layers if _legacy_weights(layer)]
    layer_names = [n for n in _attr_list(group, "layer_names") if _attr_list(group[n], "weight_names")]
    if len(layer_names) != len(filtered):
        raise ValueError(f"Layer count mismatch when loading weights from file. Model expected {len(filtered)} layers, found {len(layer_names)} saved layers.")
    for k, name in enumerate(layer_names):
        layer = filtered[k]
        values = load_subset_weights_from_hdf5_group(group[name])
        symbolic = _legacy_weights(layer)
        if len(values) != len(symbolic):
            raise ValueError(f"Weight count mismatch for layer #{k} (named {layer.name} in the current model, {name} in the save file). "
                             f"Layer expects {len(symbolic)} weight(s). Received {len(values)} saved weight(s)")
        _set_weights(layer, symbolic, values, name=f"layer #{k} (named {layer.name})", skip_mismatch=skip_mismatch)
    if "top_level_model_weights" in group:
        own = [v for v in model._trainable_variables + model._non_trainable_variables if any(v is w for w in model.weights)]
        values = load_subset_weights_from_hdf5_group(group["top_level_model_weights"])
        if len(values) != len(own):
            raise ValueError(f"Weight count mismatch for top-level weights when loading weights from file. Model expects {len(own)} top-level weight(s). Received {len(values)} saved top-level weight(s)")
        _set_weights(model, own, values, name="top-level model", skip_mismatch=skip_mismatch)


def load_weights_from_hdf5_group_by_name(group, model, skip_mismatch=False):
    index = {}
    for layer in model.layers:
        if layer.name:
            index.setdefault(layer.name, []).append(layer)
    for k, name in enumerate(_attr_list(group, "layer_names")):
        values = load_subset_weights_from_hdf5_group(group[name])
        for layer in index.get(name, []):
            symbolic = _legacy_weights(layer)
            if len(values) != len(symbolic):
                if skip_mismatch:
                    warnings.warn(f"Skipping loading of weights for layer #{k} (named {layer.name}) due to mismatch in number of weights. "
                                  f"Layer expects {len(symbolic)} weight(s). Received {len(values)} saved weight(s)", stacklevel=2)
                    continue
                raise ValueError(f"Weight count mismatch for layer #{k} (named {layer.name}). Layer expects {len(symbolic)} weight(s). Received {len(values)} saved weight(s)")
            _set_weights(layer, symbolic, values, name=f"layer #{k} (named {layer.name})", skip_mismatch=skip_mismatch)


def load_weights_from_hdf5(filepath, model, skip_mismatch=False, by_name=False):
    with hdf5.File(str(filepath), "r") as f:
        group = f["model_weights"] if "layer_names" not in f.attrs and "model_weights" in f else f
        if by_name:
            load_weights_from_hdf5_group_by_name(group, model, skip_mismatch)
        else:
            load_weights_from_hdf5_group(group, model, skip_mismatch)


def load_model_from_hdf5(filepath, custom_objects=None, compile=True, safe_mode=True):
    custom_objects = {**(custom_objects or {}), **object_registration.GLOBAL_CUSTOM_OBJECTS}
    with hdf5.File(str(filepath), "r") as f:
        model_config = f.attrs.get("model_config")
        if model_config is None:
            raise ValueError(f"No model config found in the file at {filepath}.")
        if isinstance(model_config, bytes):
            model_config = model_config.decode("utf-8")
        model_config = legacy_serialization.decode_json(model_config)
        with serialization_lib.SafeModeScope(safe_mode):
            model = legacy_serialization.model_from_config(model_config, custom_objects=custom_objects)
            load_weights_from_hdf5_group(f["model_weights"], model)
        if not compile:
            return model
        training_config = f.attrs.get("training_config")
        if training_config is None:
            warnings.warn("No training configuration found in the save file, so the model was *not* compiled. Compile it manually.")
            return model
        if isinstance(training_config, bytes):
            training_config = training_config.decode("utf-8")
        training_config = legacy_serialization.decode_json(training_config)
        model.compile(**legacy_serialization.compile_args_from_training_config(training_config, custom_objects))
        if "optimizer_weights" in f:
            try:
                model.optimizer.build(model._trainable_variables if hasattr(model, "_trainable_variables") and model._trainable_variables else model.trainable_variables)
                values = load_subset_weights_from_hdf5_group(f["optimizer_weights"])
                model.optimizer.set_weights(values)
            except (ValueError, NotImplementedError, AttributeError):
                warnings.warn("Error in loading the saved optimizer state. As a result, your model is starting with a freshly initialized optimizer.")
    return model
