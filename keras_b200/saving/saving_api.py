"""Public save / load entry points (keras/src/saving/saving_api.py:20-450): dispatch by extension."""

import os
import zipfile

from keras_b200.core.export_registry import keras_export
from keras_b200.saving import saving_lib
from keras_b200.utils import io_utils


@keras_export(["keras.saving.save_model", "keras.models.save_model"])
def save_model(model, filepath, overwrite=True, zipped=None, **kwargs):
    include_optimizer = kwargs.pop("include_optimizer", True)
    save_format = kwargs.pop("save_format", False)
    if save_format:
        if str(filepath).endswith((".h5", ".hdf5")) or str(filepath).endswith(".keras"):
            import warnings

            warnings.warn("The `save_format` argument is deprecated in Keras 3. We recommend removing this argument as it can be inferred from the file path. " f"Received: save_format={save_format}", stacklevel=2)
        else:
            raise ValueError(
                "The `save_format` argument is deprecated in Keras 3. Please remove this argument and pass a file path with either `.keras` or `.h5` extension."
                f"Received: save_format={save_format}")
    if kwargs:
        raise ValueError(f"The following argument(s) are not supported: {list(kwargs.keys())}")
    filepath = str(filepath)
    is_h5 = filepath.endswith((".h5", ".hdf5"))
    if zipped is None and not is_h5:
        zipped = not os.path.isdir(filepath)
    try:
        exists = (not is_h5) and os.path.exists(filepath)
    except TypeError:
        exists = False
    if os.path.exists(filepath) and not overwrite:
        proceed = io_utils.ask_to_proceed_with_overwrite(filepath)
        if not proceed:
            return
    if zipped and filepath.endswith(".keras"):
        return saving_lib.save_model(model, filepath)
    if not zipped and not is_h5:
        return saving_lib.save_model(model, filepath, zipped=False)
    if is_h5:
        from keras_b200.legacy.saving import legacy_h5_format

        return legacy_h5_format.save_model_to_hdf5(model, filepath, overwrite, include_optimizer)
    raise ValueError(
        "Invalid filepath extension for saving. Please add either a `.keras` extension for the native Keras format (recommended) "
        "or a `.h5` extension. Use `model.export(filepath)` if you want to export a SavedModel for use with TFLite/TFServing/etc. "
        f"Received: filepath={filepath}.")


@keras_export(["keras.saving.load_model", "keras.models.load_model"])
def load_model(filepath, custom_objects=None, compile=True, safe_mode=True):
    path = str(filepath)
    is_keras_zip = path.endswith(".keras") and os.path.isfile(path) and zipfile.is_zipfile(path)
    is_keras_dir = os.path.isdir(path) and os.path.exists(os.path.join(path, "config.json"))
    if is_keras_dir and os.path.exists(os.path.join(path, "state.npz")) is False and any(d.isdigit() for d in os.listdir(path)):
        is_keras_dir = False
    if is_keras_zip or is_keras_dir or path.startswith("hf://"):
        return saving_lib.load_model(filepath, custom_objects=custom_objects, compile=compile, safe_mode=safe_mode)
    if path.endswith((".h5", ".hdf5")):
        from keras_b200.legacy.saving import legacy_h5_format

        return legacy_h5_format.load_model_from_hdf5(filepath, custom_objects=custom_objects, compile=compile)
    if os.path.isdir(path) and any(d.isdigit() for d in os.listdir(path)):
        return _load_from_step_directory(path, custom_objects, compile, safe_mode)
    if path.endswith(".keras"):
        raise ValueError(f"File not found: filepath={filepath}. Please ensure the file is an accessible `.keras` zip file.")
    raise ValueError(
        f"File format not supported: filepath={filepath}. Keras 3 only supports V3 `.keras` files and legacy H5 format files "
        "(`.h5` extension). Note that the legacy SavedModel format is not supported by `load_model()` in Keras 3.")


def _load_from_step_directory(path, custom_objects, compile, safe_mode):
    """Checkpoint directories written by the ``OrbaxCheckpoint`` callback of this framework."""
    import json

    from keras_b200.callbacks.orbax_checkpoint import load_state_from_directory
    from keras_b200.saving.serialization_lib import deserialize_keras_object

    steps = sorted(int(d) for d in os.listdir(path) if d.isdigit())
    with open(os.path.join(path, str(steps[-1]), "config.json")) as f:
        config = json.load(f)
    if not compile:
        config["compile_config"] = None
    model = deserialize_keras_object(config, custom_objects, safe_mode=safe_mode)
    load_state_from_directory(model, path, steps[-1])
    return model


@keras_export("keras.saving.save_weights")
def save_weights(model, filepath, overwrite=True, max_shard_size=None, **kwargs):
    filepath_str = str(filepath)
    if max_shard_size is None and not filepath_str.endswith(".weights.h5"):
        raise ValueError(f"The filename must end in `.weights.h5`. Received: filepath={filepath_str}")
    if max_shard_size is not None and not filepath_str.endswith((".weights.h5", ".weights.json")):
        raise ValueError(f"The filename must end in `.weights.json` when `max_shard_size` is specified. Received: filepath={filepath_str}")
    try:
        exists = os.path.exists(filepath)
    except TypeError:
        exists = False
    if exists and not overwrite:
        proceed = io_utils.ask_to_proceed_with_overwrite(filepath_str)
        if not proceed:
            return
    saving_lib.save_weights_only(model, filepath, max_shard_size, **kwargs)


@keras_export("keras.saving.load_weights")
def load_weights(model, filepath, skip_mismatch=False, **kwargs):
    filepath_str = str(filepath)
    if os.path.isdir(filepath_str) and any(d.isdigit() for d in os.listdir(filepath_str)):
        from keras_b200.callbacks.orbax_checkpoint import load_state_from_directory

        return load_state_from_directory(model, filepath_str)
    if filepath_str.endswith(".keras"):
        if kwargs:
            raise ValueError(f"Invalid keyword arguments: {kwargs}")
        saving_lib.load_weights_only(model, filepath, skip_mismatch=skip_mismatch)
    elif filepath_str.endswith(".weights.h5") or filepath_str.endswith(".weights.json"):
        objects_to_skip = kwargs.pop("objects_to_skip", None)
        if kwargs:
            raise ValueError(f"Invalid keyword arguments: {kwargs}")
        saving_lib.load_weights_only(model, filepath, skip_mismatch=skip_mismatch, objects_to_skip=objects_to_skip)
    elif filepath_str.endswith(".h5") or filepath_str.endswith(".hdf5"):
        by_name = kwargs.pop("by_name", False)
        if kwargs:
            raise ValueError(f"Invalid keyword arguments: {kwargs}")
        from keras_b200.legacy.saving import legacy_h5_format

        legacy_h5_format.load_weights_from_hdf5(filepath, model, skip_mismatch=skip_mismatch, by_name=by_name)
    else:
        raise ValueError(f"File format not supported: filepath={filepath}. Keras 3 only supports V3 `.keras` and `.weights.h5` files, or legacy V1/V2 `.h5` files.")
