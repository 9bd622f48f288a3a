"""The ``.keras`` archive and weight-file formats.

File layout follows keras/src/saving/saving_lib.py: a zip with *stored* members
``metadata.json``, ``config.json``, ``model.weights.h5`` (or ``.npz``) and ``assets/``
(:44-56,75-270); the state walk visits children by ``sorted(dir(obj))`` with private names last,
minus a per-type skip set, ``layers`` first for Sequential/Functional, containers named
``snake_case(class)`` with ``_N`` suffixes (:731-766,937-1098); each saveable with variables gets
``<path>/vars`` with datasets ``"0","1",…`` (:1289-1483); sharded weights use a
``.weights.json`` index (:1486-1812).  HDF5 bytes are produced/consumed by
``keras_b200.saving.hdf5`` instead of ``h5py``.
"""

import datetime
import io
import json
import os
import pathlib
import re
import shutil
import tempfile
import warnings
import zipfile

import numpy as np

from keras_b200.core import global_state
from keras_b200.core.naming import to_snake_case
from keras_b200.core.tensor import convert_to_numpy
from keras_b200.ops.operation import KerasSaveable
from keras_b200.saving import hdf5
from keras_b200.saving.serialization_lib import ObjectSharingScope, deserialize_keras_object, serialize_keras_object
from keras_b200.version import KERAS_API_VERSION

_CONFIG_FILENAME = "config.json"
_METADATA_FILENAME = "metadata.json"
_VARS_FNAME = "model.weights"
_VARS_FNAME_H5 = _VARS_FNAME + ".h5"
_VARS_FNAME_NPZ = _VARS_FNAME + ".npz"
_ASSETS_DIRNAME = "assets"
_MAX_MEMBER_BYTES = 1 << 40


# --------------------------------------------------------------------------------- state walk
_SKIP_CACHE = {}


def _skip_names(obj_type):
    names = _SKIP_CACHE.get(obj_type)
    if names is None:
        from keras_b200.layers.layer import Layer
        from keras_b200.losses.loss import Loss
        from keras_b200.metrics.metric import Metric
        from keras_b200.optimizers.optimizers import Optimizer

        if obj_type == "Layer":
            ref = Layer()
        elif obj_type == "Functional":
            ref = Layer()
        elif obj_type == "Sequential":
            ref = Layer()
        elif obj_type == "Model":
            from keras_b200.models.model import Model

            ref = Model()
        elif obj_type == "Metric":
            ref = Metric()
        elif obj_type == "Optimizer":
            ref = Optimizer(1.0)
        elif obj_type == "Loss":
            ref = Loss()
        else:
            ref = None
        names = frozenset(dir(ref)) if ref is not None else frozenset()
        if obj_type in ("Functional", "Sequential"):
            from keras_b200.models.model import Model

            names = names | frozenset(dir(Model())) - {"layers"} if False else names
        _SKIP_CACHE[obj_type] = names
    return names


# Internal attributes of this framework's classes that must never appear as file paths.
_INTERNAL = frozenset({
    "_layers", "_trainable_variables", "_non_trainable_variables", "_metrics", "_seed_generators", "_functional", "_stack",
    "_operations", "_operations_by_depth", "_nodes_by_depth", "_nodes", "_inputs", "_outputs", "_inputs_struct", "_outputs_struct",
    "_inbound_nodes", "_outbound_nodes", "_losses", "_losses_override", "_plan", "_cached_vars", "_autocast_cache",
    "_compile_loss", "_compile_metrics", "_loss_tracker", "_compile_config", "_parallel_engine", "history", "_variables",
    "_trainable_variables_indices", "_exclude_from_weight_decay", "_eval_epoch_iterator", "_flat_losses", "_tracked_metrics",
})


def walk_saveable(saveable):
    """Yield ``(attribute name, child)`` pairs in the order that defines file paths."""
    obj_type = saveable._obj_type()
    skip = _skip_names(obj_type)
    names = [n for n in dir(saveable) if n not in skip and n not in _INTERNAL and not n.startswith("__")]
    public = sorted(n for n in names if not n.startswith("_"))
    private = sorted(n for n in names if n.startswith("_"))
    ordered = public + private
    if obj_type in ("Sequential", "Functional"):
        yield "layers", list(saveable.layers)
        ordered = [n for n in ordered if n != "layers"]
    for name in ordered:
        if name == "layers" and obj_type in ("Sequential", "Functional"):
            continue
        try:
            child = getattr(saveable, name)
        except Exception:
            continue
        if isinstance(child, (KerasSaveable, list, dict, tuple, set)):
            yield name, child


def _unique_name(name, used):
    if name not in used:
        used[name] = 0
        return name
    used[name] += 1
    return f"{name}_{used[name]}"


def _name_key(name):
    m = re.match(r"^(.*?)_(\d+)$", name)
    if m:
        return m.group(1), int(m.group(2))
    return name, 0


def _visit_state(saveable, weights_store, assets_store, inner_path, visited, fn, failed=None, error_msgs=None, skip_mismatch=False):
    """Depth-first walk calling ``fn(saveable, weights_entry_path, assets_path)`` once per object."""
    if id(saveable) in visited:
        return
    visited.add(id(saveable))
    fn(saveable, inner_path)
    for child_attr, child_obj in walk_saveable(saveable):
        if isinstance(child_obj, KerasSaveable):
            _visit_state(child_obj, weights_store, assets_store, _join(inner_path, child_attr), visited, fn, failed, error_msgs, skip_mismatch)
        elif isinstance(child_obj, (list, dict, tuple, set)):
            _visit_container(child_obj, weights_store, assets_store, _join(inner_path, child_attr), visited, fn, failed, error_msgs, skip_mismatch)


def _visit_container(container, weights_store, assets_store, inner_path, visited, fn, failed, error_msgs, skip_mismatch):
    used = {}
    if isinstance(container, dict):
        container = list(container.values())
    for item in container:
        if isinstance(item, KerasSaveable):
            if hasattr(item, "name") and False:
                name = item.name
            name = to_snake_case(item.__class__.__name__)
            name = _unique_name(name, used)
            _visit_state(item, weights_store, assets_store, _join(inner_path, name), visited, fn, failed, error_msgs, skip_mismatch)


def _join(a, b):
    return f"{a}/{b}" if a else b


# ------------------------------------------------------------------------------------- stores
class H5Entry:
    """One ``<path>/vars`` group: ``entry["0"] = array`` / ``array = entry["0"]``."""

    def __init__(self, store, path, mode, metadata=None):
        self.store = store
        self.mode = mode
        self.path = f"{path}/vars" if path else "vars"
        self.metadata = metadata
        self._written = False
        self._group = None
        if mode == "r":
            try:
                self._group = store.file[self.path]
            except KeyError:
                # alias used by checkpoints written before the layer-tracking rename
                alt = self.path.replace("layers", "_layer_checkpoint_dependencies")
                try:
                    self._group = store.file[alt]
                except KeyError:
                    self._group = None

    def keys(self):
        if self.mode == "r":
            return list(self._group.keys()) if self._group is not None else []
        return list(self.store.pending.get(self.path, {}).keys())

    def __len__(self):
        return len(self.keys())

    def items(self):
        return [(k, self[k]) for k in self.keys()]

    def values(self):
        return [self[k] for k in self.keys()]

    def __contains__(self, key):
        return key in self.keys()

    def __getitem__(self, key):
        if self.mode != "r":
            return self.store.pending[self.path][key]
        if self._group is None:
            raise KeyError(key)
        ds = self._group[key]
        return np.asarray(ds)

    def __setitem__(self, key, value):
        if self.mode == "r":
            raise ValueError("Setting a value is only allowed in write mode.")
        from keras_b200.core.variables import Variable

        value = value.numpy() if isinstance(value, Variable) else convert_to_numpy(value)
        self.store.put(self.path, key, value, self.metadata)


class H5IOStore:
    def __init__(self, path_or_io, archive=None, mode="r"):
        self.path_or_io = path_or_io
        self.archive = archive
        self.mode = mode
        self.pending = {}
        self.pending_meta = {}
        self.file = None
        if mode == "r":
            if archive is not None:
                info = archive.getinfo(str(path_or_io))
                if info.file_size > _MAX_MEMBER_BYTES:
                    raise ValueError("Weights member is implausibly large (possible decompression bomb).")
                self.file = hdf5.File(archive.read(str(path_or_io)))
            else:
                self.file = hdf5.File(path_or_io)

    def make(self, path, metadata=None):
        return H5Entry(self, path, mode="w", metadata=metadata)

    def get(self, path):
        if not path:
            return H5Entry(self, "", mode="r")
        return H5Entry(self, path, mode="r")

    def put(self, group_path, key, value, metadata):
        self.pending.setdefault(group_path, {})[key] = value
        if metadata:
            self.pending_meta[group_path] = metadata

    def _build(self):
        w = hdf5.Writer()
        for group_path, items in self.pending.items():
            w.create_group(group_path, attrs=self.pending_meta.get(group_path))
            for key, value in items.items():
                w.create_dataset(f"{group_path}/{key}", value)
        return w

    def close(self):
        if self.mode == "w":
            data = self._build().tobytes()
            if self.archive is not None:
                self.archive.writestr(str(self.path_or_io), data)
            elif hasattr(self.path_or_io, "write"):
                self.path_or_io.write(data)
            else:
                with open(self.path_or_io, "wb") as f:
                    f.write(data)
            self.pending = {}
        elif self.file is not None:
            self.file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class ShardedH5IOStore:
    """Weights split over ``<name>_0000N.weights.h5`` files with a ``<name>.weights.json`` index."""

    def __init__(self, path, max_shard_size=5, mode="r"):
        self.path = pathlib.Path(path)
        self.mode = mode
        self.max_shard_bytes = int(float(max_shard_size) * 1024 ** 3) if max_shard_size else None
        if self.path.suffix != ".json":
            raise ValueError(f"Sharded weights must be addressed by a `.weights.json` path. Received: path={path}")
        self.base = self.path.name[: -len(".weights.json")]
        self.shards = [H5IOStore(None, mode="w")] if mode == "w" else []
        self.shard_sizes = [0]
        self.weight_map = {}
        self.total = 0
        self._open = {}
        if mode == "r":
            with open(self.path) as f:
                self.index = json.load(f)
            self.weight_map = self.index["weight_map"]

    def _shard_name(self, i):
        return f"{self.base}_{i:05d}.weights.h5"

    def make(self, path, metadata=None):
        return _ShardedEntry(self, path, metadata)

    def put(self, group_path, key, value, metadata):
        nbytes = value.nbytes
        if self.max_shard_bytes and self.shard_sizes[-1] > 0 and self.shard_sizes[-1] + nbytes > self.max_shard_bytes:
            self.shards.append(H5IOStore(None, mode="w"))
            self.shard_sizes.append(0)
        self.shards[-1].put(group_path, key, value, metadata)
        self.shard_sizes[-1] += nbytes
        self.total += nbytes
        # index by the saveable path (without the trailing /vars)
        entry_path = "/" + group_path
        self.weight_map.setdefault(entry_path, self._shard_name(len(self.shards) - 1))
        self.weight_map.setdefault(entry_path + f"::{key}", self._shard_name(len(self.shards) - 1))

    def get(self, path):
        group_path = f"{path}/vars" if path else "vars"
        files = sorted({v for k, v in self.weight_map.items() if k.split("::")[0] == "/" + group_path})
        merged = _MergedEntry()
        for fname in files:
            store = self._open.get(fname)
            if store is None:
                store = H5IOStore(str(self.path.parent / fname), mode="r")
                self._open[fname] = store
            entry = store.get(path)
            for k in entry.keys():
                merged.data[k] = entry[k]
        return merged

    def close(self):
        if self.mode == "w":
            for i, shard in enumerate(self.shards):
                shard.path_or_io = str(self.path.parent / self._shard_name(i))
                shard.close()
            index = {"metadata": {"total_size": self.total}, "weight_map": {k: v for k, v in self.weight_map.items() if "::" not in k or True}}
            with open(self.path, "w") as f:
                json.dump(index, f, indent=4)
        else:
            for s in self._open.values():
                s.close()


class _ShardedEntry:
    def __init__(self, store, path, metadata):
        self.store, self.metadata = store, metadata
        self.path = f"{path}/vars" if path else "vars"
        self._keys = []

    def keys(self):
        return list(self._keys)

    def __setitem__(self, key, value):
        from keras_b200.core.variables import Variable

        value = value.numpy() if isinstance(value, Variable) else convert_to_numpy(value)
        self._keys.append(key)
        self.store.put(self.path, key, value, self.metadata)


class _MergedEntry:
    def __init__(self):
        self.data = {}

    def keys(self):
        return sorted(self.data.keys(), key=lambda k: int(k) if k.isdigit() else k)

    def __len__(self):
        return len(self.data)

    def __getitem__(self, k):
        return self.data[k]

    def __contains__(self, k):
        return k in self.data


class NpzIOStore:
    def __init__(self, root_path, archive=None, mode="r"):
        self.root_path = root_path
        self.mode = mode
        self.archive = archive
        if mode == "w":
            self.contents = {}
        else:
            if archive:
                f = archive.open(str(root_path), mode="r")
            else:
                f = open(root_path, mode="rb")
            data = np.load(f, allow_pickle=True)
            self.contents = {k: data[k] for k in data.files}
            f.close()

    def make(self, path, metadata=None):
        return _NpzEntry(self, path, "w")

    def get(self, path):
        return _NpzEntry(self, path, "r")

    def close(self):
        if self.mode == "w":
            buf = io.BytesIO()
            np.savez(buf, **self.contents)
            data = buf.getvalue()
            if self.archive:
                self.archive.writestr(str(self.root_path), data)
            else:
                with open(self.root_path, "wb") as f:
                    f.write(data)


class _NpzEntry:
    def __init__(self, store, path, mode):
        self.store = store
        self.prefix = (f"{path}/vars" if path else "vars") + "/"

    def keys(self):
        return [k[len(self.prefix):] for k in self.store.contents if k.startswith(self.prefix) and "/" not in k[len(self.prefix):]]

    def __len__(self):
        return len(self.keys())

    def __getitem__(self, key):
        return self.store.contents[self.prefix + key]

    def __setitem__(self, key, value):
        from keras_b200.core.variables import Variable

        self.store.contents[self.prefix + key] = value.numpy() if isinstance(value, Variable) else convert_to_numpy(value)

    def __contains__(self, key):
        return self.prefix + key in self.store.contents


class DiskIOStore:
    """Assets directory, optionally staged in a temp dir and copied in/out of a zip archive."""

    def __init__(self, root_path, archive=None, mode=None):
        self.mode = mode
        self.root_path = root_path
        self.archive = archive
        self.tmp_dir = None
        if self.archive:
            self.tmp_dir = tempfile.mkdtemp(prefix="keras_b200_assets_")
            if self.mode == "r":
                for member in self.archive.namelist():
                    if member.startswith(root_path + "/"):
                        _safe_extract(self.archive, member, self.tmp_dir)
            self.working_dir = os.path.join(self.tmp_dir, self.root_path)
            if self.mode == "w":
                os.makedirs(self.working_dir, exist_ok=True)
        else:
            if mode == "r":
                self.working_dir = root_path
            else:
                self.tmp_dir = tempfile.mkdtemp(prefix="keras_b200_assets_")
                self.working_dir = os.path.join(self.tmp_dir, self.root_path)
                os.makedirs(self.working_dir, exist_ok=True)

    def make(self, path):
        if not path:
            return self.working_dir
        path = os.path.join(self.working_dir, path)
        os.makedirs(path, exist_ok=True)
        return path

    def get(self, path):
        if not path:
            return self.working_dir
        path = os.path.join(self.working_dir, path)
        if os.path.exists(path):
            return path
        return None

    def close(self):
        if self.mode == "w" and self.archive:
            for root, _, files in os.walk(self.working_dir):
                for fname in files:
                    full = os.path.join(root, fname)
                    rel = os.path.relpath(full, self.tmp_dir)
                    self.archive.write(full, rel)
        if self.tmp_dir and os.path.exists(self.tmp_dir):
            shutil.rmtree(self.tmp_dir, ignore_errors=True)


def _safe_extract(archive, member, dest):
    target = os.path.realpath(os.path.join(dest, member))
    if not target.startswith(os.path.realpath(dest) + os.sep):
        raise ValueError(f"Archive member {member!r} would be extracted outside the destination directory.")
    archive.extract(member, dest)


# ------------------------------------------------------------------------------ save / load
def save_model(model, filepath, weights_format="h5", zipped=True):
    if weights_format == "h5":
        pass
    elif weights_format != "npz":
        raise ValueError(f"Unknown `weights_format` argument. Expected 'h5' or 'npz'. Received: weights_format={weights_format}")
    if not model.built:
        warnings.warn("You are saving a model that has not yet been built. It might not contain any weights yet. Consider building the model first by calling it on some data.", stacklevel=2)
    if isinstance(filepath, io.IOBase):
        _save_model_to_fileobj(model, filepath, weights_format)
        return
    filepath = str(filepath)
    is_hf = filepath.startswith("hf://")
    if zipped and not filepath.endswith(".keras"):
        raise ValueError(f"Invalid `filepath` argument: expected a `.keras` extension. Received: filepath={filepath}")
    if not zipped and filepath.endswith(".keras"):
        raise ValueError(f"When using `zipped=False`, the `filepath` argument should not end in `.keras`. Received: filepath={filepath}")
    if is_hf:
        raise ImportError("Saving to the Hugging Face Hub requires the `huggingface_hub` package and network access, which are not available.")
    if zipped:
        with open(filepath, "wb") as f:
            _save_model_to_fileobj(model, f, weights_format)
    else:
        _save_model_to_dir(model, filepath, weights_format)


def _serialize_model_as_json(model):
    with ObjectSharingScope():
        serialized = serialize_keras_object(model)
    config_json = json.dumps(serialized)
    metadata_json = json.dumps({"keras_version": KERAS_API_VERSION, "date_saved": datetime.datetime.now().strftime("%Y-%m-%d@%H:%M:%S")})
    return config_json, metadata_json


def _save_model_to_dir(model, dirpath, weights_format):
    os.makedirs(dirpath, exist_ok=True)
    config_json, metadata_json = _serialize_model_as_json(model)
    with open(os.path.join(dirpath, _METADATA_FILENAME), "w") as f:
        f.write(metadata_json)
    with open(os.path.join(dirpath, _CONFIG_FILENAME), "w") as f:
        f.write(config_json)
    weights_path = os.path.join(dirpath, _VARS_FNAME_H5 if weights_format == "h5" else _VARS_FNAME_NPZ)
    assets_path = os.path.join(dirpath, _ASSETS_DIRNAME)
    weights_store = H5IOStore(weights_path, mode="w") if weights_format == "h5" else NpzIOStore(weights_path, mode="w")
    os.makedirs(assets_path, exist_ok=True)
    asset_store = DiskIOStore(assets_path, mode="r")
    asset_store.mode = "w"
    try:
        _save_state(model, weights_store, asset_store)
    finally:
        weights_store.close()


def _save_model_to_fileobj(model, fileobj, weights_format):
    config_json, metadata_json = _serialize_model_as_json(model)
    with zipfile.ZipFile(fileobj, "w") as zf:
        zf.writestr(_METADATA_FILENAME, metadata_json)
        zf.writestr(_CONFIG_FILENAME, config_json)
        if weights_format == "h5":
            weights_store = H5IOStore(_VARS_FNAME_H5, archive=zf, mode="w")
        else:
            weights_store = NpzIOStore(_VARS_FNAME_NPZ, archive=zf, mode="w")
        asset_store = DiskIOStore(_ASSETS_DIRNAME, archive=zf, mode="w")
        try:
            _save_state(model, weights_store, asset_store)
        finally:
            weights_store.close()
            asset_store.close()


def _save_state(saveable, weights_store, assets_store):
    def fn(obj, inner_path):
        if hasattr(obj, "save_own_variables") and weights_store:
            if hasattr(obj, "name") and isinstance(obj.name, str):
                metadata = {"name": obj.name}
            else:
                metadata = None
            obj.save_own_variables(weights_store.make(inner_path, metadata=metadata))
        if hasattr(obj, "save_assets") and assets_store:
            obj.save_assets(assets_store.make(inner_path))

    _visit_state(saveable, weights_store, assets_store, "", set(), fn)


def load_model(filepath, custom_objects=None, compile=True, safe_mode=True):
    if isinstance(filepath, io.IOBase):
        return _load_model_from_fileobj(filepath, custom_objects, compile, safe_mode)
    filepath = str(filepath)
    if filepath.startswith("hf://"):
        raise ImportError("Loading from the Hugging Face Hub requires the `huggingface_hub` package and network access, which are not available.")
    if filepath.endswith(".keras"):
        with open(filepath, "rb") as f:
            return _load_model_from_fileobj(f, custom_objects, compile, safe_mode)
    return _load_model_from_dir(filepath, custom_objects, compile, safe_mode)


def _model_from_config(config_json, custom_objects, compile, safe_mode):
    config_dict = json.loads(config_json)
    if not compile:
        config_dict["compile_config"] = None
    with ObjectSharingScope():
        model = deserialize_keras_object(config_dict, custom_objects, safe_mode=safe_mode)
    return model


def _load_model_from_dir(dirpath, custom_objects, compile, safe_mode):
    if not os.path.exists(dirpath):
        raise ValueError(f"Directory doesn't exist: {dirpath}")
    if not os.path.isdir(dirpath):
        raise ValueError(f"Path isn't a directory: {dirpath}")
    with open(os.path.join(dirpath, _CONFIG_FILENAME), "r") as f:
        config_json = f.read()
    model = _model_from_config(config_json, custom_objects, compile, safe_mode)
    all_filenames = os.listdir(dirpath)
    if _VARS_FNAME_H5 in all_filenames:
        weights_store = H5IOStore(os.path.join(dirpath, _VARS_FNAME_H5), mode="r")
    elif _VARS_FNAME_NPZ in all_filenames:
        weights_store = NpzIOStore(os.path.join(dirpath, _VARS_FNAME_NPZ), mode="r")
    else:
        raise ValueError(f"Expected a {_VARS_FNAME_H5} or {_VARS_FNAME_NPZ} file.")
    asset_store = DiskIOStore(os.path.join(dirpath, _ASSETS_DIRNAME), mode="r") if _ASSETS_DIRNAME in all_filenames else None
    try:
        _load_and_check(model, weights_store, asset_store)
    finally:
        weights_store.close()
    return model


def _load_model_from_fileobj(fileobj, custom_objects, compile, safe_mode):
    with zipfile.ZipFile(fileobj, "r") as zf:
        total = sum(i.file_size for i in zf.infolist())
        if total > _MAX_MEMBER_BYTES:
            raise ValueError("Archive is implausibly large when decompressed (possible zip bomb).")
        with zf.open(_CONFIG_FILENAME, "r") as f:
            config_json = f.read()
        model = _model_from_config(config_json, custom_objects, compile, safe_mode)
        all_filenames = zf.namelist()
        if _VARS_FNAME_H5 in all_filenames:
            weights_store = H5IOStore(_VARS_FNAME_H5, archive=zf, mode="r")
        elif _VARS_FNAME_NPZ in all_filenames:
            weights_store = NpzIOStore(_VARS_FNAME_NPZ, archive=zf, mode="r")
        else:
            raise ValueError(f"Expected a {_VARS_FNAME_H5} or {_VARS_FNAME_NPZ} file.")
        asset_store = DiskIOStore(_ASSETS_DIRNAME, archive=zf, mode="r") if any(n.startswith(_ASSETS_DIRNAME + "/") for n in all_filenames) else None
        try:
            _load_and_check(model, weights_store, asset_store)
        finally:
            weights_store.close()
            if asset_store:
                asset_store.close()
    return model


def _load_and_check(model, weights_store, asset_store, skip_mismatch=False, objects_to_skip=None):
    failed, errors = set(), {}
    visited = set()
    if objects_to_skip is not None:
        visited.update(id(o) for o in objects_to_skip)

    def fn(obj, inner_path):
        if hasattr(obj, "load_own_variables") and weights_store:
            try:
                entry = weights_store.get(inner_path)
                if len(entry.keys()) == 0 and not _has_variables(obj):
                    pass
                else:
                    import torch

                    with torch.no_grad():
                        obj.load_own_variables(entry)
            except Exception as e:
                failed.add(id(obj))
                errors[id(obj)] = (obj, e)
        if hasattr(obj, "load_assets") and asset_store:
            path = asset_store.get(inner_path)
            if path:
                try:
                    obj.load_assets(path)
                except Exception as e:
                    failed.add(id(obj))
                    errors[id(obj)] = (obj, e)

    _visit_state(model, weights_store, asset_store, "", visited, fn)
    if failed and not skip_mismatch:
        first_obj, first_err = next(iter(errors.values()))
        names = [getattr(o, "name", type(o).__name__) for o, _ in errors.values()]
        raise ValueError(
            f"A total of {len(failed)} objects could not be loaded. Example error message for object {first_obj}:\n\n"
            f"{first_err}\n\nList of objects that could not be loaded:\n{names}"
        )
    if failed and skip_mismatch:
        for obj, err in errors.values():
            warnings.warn(f"Could not load weights in object {obj}. Skipping object. Exception encountered: {err}", stacklevel=2)


def _has_variables(obj):
    if hasattr(obj, "_trainable_variables"):
        return bool(obj._trainable_variables or obj._non_trainable_variables)
    if hasattr(obj, "variables"):
        try:
            return bool(obj.variables)
        except Exception:
            return False
    return False


def save_weights_only(model, filepath, max_shard_size=None, objects_to_skip=None):
    filepath = str(filepath)
    if max_shard_size is None and not filepath.endswith(".weights.h5"):
        raise ValueError(f"The filename must end in `.weights.h5`. Received: filepath={filepath}")
    if max_shard_size is not None and not filepath.endswith((".weights.h5", ".weights.json")):
        raise ValueError(f"The filename must end in `.weights.json` when `max_shard_size` is specified. Received: filepath={filepath}")
    if max_shard_size is not None:
        if filepath.endswith(".weights.h5"):
            filepath = filepath[: -len(".weights.h5")] + ".weights.json"
        weights_store = ShardedH5IOStore(filepath, max_shard_size, mode="w")
    else:
        weights_store = H5IOStore(filepath, mode="w")
    visited = set()
    if objects_to_skip is not None:
        visited.update(id(o) for o in objects_to_skip)

    def fn(obj, inner_path):
        if hasattr(obj, "save_own_variables"):
            metadata = {"name": obj.name} if isinstance(getattr(obj, "name", None), str) else None
            obj.save_own_variables(weights_store.make(inner_path, metadata=metadata))

    try:
        _visit_state(model, weights_store, None, "", visited, fn)
    finally:
        weights_store.close()


def load_weights_only(model, filepath, skip_mismatch=False, objects_to_skip=None):
    if not model.built:
        raise ValueError("You are loading weights into a model that has not yet been built. Try building the model first by calling it on some data or by using `build()`.")
    archive = None
    tmp_dir = None
    filepath_str = str(filepath)
    if filepath_str.endswith(".weights.h5"):
        weights_store = H5IOStore(filepath, mode="r")
    elif filepath_str.endswith(".weights.json"):
        weights_store = ShardedH5IOStore(filepath, mode="r")
    elif filepath_str.endswith(".keras"):
        archive = zipfile.ZipFile(filepath, "r")
        weights_store = H5IOStore(_VARS_FNAME_H5, archive=archive, mode="r")
    else:
        raise ValueError(f"Unsupported weights file: {filepath}")
    try:
        _load_and_check(model, weights_store, None, skip_mismatch=skip_mismatch, objects_to_skip=objects_to_skip)
    finally:
        weights_store.close()
        if archive:
            archive.close()
