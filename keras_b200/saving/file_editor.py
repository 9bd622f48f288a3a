"""``KerasFileEditor``: inspect, compare, edit and re-save the weights of a ``.keras`` / ``.weights.h5`` file
(keras/src/saving/file_editor.py:39-922).

``weights_dict`` mirrors the H5 tree with the ``vars`` level folded away: ``{"layers": {"dense": {"0": array, "1": array}}}``.
"""

import collections
import json
import pprint
import zipfile

import numpy as np

from keras_b200.core.export_registry import keras_export
from keras_b200.saving import hdf5, saving_lib
from keras_b200.utils import io_utils


def _nested():
    return collections.OrderedDict()


@keras_export("keras.saving.KerasFileEditor")
class KerasFileEditor:
    def __init__(self, filepath):
        self.filepath = filepath
        self.metadata = self.config = self.model = None
        filepath = str(filepath)
        if filepath.endswith(".keras"):
            with zipfile.ZipFile(filepath, "r") as zf:
                self.config = json.loads(zf.read("config.json"))
                self.metadata = json.loads(zf.read("metadata.json"))
                h5 = hdf5.File(zf.read("model.weights.h5"))
        elif filepath.endswith(".weights.h5"):
            h5 = hdf5.File(filepath)
        else:
            raise ValueError(f"Invalid filename: expected a `.keras` `.weights.h5` extension. Received: filepath={filepath}")
        self.weights_dict, self.object_metadata = self._extract_weights_from_store(h5)
        h5.close()
        io_utils.print_msg(self._generate_filepath_info())
        if self.metadata is not None:
            io_utils.print_msg(self._generate_metadata_info())

    # -- reading -------------------------------------------------------------------------
    def _extract_weights_from_store(self, data, metadata=None, inner_path=""):
        metadata = metadata if metadata is not None else {}
        result = _nested()
        for key in data.keys():
            inner = f"{inner_path}/{key}"
            value = data[key]
            if isinstance(value, hdf5.Group):
                if len(value) == 0 and key != "vars":
                    continue
                if key == "vars":
                    name = value.attrs.get("name") if hasattr(value, "attrs") else None
                    if name is not None and inner_path:
                        metadata[inner_path] = {"name": name}
                    for k in value.keys():
                        result[k] = np.asarray(value[k])
                else:
                    sub, metadata = self._extract_weights_from_store(value, metadata, inner)
                    if sub:
                        result[key] = sub
            else:
                result[key] = np.asarray(value)
        return result, metadata

    # -- reports -------------------------------------------------------------------------
    def _generate_filepath_info(self):
        return f"Keras model file '{self.filepath}'"

    def _generate_config_info(self):
        return pprint.pformat(self.config)

    def _generate_metadata_info(self):
        return f"Saved with Keras {self.metadata['keras_version']} - date: {self.metadata['date_saved']}"

    def _weights_lines(self, weights_dict, indent=0, prefix=""):
        lines = []
        for key, value in weights_dict.items():
            if isinstance(value, dict):
                lines.append(" " * indent + f"{prefix}{key}")
                lines += self._weights_lines(value, indent + 4)
            else:
                lines.append(" " * indent + f"{key}: shape={tuple(value.shape)}, dtype={value.dtype}")
        return lines

    def summary(self):
        """Print the weight structure of the opened file."""
        io_utils.print_msg("Weights structure")
        io_utils.print_msg("\n".join(self._weights_lines(self.weights_dict)))

    def compare(self, reference_model):
        """Check the file against ``reference_model``; returns ``{"status", "error_count", "match_count"}``."""
        io_utils.print_msg("Running comparison")
        ref_spec = get_weight_spec_of_saveable(reference_model)

        def walk(target, ref, inner_path, target_name, ref_name, checked):
            errors = matches = 0
            for key, ref_val in ref.items():
                path = f"{inner_path}/{key}"
                if path in checked:
                    continue
                if key not in target:
                    errors += 1
                    checked.add(path)
                    kind = "Object" if isinstance(ref_val, dict) else "Weight"
                    io_utils.print_msg(f"...{kind} {path} present in {ref_name}, missing from {target_name}")
                    if isinstance(ref_val, dict):
                        io_utils.print_msg(f"    In {ref_name}, {path} contains the following keys: {list(ref_val.keys())}")
                elif isinstance(ref_val, dict):
                    e, m = walk(target[key], ref_val, path, target_name, ref_name, checked)
                    errors += e
                    matches += m
                elif tuple(target[key].shape) != tuple(ref_val.shape):
                    errors += 1
                    checked.add(path)
                    io_utils.print_msg(f"...Weight shape mismatch for {path}\n    In {ref_name}: shape={tuple(ref_val.shape)}\n    In {target_name}: shape={tuple(target[key].shape)}")
                else:
                    matches += 1
            return errors, matches

        checked = set()
        errors, matches = walk(self.weights_dict, ref_spec, "", "saved file", "reference model", checked)
        e2, _ = walk(ref_spec, self.weights_dict, "", "reference model", "saved file", checked)
        errors += e2
        io_utils.print_msg("─────────────────────")
        if errors == 0:
            io_utils.print_msg("Comparison successful: saved file is compatible with the reference model")
            io_utils.print_msg(f"    Found {matches} matching weight{'' if matches == 1 else 's'}")
        else:
            io_utils.print_msg(f"Found {errors} error{'' if errors == 1 else 's'}: saved file is not compatible with the reference model")
        return {"status": "success" if errors == 0 else "error", "error_count": errors, "match_count": matches}

    # -- editing -------------------------------------------------------------------------
    def _edit_object(self, edit_fn, source_name, target_name=None):
        if target_name is not None and "/" in target_name:
            raise ValueError(f"Argument `target_name` should be a leaf name, not a full path name. Received: target_name='{target_name}'")
        if "/" in source_name:
            elements = source_name.split("/")
            d = self.weights_dict
            for e in elements[:-1]:
                if e not in d:
                    raise ValueError(f"Path '{source_name}' not found in model.")
                d = d[e]
            if elements[-1] not in d:
                raise ValueError(f"Path '{source_name}' not found in model.")
            edit_fn(d, source_name=elements[-1], target_name=target_name)
        else:
            def count(d, name, n=0):
                for k, v in d.items():
                    if isinstance(v, dict):
                        if k == name:
                            n += 1
                        n += count(v, name, 0)
                return n

            occurrences = count(self.weights_dict, source_name)
            if occurrences > 1:
                raise ValueError(f"Name '{source_name}' occurs more than once in the model; try passing a complete path")
            if occurrences == 0:
                raise ValueError(f"Source name '{source_name}' does not appear in the model. Use `editor.weights_summary()` to list all objects.")

            def edit(d):
                for k, v in list(d.items()):
                    if isinstance(v, dict):
                        if k == source_name:
                            edit_fn(d, source_name=source_name, target_name=target_name)
                            return True
                        if edit(v):
                            return True
                return False

            edit(self.weights_dict)

    def rename_object(self, object_name, new_name):
        def fn(d, source_name, target_name):
            items = [(target_name if k == source_name else k, v) for k, v in d.items()]
            d.clear()
            d.update(items)

        self._edit_object(fn, object_name, new_name)

    def delete_object(self, object_name):
        def fn(d, source_name, target_name=None):
            d.pop(source_name)

        self._edit_object(fn, object_name)

    def add_object(self, object_path, weights):
        if not isinstance(weights, dict):
            raise ValueError(f"Argument `weights` should be a dict where keys are weight names (usually '0', '1', etc.) and values are NumPy arrays. Received: type(weights)={type(weights)}")
        if "/" in object_path:
            elements = object_path.split("/")
            d = self.weights_dict
            for e in elements[:-1]:
                if e not in d:
                    raise ValueError(f"Path '{'/'.join(elements[:-1])}' not found in model.")
                d = d[e]
            d[elements[-1]] = _nested()
            d[elements[-1]].update(weights)
        else:
            self.weights_dict[object_path] = _nested()
            self.weights_dict[object_path].update(weights)

    def delete_weight(self, object_name, weight_name):
        def fn(d, source_name, target_name=None):
            if weight_name not in d[source_name]:
                raise ValueError(f"Weight {weight_name} not found in object {object_name}. Weights found: {list(d[source_name].keys())}")
            d[source_name].pop(weight_name)

        self._edit_object(fn, object_name)

    def add_weights(self, object_name, weights):
        if not isinstance(weights, dict):
            raise ValueError(f"Argument `weights` should be a dict where keys are weight names (usually '0', '1', etc.) and values are NumPy arrays. Received: type(weights)={type(weights)}")

        def fn(d, source_name, target_name=None):
            d[source_name].update(weights)

        self._edit_object(fn, object_name)

    # -- writing -------------------------------------------------------------------------
    def save(self, filepath):
        filepath = str(filepath)
        if not filepath.endswith(".weights.h5"):
            raise ValueError(f"Invalid `filepath` argument: expected a `.weights.h5` extension. Received: filepath={filepath}")
        writer = hdf5.Writer()

        def write(d, inner_path):
            arrays = {k: v for k, v in d.items() if not isinstance(v, dict)}
            if arrays and inner_path:
                meta = self.object_metadata.get("/" + inner_path)
                writer.create_group(f"{inner_path}/vars", attrs=meta)
                for k, v in arrays.items():
                    writer.create_dataset(f"{inner_path}/vars/{k}", np.asarray(v))
            elif arrays:
                writer.create_group("vars")
                for k, v in arrays.items():
                    writer.create_dataset(f"vars/{k}", np.asarray(v))
            for k, v in d.items():
                if isinstance(v, dict):
                    write(v, f"{inner_path}/{k}" if inner_path else k)

        write(self.weights_dict, "")
        writer.save(filepath)

    def resave_weights(self, filepath):
        self.save(filepath)


def get_weight_spec_of_saveable(saveable):
    """Nested ``{path: {weight index: array}}`` that saving ``saveable`` would produce."""
    store = saving_lib.H5IOStore(None, mode="w")
    saving_lib._save_state(saveable, store, None)
    spec = _nested()
    for group_path, items in store.pending.items():
        parts = [p for p in group_path.split("/") if p]
        if parts and parts[-1] == "vars":
            parts = parts[:-1]
        d = spec
        for p in parts:
            d = d.setdefault(p, _nested())
        for k, v in items.items():
            d[k] = np.asarray(v)
    return spec
