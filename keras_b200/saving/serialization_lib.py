"""Object (de)serialization to JSON-able dicts.

Schema of keras/src/saving/serialization_lib.py:66-905: ``{module, class_name, config,
registered_name[, build_config, compile_config, shared_object_id]}``; special class names
``__tensor__ __numpy__ __bytes__ __slice__ __ellipsis__ __keras_tensor__ __lambda__``; public
symbols are identified by their canonical ``keras.*`` export name so that files interchange with
reference Keras; safe mode blocks lambdas.
"""

import codecs
import importlib
import inspect
import marshal
import os
import types
import warnings

import numpy as np
import torch

from keras_b200.core import global_state
from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.export_registry import get_name_from_symbol, get_symbol_from_name, keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.ops.operation import KerasSaveable
from keras_b200.saving import object_registration

PLAIN_TYPES = (str, int, float, bool)
BUILTIN_MODULES = frozenset({"activations", "constraints", "initializers", "losses", "metrics", "optimizers", "regularizers"})
# Private module paths that reference Keras writes into configs, mapped to public namespaces.
_PRIVATE_MODULE_PREFIXES = ("keras.src.", "keras_b200.")


class SerializableDict:
    def __init__(self, **config):
        self.config = config

    def serialize(self):
        return serialize_keras_object(self.config)


class SafeModeScope:
    def __init__(self, safe_mode=True):
        self.safe_mode = safe_mode

    def __enter__(self):
        self.original_value = in_safe_mode()
        global_state.set_global_attribute("safe_mode_saving", self.safe_mode)

    def __exit__(self, *args, **kwargs):
        global_state.set_global_attribute("safe_mode_saving", self.original_value)


@keras_export("keras.config.enable_unsafe_deserialization")
def enable_unsafe_deserialization():
    global_state.set_global_attribute("safe_mode_saving", False)


def in_safe_mode():
    return global_state.get_global_attribute("safe_mode_saving")


class ObjectSharingScope:
    def __enter__(self):
        global_state.set_global_attribute("shared_objects/id_to_obj_map", {})
        global_state.set_global_attribute("shared_objects/id_to_config_map", {})

    def __exit__(self, *args, **kwargs):
        global_state.set_global_attribute("shared_objects/id_to_obj_map", None)
        global_state.set_global_attribute("shared_objects/id_to_config_map", None)


def get_shared_object(obj_id):
    m = global_state.get_global_attribute("shared_objects/id_to_obj_map")
    return m.get(obj_id) if m is not None else None


def record_object_after_serialization(obj, config):
    if config.get("module") == "__main__":
        config["module"] = None
    m = global_state.get_global_attribute("shared_objects/id_to_config_map")
    if m is None:
        return
    obj_id = int(id(obj))
    if obj_id not in m:
        m[obj_id] = config
    else:
        config["shared_object_id"] = obj_id
        m[obj_id]["shared_object_id"] = obj_id


def record_object_after_deserialization(obj, obj_id):
    m = global_state.get_global_attribute("shared_objects/id_to_obj_map")
    if m is not None:
        m[obj_id] = obj


def func_dump(func):
    if os.name == "nt":
        raw = marshal.dumps(func.__code__).replace(b"\\", b"/")
        code = codecs.encode(raw, "base64").decode("ascii")
    else:
        code = codecs.encode(marshal.dumps(func.__code__), "base64").decode("ascii")
    defaults = func.__defaults__
    closure = tuple(c.cell_contents for c in func.__closure__) if func.__closure__ else None
    return code, defaults, closure


def func_load(code, defaults=None, closure=None, globs=None):
    if isinstance(code, (tuple, list)):
        code, defaults, closure = code
        if isinstance(defaults, list):
            defaults = tuple(defaults)

    def ensure_value_to_cell(value):
        def dummy_fn():
            value  # noqa: B018

        cell_value = dummy_fn.__closure__[0]
        if not isinstance(value, type(cell_value)):
            return cell_value
        return value

    if closure is not None:
        closure = tuple(ensure_value_to_cell(_) for _ in closure)
    try:
        raw = codecs.decode(code.encode("ascii"), "base64")
    except (UnicodeEncodeError, ValueError):
        raw = code.encode("raw_unicode_escape")
    code_obj = marshal.loads(raw)
    if globs is None:
        globs = globals()
    return types.FunctionType(code_obj, globs, name=code_obj.co_name, argdefs=defaults, closure=closure)


@keras_export(["keras.saving.serialize_keras_object", "keras.utils.serialize_keras_object"])
def serialize_keras_object(obj):
    if obj is None or isinstance(obj, PLAIN_TYPES):
        return obj
    if isinstance(obj, (list, tuple)):
        items = [serialize_keras_object(x) for x in obj]
        return tuple(items) if isinstance(obj, tuple) else items
    if isinstance(obj, dict):
        return serialize_dict(obj)
    if isinstance(obj, bytes):
        return {"class_name": "__bytes__", "config": {"value": obj.decode("utf-8")}}
    if isinstance(obj, slice):
        return {"class_name": "__slice__", "config": {"start": serialize_keras_object(obj.start), "stop": serialize_keras_object(obj.stop), "step": serialize_keras_object(obj.step)}}
    if obj is Ellipsis:
        return {"class_name": "__ellipsis__", "config": {}}
    if isinstance(obj, KerasTensor):
        history = getattr(obj, "_keras_history", None)
        if history:
            history = list(history)
            history[0] = history[0].name
        return {"class_name": "__keras_tensor__", "config": {"shape": obj.shape, "dtype": obj.dtype, "keras_history": history}}
    if isinstance(obj, torch.Tensor):
        from keras_b200.core.tensor import convert_to_numpy

        arr = convert_to_numpy(obj)
        return {"class_name": "__tensor__", "config": {"value": arr.astype("float32").tolist() if arr.dtype.name == "bfloat16" else arr.tolist(), "dtype": standardize_dtype(obj.dtype)}}
    if isinstance(obj, torch.dtype):
        return standardize_dtype(obj)
    if type(obj).__module__ == np.__name__:
        if isinstance(obj, np.ndarray) and obj.ndim > 0:
            return {"class_name": "__numpy__", "config": {"value": obj.tolist(), "dtype": standardize_dtype(obj.dtype)}}
        return obj.item()
    if isinstance(obj, types.FunctionType) and obj.__name__ == "<lambda>":
        warnings.warn(
            "The object being serialized includes a `lambda`. This is unsafe. In order to reload the object, you will have "
            "to pass `safe_mode=False` to the loading function. Please avoid using `lambda` in the future, and use named "
            "Python functions instead.", stacklevel=2)
        return {"class_name": "__lambda__", "config": {"value": func_dump(obj)}}
    if isinstance(obj, (types.FunctionType, types.BuiltinFunctionType)) or (callable(obj) and hasattr(obj, "__name__") and not hasattr(obj, "get_config") and not inspect.isclass(obj)):
        return _serialize_function(obj)

    inner = _class_config(obj)
    cfg = _public_class_config(obj.__class__, inner)
    if cfg is None:
        module = obj.__class__.__module__
        registered = None if module == "builtins" else object_registration.get_registered_name(obj.__class__)
        cfg = {"module": module, "class_name": obj.__class__.__name__, "config": inner, "registered_name": registered}
    _add_build_and_compile_config(obj, cfg)
    record_object_after_serialization(obj, cfg)
    return cfg


def _serialize_function(fn):
    name = get_name_from_symbol(fn)
    fn_name = fn.__name__
    if name:
        parts = name.split(".")
        return {"module": ".".join(parts[:-1]), "class_name": "function", "config": parts[-1], "registered_name": parts[-1]}
    registered = object_registration.GLOBAL_CUSTOM_NAMES.get(fn) if _hashable(fn) else None
    module = getattr(fn, "__module__", None)
    if module == "__main__":
        module = None
    return {"module": module, "class_name": "function", "config": registered or fn_name, "registered_name": registered or fn_name}


def _hashable(x):
    try:
        hash(x)
        return True
    except TypeError:
        return False


def _class_config(obj):
    if hasattr(obj, "get_config"):
        config = obj.get_config()
        if not isinstance(config, dict):
            raise TypeError(f"The `get_config()` method of {obj} should return a dict. It returned: {config}")
        return serialize_dict(config)
    if hasattr(obj, "__name__"):
        return object_registration.get_registered_name(obj)
    raise TypeError(f"Cannot serialize object {obj} of type {type(obj)}. To be serializable, a class must implement the `get_config()` method.")


def _public_class_config(cls, inner_config):
    if cls.__name__ == "Functional" and cls.__module__.endswith("models.functional"):
        # a model built as `keras.Model(inputs, outputs)`: the reference names its (unexported) class by module path, and
        # that is the only spelling it accepts back (keras/src/models/functional.py, keras/src/saving/serialization_lib.py:157-313)
        return {"module": "keras.src.models.functional", "class_name": "Functional", "config": inner_config, "registered_name": "Functional"}
    api_name = get_name_from_symbol(cls)
    if api_name is None:
        registered = object_registration.GLOBAL_CUSTOM_NAMES.get(cls)
        if registered is None:
            return None
        return {"module": cls.__module__, "class_name": cls.__name__, "config": inner_config, "registered_name": registered}
    parts = api_name.split(".")
    return {"module": ".".join(parts[:-1]), "class_name": parts[-1], "config": inner_config, "registered_name": None}


def _add_build_and_compile_config(obj, config):
    if hasattr(obj, "get_build_config"):
        build_config = obj.get_build_config()
        if build_config is not None:
            config["build_config"] = serialize_dict(build_config)
    if hasattr(obj, "get_compile_config"):
        compile_config = obj.get_compile_config()
        if compile_config is not None:
            config["compile_config"] = serialize_dict(compile_config)


def serialize_dict(obj):
    return {key: serialize_keras_object(value) for key, value in obj.items()}


@keras_export(["keras.saving.deserialize_keras_object", "keras.utils.deserialize_keras_object"])
def deserialize_keras_object(config, custom_objects=None, safe_mode=True, **kwargs):
    safe_scope_arg = in_safe_mode()
    safe_mode = safe_scope_arg if safe_scope_arg is not None else safe_mode
    module_objects = kwargs.pop("module_objects", None)
    custom_objects = custom_objects or {}
    scoped = global_state.get_global_attribute("custom_objects_scope_dict", {})
    custom_objects = {**object_registration.GLOBAL_CUSTOM_OBJECTS, **scoped, **custom_objects}

    if config is None or isinstance(config, PLAIN_TYPES):
        if isinstance(config, str) and module_objects is not None and config in module_objects:
            obj = module_objects[config]
            return obj
        if isinstance(config, str) and config in custom_objects:
            return custom_objects[config]
        return config
    if isinstance(config, (list, tuple)):
        return [deserialize_keras_object(x, custom_objects=custom_objects, safe_mode=safe_mode) for x in config]
    if module_objects is not None:
        inner_config, fn_name, cls = None, None, None
        if isinstance(config, dict):
            if "config" in config:
                inner_config = config["config"]
            if "class_name" not in config:
                raise ValueError(f"Unknown `config` as a `dict`, config={config}")
            if custom_objects and (config["class_name"] in custom_objects or config.get("registered_name") in custom_objects or (isinstance(inner_config, str) and inner_config in custom_objects)):
                pass
            elif config["class_name"] == "function":
                fn_name = inner_config
                if fn_name in module_objects:
                    return module_objects[fn_name]
            elif config["class_name"] in module_objects and not (config.get("module") or "").startswith("keras.") or (config["class_name"] in module_objects and config.get("module") is None):
                cls = module_objects[config["class_name"]]
                if inspect.isclass(cls):
                    with object_registration.CustomObjectScope(custom_objects), SafeModeScope(safe_mode):
                        return cls.from_config(inner_config)
                return cls
    if not isinstance(config, dict):
        raise TypeError(f"Could not parse config: {config}")
    if "class_name" not in config or "config" not in config:
        return {key: deserialize_keras_object(value, custom_objects=custom_objects, safe_mode=safe_mode) for key, value in config.items()}

    class_name = config["class_name"]
    inner_config = config["config"] if config["config"] is not None else {}
    if class_name == "__keras_tensor__":
        obj = KerasTensor(inner_config["shape"], dtype=inner_config["dtype"])
        obj._pre_serialization_keras_history = inner_config["keras_history"]
        return obj
    if class_name == "__tensor__":
        from keras_b200.core.tensor import convert_to_tensor

        return convert_to_tensor(np.asarray(inner_config["value"]), dtype=inner_config["dtype"])
    if class_name == "__numpy__":
        return np.array(inner_config["value"], dtype=inner_config["dtype"])
    if class_name == "__bytes__":
        return inner_config["value"].encode("utf-8")
    if class_name == "__ellipsis__":
        return Ellipsis
    if class_name == "__slice__":
        return slice(*(deserialize_keras_object(inner_config[k], custom_objects=custom_objects, safe_mode=safe_mode) for k in ("start", "stop", "step")))
    if class_name == "__lambda__":
        if safe_mode:
            raise ValueError(
                "Requested the deserialization of a Python lambda. This carries a potential risk of arbitrary code execution "
                "and thus it is disallowed by default. If you trust the source of the artifact, you can override this error by "
                "passing `safe_mode=False` to the loading function, or calling `keras.config.enable_unsafe_deserialization()`."
            )
        return func_load(inner_config["value"])
    if class_name == "__typespec__":
        raise ValueError("TensorFlow TypeSpec objects cannot be deserialized by this framework.")

    module = config.get("module", None)
    registered_name = config.get("registered_name", class_name)
    if class_name == "function":
        fn_name = inner_config
        if not isinstance(fn_name, str):
            raise TypeError(f"Expected 'config' to be a non-null str for a function classname,\ninstead got {type(fn_name)}\nFull config: {config}")
        return _retrieve(fn_name, registered_name, module, "function", config, custom_objects)
    if not isinstance(inner_config, dict):
        raise TypeError(f"Expected 'config' to be a dict for {class_name},\ninstead got {type(inner_config)}\nFull config: {config}")
    if "shared_object_id" in config:
        obj = get_shared_object(config["shared_object_id"])
        if obj is not None:
            return obj
    cls = _retrieve(class_name, registered_name, module, "class", config, custom_objects)
    if isinstance(cls, types.FunctionType):
        return cls
    if not hasattr(cls, "from_config"):
        raise TypeError(f"Unable to reconstruct an instance of '{class_name}' because the class is missing a `from_config()` method. Full object config: {config}")
    with object_registration.CustomObjectScope(custom_objects), SafeModeScope(safe_mode):
        try:
            instance = cls.from_config(inner_config)
        except TypeError as e:
            raise TypeError(
                f"{cls} could not be deserialized properly. Please ensure that components that are Python object instances "
                "(layers, models, etc.) returned by `get_config()` are explicitly deserialized in the model's `from_config()` "
                f"method.\n\nconfig={config}.\n\nException encountered: {e}"
            )
        build_config = config.get("build_config", None)
        if build_config and not instance.built:
            instance.build_from_config(build_config)
            instance.built = True
        compile_config = config.get("compile_config", None)
        if compile_config:
            instance.compile_from_config(compile_config)
            instance.compiled = True
    if "shared_object_id" in config:
        record_object_after_deserialization(instance, config["shared_object_id"])
    return instance


# Packages whose modules may be imported while resolving a config.  Anything else has to be registered
# (`register_keras_serializable`) or passed in `custom_objects`: a model file must never be able to make the loader import
# a module of its choosing (the reference draws the same line, keras/src/saving/serialization_lib.py:880-891).
_IMPORTABLE_PACKAGES = frozenset({"keras_b200", "keras_hub", "keras_cv", "keras_nlp"})


def _lookup_public(module, name):
    """Symbol behind a `keras...` module path, public (`keras.layers`) or private to the reference (`keras.src...`)."""
    obj = get_symbol_from_name(f"{module}.{name}")
    if obj is None and module.startswith("keras.src."):
        obj = _resolve_private(module, name)
    return obj


def _retrieve(name, registered_name, module, obj_type, full_config, custom_objects):
    # 1. objects the caller vouches for: `custom_objects`, the custom-object scope, the global registry
    key = name if obj_type == "function" else registered_name
    if key is not None and key in custom_objects:
        return custom_objects[key]
    if obj_type == "class" and name in custom_objects and registered_name in (None, name):
        return custom_objects[name]
    # 2. this framework's own symbols, addressed by their Keras names
    if module and (module == "keras" or module.startswith("keras.")):
        obj = _lookup_public(module, name)
        if obj is not None:
            return obj
    if obj_type == "function":
        if module in (None, "builtins"):
            for area in BUILTIN_MODULES:
                obj = get_symbol_from_name(f"keras.{area}.{name}")
                if obj is not None:
                    return obj
        # files written before registered names were stored for functions carry the bare name only
        for custom_name, custom_object in custom_objects.items():
            if custom_name.endswith(f">{name}"):
                return custom_object
    # 3. classes inside allow-listed packages, and only savable ones
    if module and obj_type == "class" and module.split(".", 1)[0] in _IMPORTABLE_PACKAGES:
        try:
            candidate = vars(importlib.import_module(module)).get(name)
        except ModuleNotFoundError:
            raise TypeError(f"Could not deserialize {obj_type} '{name}' because its parent module {module} cannot be imported. Full object config: {full_config}")
        if isinstance(candidate, type) and issubclass(candidate, KerasSaveable):
            return candidate
        raise TypeError(f"Could not deserialize '{module}.{name}' because it is not a KerasSaveable subclass")
    raise TypeError(
        f"Could not locate {obj_type} '{name}'. Make sure custom classes and functions are decorated with "
        "`@keras.saving.register_keras_serializable()`. If they are already decorated, make sure they are all imported so that "
        f"the decorator is run before trying to load them. Full object config: {full_config}"
    )


def _resolve_private(module, name):
    if name == "Functional" and module.endswith("models.functional"):
        from keras_b200.models.functional import Functional

        return Functional
    parts = module.split(".")
    if len(parts) >= 3:
        area = parts[2]
        if area == "backend" and "optimizers" in parts:
            area = "optimizers"
        for ns in (area, "layers", "optimizers", "losses", "metrics", "models", "initializers", "regularizers", "constraints", "quantizers", "dtype_policies"):
            obj = get_symbol_from_name(f"keras.{ns}.{name}")
            if obj is not None:
                return obj
        if area == "ops":
            obj = get_symbol_from_name(f"keras.ops.{name}__op")
            if obj is not None:
                return obj
        obj = get_symbol_from_name(f"keras.{name}")
        if obj is not None:
            return obj
    return None
