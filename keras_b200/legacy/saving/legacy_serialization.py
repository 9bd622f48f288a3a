"""Keras 2 style (de)serialisation: ``{"class_name": ..., "config": ...}`` dicts without module paths, tuples encoded
as ``{"class_name": "__tuple__", "items": [...]}`` in JSON (keras/src/legacy/saving/{serialization,json_utils,
saving_utils}.py)."""

import inspect
import json

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export
from keras_b200.saving import object_registration, serialization_lib


def decode_json(json_string):
    def hook(obj):
        if isinstance(obj, dict) and obj.get("class_name") == "__tuple__" and "items" in obj:
            return tuple(obj["items"])
        if isinstance(obj, dict) and obj.get("class_name") == "TensorShape" and "items" in obj:
            return tuple(obj["items"]) if obj["items"] is not None else None
        return obj

    return json.loads(json_string, object_hook=hook)


@keras_export(["keras.legacy.saving.serialize_keras_object", "keras.utils.legacy.serialize_keras_object"])
def serialize_keras_object(instance):
    """Legacy ``{"class_name", "config"}`` form of a Keras object."""
    if instance is None:
        return None
    if hasattr(instance, "get_config"):
        name = object_registration.get_registered_name(instance.__class__)
        config = instance.get_config()
        out = {}
        for key, item in config.items():
            if isinstance(item, str):
                out[key] = item
                continue
            try:
                serialized = serialize_keras_object(item)
                if isinstance(serialized, dict) and not isinstance(item, dict):
                    serialized["__passive_serialization__"] = True
                out[key] = serialized
            except ValueError:
                out[key] = item
        return {"class_name": name, "config": out}
    if hasattr(instance, "__name__"):
        return object_registration.get_registered_name(instance)
    raise ValueError(f"Cannot serialize {instance} because it doesn't implement `get_config()`.")


def serialize_nested(config):
    def one(obj):
        if callable(obj) or hasattr(obj, "get_config"):
            try:
                return serialize_keras_object(obj)
            except ValueError:
                return obj
        return obj

    return tree.map_structure(one, config)


def _lookup(class_name, module_objects, custom_objects, printable_module_name):
    custom_objects = custom_objects or {}
    if class_name in custom_objects:
        return custom_objects[class_name]
    obj = object_registration.get_registered_object(class_name, custom_objects, module_objects)
    if obj is not None:
        return obj
    from keras_b200.core import export_registry

    for prefix in ("keras.layers.", "keras.models.", "keras.", "keras.optimizers.", "keras.losses.", "keras.metrics.", "keras.initializers.",
                   "keras.regularizers.", "keras.constraints.", "keras.activations.", "keras.optimizers.schedules."):
        found = export_registry.get_symbol_from_name(prefix + class_name)
        if found is not None:
            return found
    raise ValueError(f"Unknown {printable_module_name}: '{class_name}'. Please ensure you are using a `keras.utils.custom_object_scope` and that this object is included in the scope.")


@keras_export(["keras.legacy.saving.deserialize_keras_object", "keras.utils.legacy.deserialize_keras_object"])
def deserialize_keras_object(identifier, module_objects=None, custom_objects=None, printable_module_name="object"):
    if identifier is None:
        return None
    if isinstance(identifier, dict):
        config = identifier
        if "class_name" not in config or "config" not in config:
            raise ValueError(f"Improper config format for {config}. Expecting python dict contains `class_name` and `config` as keys")
        if "module" in config and "registered_name" in config:
            return serialization_lib.deserialize_keras_object(config, custom_objects=custom_objects)
        cls = _lookup(config["class_name"], module_objects, custom_objects, printable_module_name)
        cls_config = config["config"]
        if isinstance(cls_config, list):
            return cls(cls_config) if not hasattr(cls, "from_config") else cls.from_config(cls_config)
        cls_config = dict(cls_config)
        for key, item in list(cls_config.items()):
            if isinstance(item, dict) and "__passive_serialization__" in item:
                cls_config[key] = deserialize_keras_object(item, module_objects=module_objects, custom_objects=custom_objects,
                                                           printable_module_name="config_item")
        if hasattr(cls, "from_config"):
            params = inspect.signature(cls.from_config).parameters
            with object_registration.CustomObjectScope(custom_objects or {}):
                if "custom_objects" in params:
                    return cls.from_config(cls_config, custom_objects=custom_objects or {})
                return cls.from_config(cls_config)
        with object_registration.CustomObjectScope(custom_objects or {}):
            return cls(**cls_config)
    if isinstance(identifier, str):
        return _lookup(identifier, module_objects, custom_objects, printable_module_name)
    if inspect.isfunction(identifier):
        return identifier
    raise ValueError(f"Could not interpret serialized {printable_module_name}: {identifier}")


def model_from_config(config, custom_objects=None):
    if isinstance(config, list):
        raise TypeError(f"`model_from_config` expects a dictionary, not a list. Received: config={config}. Did you meant to use `Sequential.from_config(config)`?")
    config = dict(config)
    inner = dict(config.get("config", {})) if isinstance(config.get("config"), dict) else config.get("config")
    if config.get("class_name") == "Sequential" and isinstance(inner, dict):
        # Keras 2 files carry `batch_input_shape` on the first layer instead of an InputLayer
        layers = [dict(l) for l in inner.get("layers", [])]
        if layers:
            first_cfg = dict(layers[0].get("config", {}))
            if layers[0].get("class_name") != "InputLayer" and ("batch_input_shape" in first_cfg or "batch_shape" in first_cfg):
                shape = first_cfg.pop("batch_input_shape", None) or first_cfg.pop("batch_shape", None)
                dtype = first_cfg.get("dtype", None)
                layers[0]["config"] = first_cfg
                layers.insert(0, {"class_name": "InputLayer", "config": {"batch_shape": list(shape), "dtype": dtype if isinstance(dtype, str) else None,
                                                                        "name": "input_layer_legacy"}})
        inner["layers"] = layers
        config["config"] = inner
    with object_registration.CustomObjectScope(custom_objects or {}):
        if "module" in config:
            return serialization_lib.deserialize_keras_object(config, custom_objects=custom_objects)
        return deserialize_keras_object(config, custom_objects=custom_objects, printable_module_name="layer")


def compile_args_from_training_config(training_config, custom_objects=None):
    from keras_b200 import losses, metrics, optimizers

    custom_objects = custom_objects or {}

    def nested(fn, cfg):
        if cfg is None:
            return None
        if isinstance(cfg, dict) and "class_name" in cfg:
            return fn(cfg)
        if isinstance(cfg, dict):
            return {k: nested(fn, v) for k, v in cfg.items()}
        if isinstance(cfg, (list, tuple)):
            return [nested(fn, v) for v in cfg]
        return fn(cfg) if isinstance(cfg, str) else cfg

    def metric(cfg):
        if cfg in ("accuracy", "acc", "crossentropy", "ce"):
            return cfg
        return metrics.deserialize(cfg)

    with object_registration.CustomObjectScope(custom_objects):
        optimizer = optimizers.deserialize(training_config["optimizer_config"])
        loss = nested(losses.deserialize, training_config.get("loss"))
        mets = nested(metric, training_config.get("metrics"))
        wmets = nested(metric, training_config.get("weighted_metrics"))
    return dict(optimizer=optimizer, loss=loss, metrics=mets, weighted_metrics=wmets, loss_weights=training_config.get("loss_weights"))


def deserialize_layer(layer_config, custom_objects=None):
    """A layer from a Keras 2 style ``{"class_name", "config"}`` entry of a model config."""
    layer_config = dict(layer_config)
    cfg = dict(layer_config.get("config", {}))
    if layer_config.get("class_name") != "InputLayer":
        cfg.pop("batch_input_shape", None)
    elif "batch_input_shape" in cfg:
        cfg["batch_shape"] = cfg.pop("batch_input_shape")
    if isinstance(cfg.get("dtype"), dict) and cfg["dtype"].get("class_name") == "Policy":
        cfg["dtype"] = cfg["dtype"].get("config", {}).get("name")
    layer_config["config"] = cfg
    return deserialize_keras_object(layer_config, custom_objects=custom_objects, printable_module_name="layer")
