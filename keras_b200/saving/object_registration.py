"""Registry of user-defined serializable objects (keras/src/saving/object_registration.py:18-230)."""

import inspect

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export

GLOBAL_CUSTOM_OBJECTS = {}
GLOBAL_CUSTOM_NAMES = {}


@keras_export(["keras.saving.CustomObjectScope", "keras.saving.custom_object_scope", "keras.utils.CustomObjectScope", "keras.utils.custom_object_scope"])
class CustomObjectScope:
    def __init__(self, custom_objects):
        self.custom_objects = custom_objects or {}
        self.backup = None

    def __enter__(self):
        self.backup = global_state.get_global_attribute("custom_objects_scope_dict", {}).copy()
        merged = dict(self.backup)
        merged.update(self.custom_objects)
        global_state.set_global_attribute("custom_objects_scope_dict", merged)
        return self

    def __exit__(self, *args, **kwargs):
        global_state.set_global_attribute("custom_objects_scope_dict", self.backup.copy())


custom_object_scope = CustomObjectScope


@keras_export(["keras.saving.get_custom_objects", "keras.utils.get_custom_objects"])
def get_custom_objects():
    return GLOBAL_CUSTOM_OBJECTS


@keras_export(["keras.saving.register_keras_serializable", "keras.utils.register_keras_serializable"])
def register_keras_serializable(package="Custom", name=None):
    def decorator(arg):
        class_name = name if name is not None else arg.__name__
        registered_name = package + ">" + class_name
        if inspect.isclass(arg) and not hasattr(arg, "get_config"):
            raise ValueError("Cannot register a class that does not have a get_config() method.")
        GLOBAL_CUSTOM_OBJECTS[registered_name] = arg
        GLOBAL_CUSTOM_NAMES[arg] = registered_name
        return arg

    return decorator


@keras_export(["keras.saving.get_registered_name", "keras.utils.get_registered_name"])
def get_registered_name(obj):
    if obj in GLOBAL_CUSTOM_NAMES:
        return GLOBAL_CUSTOM_NAMES[obj]
    return obj.__name__


@keras_export(["keras.saving.get_registered_object", "keras.utils.get_registered_object"])
def get_registered_object(name, custom_objects=None, module_objects=None):
    scope = global_state.get_global_attribute("custom_objects_scope_dict", {})
    if name in scope:
        return scope[name]
    if name in GLOBAL_CUSTOM_OBJECTS:
        return GLOBAL_CUSTOM_OBJECTS[name]
    if custom_objects and name in custom_objects:
        return custom_objects[name]
    if module_objects and name in module_objects:
        return module_objects[name]
    return None
