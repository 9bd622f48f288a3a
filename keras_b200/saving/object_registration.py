"""Where user-defined serialisable objects are looked up by name
(behaviour of keras/src/saving/object_registration.py:18-230).

Three tiers answer a lookup, in this order: the innermost active ``CustomObjectScope`` (scopes nest; each entry sees the
union of the scopes around it), the process-wide registry filled by ``register_keras_serializable``, and the tables the
caller passes in (``custom_objects`` before ``module_objects``).  The registry is kept in both directions so that
``get_registered_name`` is a dictionary lookup as well.
"""

import inspect

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export

GLOBAL_CUSTOM_OBJECTS = {}  # "package>name" -> object
GLOBAL_CUSTOM_NAMES = {}    # object -> "package>name"

_SCOPE_KEY = "custom_objects_scope_dict"


def _active_scope():
    return global_state.get_global_attribute(_SCOPE_KEY, {})


@keras_export(["keras.saving.CustomObjectScope", "keras.saving.custom_object_scope", "keras.utils.CustomObjectScope", "keras.utils.custom_object_scope"])
class CustomObjectScope:
    """``with CustomObjectScope({"name": obj}): ...`` makes ``obj`` resolvable by ``name`` inside the block."""

    def __init__(self, custom_objects):
        self.custom_objects = custom_objects or {}
        self.backup = None

    def __enter__(self):
        outer = dict(_active_scope())
        self.backup = outer
        global_state.set_global_attribute(_SCOPE_KEY, {**outer, **self.custom_objects})
        return self

    def __exit__(self, *exc_info):
        global_state.set_global_attribute(_SCOPE_KEY, dict(self.backup))


custom_object_scope = CustomObjectScope


@keras_export(["keras.saving.get_custom_objects", "keras.utils.get_custom_objects"])
def get_custom_objects():
    """The process-wide registry itself (callers may edit it)."""
    return GLOBAL_CUSTOM_OBJECTS


@keras_export(["keras.saving.register_keras_serializable", "keras.utils.register_keras_serializable"])
def register_keras_serializable(package="Custom", name=None):
    """Decorator: file the class or function under ``"{package}>{name}"`` (``name`` defaults to its ``__name__``)."""

    def file_under_key(target):
        if inspect.isclass(target) and not hasattr(target, "get_config"):
            raise ValueError("Cannot register a class that does not have a get_config() method.")
        key = f"{package}>{target.__name__ if name is None else name}"
        GLOBAL_CUSTOM_OBJECTS[key] = target
        GLOBAL_CUSTOM_NAMES[target] = key
        return target

    return file_under_key


@keras_export(["keras.saving.get_registered_name", "keras.utils.get_registered_name"])
def get_registered_name(obj):
    """The registry key of ``obj``, or its plain ``__name__`` when it was never registered."""
    return GLOBAL_CUSTOM_NAMES.get(obj, None) or obj.__name__


@keras_export(["keras.saving.get_registered_object", "keras.utils.get_registered_object"])
def get_registered_object(name, custom_objects=None, module_objects=None):
    for table in (_active_scope(), GLOBAL_CUSTOM_OBJECTS, custom_objects, module_objects):
        if table and name in table:
            return table[name]
    return None
